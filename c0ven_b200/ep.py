"""Expert parallel over the GPUs of one node: one process per GPU, each holding a contiguous range of the experts, the
router and the shared expert replicated, the rows sharded. A step routes its own rows, sends each assignment's
quantised activation row to the GPU that owns its expert (all-to-all), runs its experts on the rows it received, sends
the results back (all-to-all) and combines them with its own shared expert. The reference has no expert parallelism
(both its cards hold the same experts: docs/DESIGN.md:294-297); its two cards exchange partial sums instead
(core/models/qwen4exp/model.cpp:1404-1418).

Two forms of the exchange. Per assignment (ExpertParallelMoE with by_token=False): a token's row travels once for each
of its experts and every result comes back as a row; the outputs are then one GPU's bit for bit. Per token and GPU
(by_token=True, the default): a token's row travels once to each GPU that holds any of its experts, with the list of
those experts and their weights, and each GPU returns one row, the weighted sum of its experts' results for the token;
at 2, 4 and 8 GPUs that is about 0.2, 0.38 and 0.59 of the per-assignment bytes each way, and the outputs agree with
one GPU's within the layer's tolerance (the sum over a token's experts is taken GPU by GPU).

Ownership: GPU g holds experts [g * per, (g + 1) * per) of the layer it was given. With interleave=True the layer is
renumbered first so that those are the experts e with e % world == g of the caller's numbering: neighbouring experts
then sit on different GPUs, which spreads a routing skew that follows the numbering; ties between exactly equal
logits then break by the new numbering.

The collectives are torch.distributed's (NCCL over NVLink on GPUs): per step one all-gather of the ranks' per-expert row
counts (from which every rank knows what it sends, what it receives and which expert each received row is for, so no
ids travel), one all-to-all of rows out and one of results back; one wait on the host, for the split sizes. The
stages between them are the C ABI's moe_layer_*_device calls, behind a small backend object so that the exchange logic
also runs on CPU ranks (gloo) in the tests, with a CPU stand-in for the stages.
"""
from __future__ import annotations

import os

import numpy as np
import torch
import torch.distributed as dist


def owner_ranges(n_experts: int, world: int):
    """Experts [first, first + count) of every rank: equal contiguous ranges."""
    if n_experts % world:
        raise ValueError("the experts must divide evenly over the ranks")
    per = n_experts // world
    return [(r * per, per) for r in range(world)]


def split_sizes(cnt_all: np.ndarray, rank: int):
    """From every rank's rows per expert, cnt_all [world][n_experts]: the rows this rank sends to each rank and receives
    from each rank."""
    world, ne = cnt_all.shape
    per = ne // world
    by_owner = cnt_all.reshape(world, world, per).sum(-1)  # [source][owner]
    return [int(v) for v in by_owner[rank]], [int(v) for v in by_owner[:, rank]]


def interleaved_order(n_experts: int, world: int) -> np.ndarray:
    """The renumbering (new index -> caller's index) under which equal contiguous ranges of the new numbering are the
    residue classes of the old: new expert g * per + j is the caller's expert j * world + g."""
    return np.arange(n_experts).reshape(n_experts // world, world).T.reshape(-1)


def balanced_order(counts, world: int) -> np.ndarray:
    """A renumbering (new index -> caller's index) that spreads the load the counts show: counts[e] = rows expert e got
    over some steps (moe_layer_read_counts, summed by the caller). Experts are dealt, heaviest first, each to the GPU
    with the least load so far that still has room (every GPU holds the same number of experts); inside a GPU they keep
    the caller's order. The reference answers routing skew by swapping which experts its cards cache
    (core/models/qwen4exp/swap.cpp); with every expert resident somewhere, the analogue is where."""
    counts = np.asarray(counts, dtype=np.int64)
    ne = counts.size
    per = ne // world
    load, room = np.zeros(world, dtype=np.int64), np.full(world, per)
    owner = np.empty(ne, dtype=np.int64)
    for e in np.argsort(-counts, kind="stable"):
        open_ = np.nonzero(room > 0)[0]
        g = open_[np.argmin(load[open_])]
        owner[e], load[g], room[g] = g, load[g] + counts[e], room[g] - 1
    return np.concatenate([np.nonzero(owner == g)[0] for g in range(world)])


def reordered(layer: dict, order) -> dict:
    """The layer with its experts renumbered by order (new index -> caller's index). Copies the experts: for tests and
    CPU stand-ins; GpuStages takes only its own rank's."""
    order = np.asarray(order)
    out = dict(layer)
    out["router"] = np.ascontiguousarray(layer["router"][order])
    if layer.get("router_bias") is not None:
        out["router_bias"] = np.ascontiguousarray(layer["router_bias"][order])
    for k in ("gate_exps", "up_exps", "down_exps"):
        out[k] = layer[k][order]
    return out


def interleaved(layer: dict, world: int) -> dict:
    return reordered(layer, interleaved_order(layer["n_experts"], world))


def received_ids(cnt_all: np.ndarray, rank: int) -> np.ndarray:
    """The expert of every row this rank receives: source by source, each source's rows in expert order."""
    world, ne = cnt_all.shape
    per = ne // world
    mine = cnt_all[:, rank * per:(rank + 1) * per].astype(np.int64)  # [source][local expert]
    return np.repeat(np.tile(np.arange(rank * per, (rank + 1) * per, dtype=np.int32), world), mine.reshape(-1))


class GpuStages:
    """The stages on a GPU, through the C ABI."""

    def __init__(self, layer: dict, rank: int, world: int, max_tokens: int, device: int, max_expert_rows: int = 0,
                 y_f16: bool = True, profile: bool = False, tensor_min_rows: int = 0, stream_ptr: int | None = None,
                 interleave: bool = False, order=None):
        """order: a renumbering of the experts (new index -> the caller's index, e.g. balanced_order's); rank g then holds
        the caller's experts order[g * per : (g + 1) * per]. interleave: interleaved_order."""
        from .layer import MoELayer

        first, count = owner_ranges(layer["n_experts"], world)[rank]
        own = None
        if interleave and order is None:
            order = interleaved_order(layer["n_experts"], world)
        if order is not None:
            # The router renumbered; of the experts only this rank's are touched.
            order = np.asarray(order)
            if sorted(order.tolist()) != list(range(layer["n_experts"])):
                raise ValueError("order must be a permutation of the experts")
            mine = order[first:first + count]
            own = (layer["gate_exps"][mine], layer["up_exps"][mine], layer["down_exps"][mine])
            layer = dict(layer, router=np.ascontiguousarray(layer["router"][order]),
                         router_bias=None if layer.get("router_bias") is None else np.ascontiguousarray(layer["router_bias"][order]))
        self.device = torch.device("cuda", device)
        self.y_dtype = torch.float16 if y_f16 else torch.float32
        self.n_embd, self.n_used, self.n_experts = layer["n_embd"], layer["n_used"], layer["n_experts"]
        self.moe = MoELayer(layer, max_tokens=max_tokens, device=device, expert_first=first, expert_count=count,
                            max_expert_rows=max_expert_rows or max_tokens * layer["n_used"] * world, profile=profile,
                            tensor_min_rows=tensor_min_rows, own_experts=own)
        # The stream every stage is queued on: the layer's own, or the caller's (several layers of a stack share one).
        self._sp = stream_ptr
        self.stream = torch.cuda.ExternalStream(stream_ptr or self.moe.stream, device=self.device)
        self.wire = self.moe.wire_row_bytes
        self.dispatch_bytes = self.moe.dispatch_row_bytes
        self.max_expert_rows = max_expert_rows or max_tokens * layer["n_used"] * world
        self._bufs = {}
        # The shared expert needs no other GPU: it runs on a stream of its own beside the exchanges and the experts.
        self.side = torch.cuda.Stream(device=self.device)
        self.shared_beside = not profile and os.environ.get("C0VEN_EP_SHARED_INLINE") != "1"

    def route(self, x: torch.Tensor) -> torch.Tensor:
        """Routes and packs x's rows; returns the rows per expert, an int32 tensor [n_experts] on the device."""
        self.T = x.shape[0]
        self.moe.route_device(x.data_ptr(), self.T, self._sp)
        cnt = self.empty((self.n_experts,), torch.int32, "cnt")
        self.moe.counts_device(cnt.data_ptr(), self._sp)
        return cnt

    def gather(self) -> torch.Tensor:
        rows = self.empty((self.T * self.n_used, self.wire), torch.uint8, "rows")
        ids = self.empty((self.T * self.n_used,), torch.int32, "ids")
        self.moe.gather_rows_device(rows.data_ptr(), ids.data_ptr(), self._sp)
        return rows

    def experts(self, rows: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
        R = rows.shape[0]
        y = self.empty((R, self.n_embd), self.y_dtype, "y_in")
        if R:
            self.moe.experts_device(rows.data_ptr(), ids.data_ptr(), R, y.data_ptr(), self.y_dtype == torch.float16, self._sp)
        return y

    # One row per (token, GPU).
    def plan(self) -> torch.Tensor:
        """After route: the rows this rank sends to GPUs 0 .. 7, then the assignments in them: int32 [16] on the device."""
        tot = self.empty((16,), torch.int32, "totals")
        self.moe.dispatch_plan_device(tot.data_ptr(), self._sp)
        return tot

    def dispatch(self, nrows: int) -> torch.Tensor:
        rows = self.empty((nrows, self.moe.dispatch_row_bytes), torch.uint8, "drows")
        self.moe.dispatch_rows_device(rows.data_ptr(), self._sp)
        return rows

    def experts_partial(self, rows: torch.Tensor, assignments: int) -> torch.Tensor:
        R = rows.shape[0]
        y = self.empty((R, self.n_embd), torch.float16, "y_part")
        if R:
            self.moe.experts_partial_device(rows.data_ptr(), R, assignments, y.data_ptr(), self._sp)
        return y

    def combine_partials(self, back: torch.Tensor, out: torch.Tensor):
        self.moe.combine_partials_device(back.data_ptr(), out.data_ptr(), self._sp)

    def shared(self):
        self.moe.shared_device(self._sp)

    def shared_start(self):
        """The shared expert on the side stream, after what the main stream holds so far (the routing)."""
        if not self.shared_beside:
            return
        self.side.wait_stream(self.stream)
        self.moe.shared_device(self.side.cuda_stream)

    def shared_finish(self):
        """The main stream waits for the shared expert; without the side stream, runs it in line."""
        if self.shared_beside:
            self.stream.wait_stream(self.side)
        else:
            self.shared()

    def ids_from_counts(self, cnt_all: torch.Tensor, world: int, R: int) -> torch.Tensor:
        """The expert of every received row, computed on the device from the gathered counts."""
        ids = self.empty((max(R, 1),), torch.int32, "ids_in")
        self.moe.received_ids_device(cnt_all.data_ptr(), world, ids.data_ptr(), self._sp)
        return ids[:R]

    def combine(self, y: torch.Tensor, out: torch.Tensor):
        self.moe.combine_device(y.data_ptr(), y.dtype == torch.float16, out.data_ptr(), self._sp)

    def empty(self, shape, dtype, name=None):
        """A device tensor; with a name, a view of a buffer kept and grown between steps."""
        if name is None:
            return torch.empty(shape, dtype=dtype, device=self.device)
        n = int(np.prod(shape)) if len(shape) else 1
        buf = self._bufs.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < n:
            buf = torch.empty(max(n, 1) + max(n, 1) // 4, dtype=dtype, device=self.device)
            self._bufs[name] = buf
        return buf[:n].view(shape)

    def to_device(self, a: np.ndarray) -> torch.Tensor:
        return torch.from_numpy(a).to(self.device, non_blocking=True)

    def sync(self):
        self.moe.sync()

    def close(self):
        self._bufs.clear()
        self.moe.close()


class ExpertParallelMoE:
    """One MoE layer over the process group's ranks. forward() takes this rank's rows and returns their outputs."""

    def __init__(self, stages, group=None, by_token: bool = True):
        self.st, self.group, self.by_token = stages, group, by_token and hasattr(stages, "plan")
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.sent_rows = self.received_rows = self.expert_rows = 0  # of the last step: rows sent to and received from other ranks; rows its experts ran
        # With time_phases set, forward_by_token brackets its phases with CUDA events on the stages' stream and leaves
        # their device times in phase_ms after a wait for the step's end (a measuring aid: the wait costs the step).
        self.time_phases, self.phase_ms = False, {}

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """A stage that fails on one rank (a bad argument, a timeout, a launch error) must not leave the others waiting
        in a collective: what can be known on every rank (a rank receiving more rows than it has room for) is checked
        on every rank from the gathered counts, before any row moves; any other failure is held until the step's
        collectives have all been entered with the sizes agreed, and raised then."""
        if self.by_token:
            return self.forward_by_token(x, out)
        st, W = self.st, self.world
        held = None
        with torch.cuda.stream(st.stream) if hasattr(st, "stream") else _null():
            cnt = st.route(x)
            if hasattr(st, "shared_start"):
                st.shared_start()
            cnt_all = st.empty((W * cnt.numel(),), cnt.dtype, "cnt_all")
            dist.all_gather_into_tensor(cnt_all, cnt, group=self.group)
            counts = cnt_all.cpu().numpy().reshape(W, -1)      # the step's one wait on the host
            send, recv = split_sizes(counts, self.rank)
            most = getattr(st, "max_expert_rows", 0)
            if most:
                per = counts.shape[1] // W
                by_owner = counts.reshape(W, W, per).sum(-1).sum(0)  # rows every rank receives: the same sum on every rank
                if int(by_owner.max()) > most:
                    raise RuntimeError(f"rank {int(by_owner.argmax())} would receive {int(by_owner.max())} rows, more than max_expert_rows "
                                       f"{most}: every rank stops here, before the exchange")
            R = sum(recv)
            try:
                rows = st.gather()                             # [A][wire] in expert order = destination order
            except Exception as e:  # noqa: BLE001
                held, rows = e, st.empty((sum(send), st.wire), torch.uint8, "rows")
            rows_in = st.empty((R, rows.shape[1]), rows.dtype, "rows_in")
            dist.all_to_all_single(rows_in, rows, recv, send, group=self.group)
            y_in = None
            if held is None:
                try:
                    if hasattr(st, "ids_from_counts"):
                        ids_in = st.ids_from_counts(cnt_all, W, R)
                    else:
                        ids_in = st.to_device(received_ids(counts, self.rank))
                    y_in = st.experts(rows_in, ids_in)         # [R][E] in arrival order
                except Exception as e:  # noqa: BLE001
                    held = e
            if y_in is None:
                y_in = st.empty((R, x.shape[1]), getattr(st, "y_dtype", torch.float32), "y_in")
            y = st.empty((rows.shape[0], y_in.shape[1]), y_in.dtype, "y")
            dist.all_to_all_single(y, y_in, send, recv, group=self.group)
            if held is not None:
                raise held
            if hasattr(st, "shared_finish"):
                st.shared_finish()
            else:
                st.shared()
            if out is None:
                out = st.empty(tuple(x.shape), torch.float32)
            st.combine(y, out)
        self.sent_rows, self.received_rows, self.expert_rows = sum(send) - send[self.rank], R - recv[self.rank], R
        return out

    def forward_host(self, x_host: torch.Tensor, out_host: torch.Tensor, chunks: int = 4) -> torch.Tensor:
        """From page-locked host rows to page-locked host rows, the step cut into `chunks` steps of about equal rows
        (the same number on every rank, none with more chunks than rows: each is a step of the whole group) so that a chunk's copy in and the copy out
        of the one before run beside a chunk's computation and exchanges, each on a stream of its own. What
        sent_rows, received_rows and expert_rows say afterwards is the sum over the chunks."""
        st = self.st
        T = x_host.shape[0]
        if chunks < 1 or chunks > T:
            raise ValueError("every rank needs at least one row in each of the chunks (the ranks take them in step)")
        if not hasattr(self, "_copy_in"):
            self._copy_in, self._copy_out = torch.cuda.Stream(device=st.device), torch.cuda.Stream(device=st.device)
        x_dev = st.empty(tuple(x_host.shape), x_host.dtype, "host_x")
        o_dev = st.empty(tuple(x_host.shape), torch.float32, "host_out")
        bounds = [(T * c // chunks, T * (c + 1) // chunks) for c in range(chunks)]
        self._copy_in.wait_stream(st.stream)       # the buffers' last readers and writers, a call ago
        self._copy_out.wait_stream(st.stream)
        arrived = []
        with torch.cuda.stream(self._copy_in):
            for a, b in bounds:
                x_dev[a:b].copy_(x_host[a:b], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._copy_in)
                arrived.append(ev)
        totals = [0, 0, 0]
        for (a, b), ev in zip(bounds, arrived):
            st.stream.wait_event(ev)
            self.forward(x_dev[a:b], o_dev[a:b])
            done = torch.cuda.Event()
            done.record(st.stream)
            self._copy_out.wait_event(done)
            with torch.cuda.stream(self._copy_out):
                out_host[a:b].copy_(o_dev[a:b], non_blocking=True)
            totals = [t + v for t, v in zip(totals, (self.sent_rows, self.received_rows, self.expert_rows))]
        self._copy_out.synchronize()
        self.sent_rows, self.received_rows, self.expert_rows = totals
        return out_host

    def forward_by_token(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """One row per (token, GPU) out, one weighted partial sum per (token, GPU) back. Failures are handled as in
        forward(): what every rank can know is checked on every rank before a row moves; a stage's own failure is held until
        the step's collectives have been entered. The step is the five phases below one after another."""
        s = self.by_token_begin(x, out)
        self.by_token_counts(s)
        self.by_token_rows_out(s)
        self.by_token_experts(s)
        return self.by_token_finish(s)

    def _on_stream(self):
        return torch.cuda.stream(self.st.stream) if hasattr(self.st, "stream") else _null()

    def _mark(self, s, name):
        if self.time_phases and hasattr(self.st, "stream"):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(self.st.stream)
            s["marks"].append((name, ev))

    def by_token_begin(self, x, out=None) -> dict:
        """Route, start the shared expert, plan the dispatch, gather every rank's totals (on the device: nothing waits yet)."""
        st, W = self.st, self.world
        s = dict(x=x, out=out, held=None, marks=[])
        with self._on_stream():
            self._mark(s, "route")
            st.route(x)
            if hasattr(st, "shared_start"):
                st.shared_start()
            self._mark(s, "plan")
            tot = st.plan()                                          # [16]: rows to each GPU, then assignments to each
            s["tot_all"] = st.empty((W * 16,), tot.dtype, "tot_all")
            dist.all_gather_into_tensor(s["tot_all"], tot, group=self.group)
        return s

    def by_token_counts(self, s: dict) -> None:
        """The step's one wait on the host: the split sizes; what every rank can refuse is refused here, on every rank."""
        st, W = self.st, self.world
        with self._on_stream():
            m = s["tot_all"].cpu().numpy().reshape(W, 2, 8)
        s["send"], s["recv"] = [int(v) for v in m[self.rank, 0, :W]], [int(v) for v in m[:, 0, self.rank]]
        s["asg_in"] = int(m[:, 1, self.rank].sum())
        most = getattr(st, "max_expert_rows", 0)
        if most:
            entries = m[:, 0, :W].sum(0) * st.n_used                 # what every rank would receive, the same on every rank
            if int(entries.max()) > most:
                raise RuntimeError(f"rank {int(entries.argmax())} would receive {int(entries.max())} row entries, more than "
                                   f"max_expert_rows {most}: every rank stops here, before the exchange")

    def by_token_rows_out(self, s: dict) -> None:
        st = self.st
        send, recv = s["send"], s["recv"]
        with self._on_stream():
            self._mark(s, "dispatch")
            try:
                rows = st.dispatch(sum(send))
            except Exception as e:  # noqa: BLE001
                s["held"], rows = e, st.empty((sum(send), st.dispatch_bytes), torch.uint8, "drows")
            s["rows_in"] = st.empty((sum(recv), rows.shape[1]), rows.dtype, "drows_in")
            self._mark(s, "rows out")
            dist.all_to_all_single(s["rows_in"], rows, recv, send, group=self.group)

    def by_token_experts(self, s: dict) -> None:
        st = self.st
        send, recv, R = s["send"], s["recv"], sum(s["recv"])
        with self._on_stream():
            self._mark(s, "experts")
            y_in = None
            if s["held"] is None:
                try:
                    y_in = st.experts_partial(s["rows_in"], s["asg_in"])   # [R][E] f16, in arrival order
                except Exception as e:  # noqa: BLE001
                    s["held"] = e
            if y_in is None:
                y_in = st.empty((R, s["x"].shape[1]), getattr(st, "partial_dtype", torch.float16), "y_part")   # the type every rank sends
            s["back"] = st.empty((sum(send), y_in.shape[1]), y_in.dtype, "y_back")
            self._mark(s, "sums back")
            dist.all_to_all_single(s["back"], y_in, send, recv, group=self.group)

    def by_token_finish(self, s: dict) -> torch.Tensor:
        st = self.st
        if s["held"] is not None:
            raise s["held"]
        with self._on_stream():
            self._mark(s, "combine")
            if hasattr(st, "shared_finish"):
                st.shared_finish()
            else:
                st.shared()
            out = s["out"]
            if out is None:
                out = st.empty(tuple(s["x"].shape), torch.float32)
            st.combine_partials(s["back"], out)
            self._mark(s, "end")
        marks = s["marks"]
        if marks:
            marks[-1][1].synchronize()
            self.phase_ms = {a[0]: a[1].elapsed_time(b[1]) for a, b in zip(marks, marks[1:])}
        send, recv = s["send"], s["recv"]
        self.sent_rows, self.received_rows, self.expert_rows = sum(send) - send[self.rank], sum(recv) - recv[self.rank], s["asg_in"]
        return out


class _null:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False
