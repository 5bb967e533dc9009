"""Shared by the expert-parallel tests: a CPU stand-in for the GPU stages, built on the oracle, so that the exchange
logic of c0ven_b200.ep runs on gloo ranks without a GPU. Test infrastructure only."""
import numpy as np
import torch

from c0ven_b200 import ep
from oracle import oracle as O


class OracleStages:
    """The stages of c0ven_b200.ep.GpuStages on the CPU: a wire row is the f32 activation row itself."""

    def __init__(self, layer, rank, world):
        self.L, self.rank, self.world = layer, rank, world
        self.first, self.count = ep.owner_ranges(layer["n_experts"], world)[rank]
        self.K, self.E, self.F = layer["n_used"], layer["n_embd"], layer["n_ff"]
        self.wire = self.E * 4  # bytes of a row as it travels

    def route(self, x):
        self.x = x.numpy()
        L = self.L
        rl = O.router_logits(self.x, L["router"], L["shexp_gate_inp"], L.get("router_bias"))
        self.ids, self.w, self.gs = O.router_topk(rl, self.K)
        cnt, base, self.inv, _ = O.pack(self.ids, L["n_experts"])
        return torch.from_numpy(cnt.astype(np.int32))

    def gather(self):
        A = self.ids.size
        order = np.empty(A, dtype=np.int64)
        order[self.inv] = np.arange(A)
        rows = self.x[order // self.K]
        return torch.from_numpy(np.ascontiguousarray(rows).view(np.uint8).reshape(A, -1))

    def experts(self, rows, ids):
        L, R = self.L, rows.shape[0]
        x = rows.numpy().view(np.float32).reshape(R, self.E)
        ids = ids.numpy()
        assert np.all((ids >= self.first) & (ids < self.first + self.count))
        jobs = [(L["gate_exps"][e], L["up_exps"][e], L["down_exps"][e], r, 1.0) for r, e in enumerate(ids)]
        y = O.compute_many(L["gate_type"], L["down_type"], self.E, self.F, jobs, x) if R else np.zeros((0, self.E), np.float32)
        return torch.from_numpy(y)

    # One row per (token, GPU): the same four stages on the CPU. A travelling row is the f32 row, then K int32 expert
    # ids (-1: not on that GPU) and K f32 weights.
    partial_dtype = torch.float32   # what experts_partial returns here; the GPU stages send f16

    @property
    def dispatch_bytes(self):
        return self.E * 4 + self.K * 8

    @property
    def n_used(self):
        return self.K

    def plan(self):
        per = self.L["n_experts"] // self.world
        owner = self.ids // per                                   # [T][K]
        self.goes = np.stack([(owner == g).any(1) for g in range(self.world)], 1)   # [T][world]
        tot = np.zeros(16, dtype=np.int32)
        tot[:self.world] = self.goes.sum(0)
        tot[8:8 + self.world] = [(owner == g).sum() for g in range(self.world)]
        self.owner = owner
        return torch.from_numpy(tot)

    def dispatch(self, nrows):
        out = np.zeros((nrows, self.dispatch_bytes), dtype=np.uint8)
        r = 0
        self.sent_at = {}
        for g in range(self.world):
            for t in np.nonzero(self.goes[:, g])[0]:
                on = self.owner[t] == g
                out[r, :self.E * 4] = self.x[t].view(np.uint8)
                out[r, self.E * 4:self.E * 4 + self.K * 4] = np.where(on, self.ids[t], -1).astype(np.int32).view(np.uint8)
                out[r, self.E * 4 + self.K * 4:] = np.where(on, self.w[t], 0).astype(np.float32).view(np.uint8)
                self.sent_at[(int(t), g)] = r
                r += 1
        assert r == nrows
        return torch.from_numpy(out)

    def experts_partial(self, rows, assignments):
        L, R = self.L, rows.shape[0]
        b = rows.numpy()
        x = np.ascontiguousarray(b[:, :self.E * 4]).view(np.float32).reshape(R, self.E)
        ids = np.ascontiguousarray(b[:, self.E * 4:self.E * 4 + self.K * 4]).view(np.int32).reshape(R, self.K)
        w = np.ascontiguousarray(b[:, self.E * 4 + self.K * 4:]).view(np.float32).reshape(R, self.K)
        # Rows from a rank whose own stage failed are whatever its buffer held: as the GPU stage does, take what is a
        # valid list entry and ignore the rest, rather than fail here too.
        ids = np.where((ids >= self.first) & (ids < self.first + self.count), ids, -1)
        w = np.nan_to_num(w, nan=0.0, posinf=0.0, neginf=0.0)
        x = np.nan_to_num(x, nan=0.0, posinf=0.0, neginf=0.0)
        jobs = [(L["gate_exps"][e], L["up_exps"][e], L["down_exps"][e], r, float(w[r, k]))
                for r in range(R) for k, e in enumerate(ids[r]) if e >= 0]   # a row's jobs in rank order, as compute_many sums them
        y = O.compute_many(L["gate_type"], L["down_type"], self.E, self.F, jobs, x) if jobs else np.zeros((R, self.E), np.float32)
        return torch.from_numpy(y)

    def combine_partials(self, back, out):
        back = back.numpy()
        T = self.x.shape[0]
        o = np.zeros((T, self.E), dtype=np.float32)
        for g in range(self.world):                               # the GPUs' sums in GPU order
            for t in np.nonzero(self.goes[:, g])[0]:
                o[t] += back[self.sent_at[(int(t), g)]]
        o += self.gs[:, None] * self.s
        out.copy_(torch.from_numpy(o))

    def shared(self):
        L = self.L
        T = self.x.shape[0]
        jobs = [(L["gate_shexp"], L["up_shexp"], L["down_shexp"], t, 1.0) for t in range(T)]
        self.s = O.compute_many(L["shexp_gate_type"], L["shexp_down_type"], self.E, self.F, jobs, self.x)

    def combine(self, y, out):
        y = y.numpy()
        T = self.x.shape[0]
        o = np.zeros((T, self.E), dtype=np.float32)
        for k in range(self.K):  # rank order, as the oracle's compute_many sums a token's jobs
            o += self.w[:, k:k + 1] * y[self.inv.reshape(T, self.K)[:, k]]
        o += self.gs[:, None] * self.s
        out.copy_(torch.from_numpy(o))

    def empty(self, shape, dtype, name=None):
        return torch.empty(shape, dtype=dtype)

    def to_device(self, a):
        return torch.from_numpy(a)


def run_ranks(worker, world, args=(), timeout=180):
    """Runs worker(rank, world, port, queue, *args) as `world` daemon processes; returns what each put on the queue,
    sorted. The results are read before the processes are joined (a full pipe would block the child's exit), and a
    process still alive at the end, whatever the reason, is terminated and then killed, so that no rank is left inside a
    collective holding a device."""
    import socket

    import torch.multiprocessing as mp

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, port, q) + tuple(args), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    try:
        res = [q.get(timeout=timeout) for _ in range(world)]
        for p in procs:
            p.join(timeout=30)
        return sorted(res, key=lambda r: r[0])
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=5)
            if p.is_alive():
                p.kill()
