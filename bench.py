"""MoE-layer throughput on B200: one step is one pass of the layer over one packed ragged batch.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

Prints one JSON line. `value` is tokens/s with the batch resident in HBM; `e2e` the same through the host-buffer C ABI
call (moe_layer_forward), copies included; `roofline` the dominant kernel against the measured peak; `cpu_baseline`
the CPU oracle on the box's host cores (a port of the reference's CPU expert path: the reference itself needs ggml,
which is absent). `--impl reference` times that CPU path alone.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from c0ven_b200 import synth  # noqa: E402

METRIC = "moe_layer_tokens_per_s"
UNIT = "tokens/s"
E, F, NE, K = 2048, 512, 512, 10


def measured_peaks():
    """The box's measured peaks when the driver left them beside this file, else the pool's earlier measurement."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], bf16_tflops_sustained=d.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


def workload(name: str) -> dict:
    w = dict(synth.CONFIGS[name])
    w["name"] = name
    return w


def build_layer(w: dict, seed: int = 0) -> dict:
    return synth.make_layer(E, F, NE, K, gate_type=w["gate_type"], down_type=w.get("down_type"),
                            shexp_gate_type=w.get("shexp_gate_type"), shexp_down_type=w.get("shexp_down_type"),
                            zipf_s=w.get("zipf_s", 0.0), seed=seed)


class ClockSampler:
    """nvidia-smi's SM clock and throttle reasons, sampled while the timed region runs."""
    Q = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, devices):
        """devices: the GPU indices to watch, or None to watch nothing (with several ranks only rank 0 samples, every
        rank's GPU in one nvidia-smi process: a poller per rank slows the ranks' own driver calls)."""
        self.devices, self.lines, self.proc = devices, [], None

    def __enter__(self):
        if not self.devices:
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100" if len(self.devices) == 1 else "250",
                                          "-i", ",".join(str(d) for d in self.devices)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def window(self, t0: float, t1: float):
        """The timed region, as time.time() values: summary() keeps the samples taken inside it (the poller starts
        before the warm-up, so that its own start-up, which takes the driver's locks, is not in the timed steps)."""
        self.t0, self.t1 = t0, t1

    def summary(self) -> dict:
        import datetime

        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 10:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
            except ValueError:
                ts = None
            rows.append((ts, f[1:]))
        t0, t1 = getattr(self, "t0", None), getattr(self, "t1", None)
        inside = [f for ts, f in rows if ts is not None and t0 is not None and t0 - 0.3 <= ts <= t1 + 0.3]
        for f in inside or [f for _, f in rows]:
            try:
                sm.append(float(f[1])), mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


_STAGES = ("quantize", "router", "pack", "gate_up", "down", "shared", "combine", "copies")

# DRAM bytes per launch of the dominant kernel from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum), by
# (workload, rows, stage), per launch (one layer); the summaries under profiles/ say which capture. None: not captured.
TRAFFIC = {("prefill32768_q4_k", 32768, "gate_up"): 2747.6e6, ("prefill32768_q4_k", 32768, "down"): 1932.4e6,
           ("ragged3521_q4_k_zipf", 3521, "gate_up"): 417.9e6, ("ragged3521_q4_k_zipf", 3521, "down"): 258.9e6,
           ("decode1_q8_0", 32, "gate_up"): 554.2e6, ("decode1_q8_0", 32, "down"): 280.5e6, ("stack48_verify32_iq3_s", 32, "gate_up"): 220.6e6}


def host_chunk_for(T: int) -> int:
    """Rows a chunk of a host-buffer call takes (the layer's host_chunk_rows; 0: the call whole). Long batches go in
    chunks of 8,192 rows; batches of a few thousand in two halves (3,521 rows: 1.71 -> 1.56 ms end to end; in three or
    four parts 1.79 and 1.85); shorter ones whole."""
    return 8192 if T >= 16384 else T // 2 if T >= 2048 else 0


def traffic_for(name: str, T: int, stage: str):
    """The captured DRAM bytes per launch of a workload's dominant kernel, or None when there is no capture."""
    return TRAFFIC.get((name, T, stage))


def algorithmic(w: dict, T: int, experts_hit: int, world: int = 1) -> dict:
    """Bytes and flops one GPU's part of the layer needs for its T rows, with `experts_hit` distinct experts hit there.
    Expert parallel, the rows a GPU's experts compute are taken as its share, T * K, of all the rows."""
    gt, dt = w["gate_type"], w.get("down_type") or w["gate_type"]
    sgt, sdt = w.get("shexp_gate_type") or gt, w.get("shexp_down_type") or dt
    routed, shared = synth.expert_bytes(gt, dt, E, F), synth.expert_bytes(sgt, sdt, E, F)
    A = T * K
    return dict(bytes_layer=(NE + 1) * E * 4 + experts_hit * routed + shared + 2 * T * E * 4,
                bytes_gate_up=experts_hit * 2 * F * synth.row_bytes(gt, E), bytes_down=experts_hit * E * synth.row_bytes(dt, F),
                flops_gate_up=2.0 * A * 2 * F * E, flops_down=2.0 * A * E * F,
                flops_layer=2.0 * T * (K * 3 * E * F + 3 * E * F + E * (NE + 1)))


def cpu_step(layer, x, threads):
    from oracle import oracle

    t0 = time.perf_counter()
    oracle.moe_forward(layer, x, nthreads=threads, want_pack=True)
    return time.perf_counter() - t0


def static_config(w: dict, args, world: int) -> dict:
    """What names the workload, the same in both arms: nothing measured goes here."""
    T_total, scaling = args.tokens or w["tokens"], w.get("scaling", "weak")
    T = T_total if world == 1 or scaling == "weak" else max(1, T_total // world)
    return dict(workload=w["name"], rows=world * T, rows_per_gpu=T, layers=args.layers or w.get("layers", 1), runs=w.get("runs"),
                hidden=E, ffn=F, experts=NE, top_k=K, weights=synth.TYPE_NAMES[w["gate_type"]],
                down_weights=synth.TYPE_NAMES[w.get("down_type") or w["gate_type"]], zipf_s=w.get("zipf_s", 0.0),
                l2="flushed between timed steps")


CPU_PASSES = 5  # passes the CPU path is timed over, after one warm pass, in both CPU legs; the median is reported


def cpu_leg(layer, x_full, Tc):
    """The CPU expert path (the oracle port) on the first Tc rows, every core the process may run on."""
    from oracle import oracle

    threads = oracle.host_threads()
    x = np.ascontiguousarray(x_full[:Tc])
    cpu_step(layer, x, threads)
    dt = statistics.median([cpu_step(layer, x, threads) for _ in range(CPU_PASSES)])
    return dict(value=Tc / dt, unit=UNIT, cores=threads, kind="port",
                sample=f"first {Tc} of {x_full.shape[0]} rows a pass, median of {CPU_PASSES} passes after one warm pass"), dt


def run_reference(args, w):
    """The CPU expert path on the host's cores: the oracle port, every core the process may run on."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    T_full = args.tokens or w["tokens"]
    T = min(T_full, args.cpu_tokens)
    layer, x = build_layer(w), synth.make_input(T_full, E, seed=1)
    cpu, dt = cpu_leg(layer, x, T)
    v = cpu["value"]
    print(json.dumps(dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                          ms_per_step=dt * 1e3, higher_is_better=True, scaling=w.get("scaling", "weak"), vs_baseline=None, dtype="i8",
                          data="synthetic", impl="reference",
                          config=static_config(w, args, int(os.environ.get("WORLD_SIZE", "1"))),
                          cpu_baseline=cpu,
                          e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))))


MIN_TIMED_S = 0.5     # device time a reported figure is taken over, at least
MAX_TIMED_STEPS = 2000


def measure(args, w, steps, world, rank, local, dist, cpu=True):
    """One workload on this process's GPU (and, with world > 1, its peers): the JSON line's fields, on rank 0."""
    import torch

    from c0ven_b200 import MoELayer, ep

    T_total, nlayers = args.tokens or w["tokens"], args.layers or w.get("layers", 1)
    scaling = w.get("scaling", "weak")
    # Weak scaling: every rank brings the workload's rows. Strong: the workload's rows are shared out.
    T = T_total if world == 1 or scaling == "weak" else max(1, T_total // world)
    base = build_layer(w)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2
    x_np = synth.make_input(T, E, seed=1 + rank)
    x_host = torch.from_numpy(x_np).pin_memory()  # a page-locked copy
    out_host = torch.empty_like(x_host).pin_memory()

    # The layers of a stack share their experts' bytes on the host (each layer still has its own copy in HBM, so the
    # traffic is a stack's) and differ in their routers.
    layers, moes, stages, main_sp = [], [], [], None
    for i in range(nlayers):
        lw = base if i == 0 else dict(base, router=(np.random.default_rng(100 + i).standard_normal((NE, E)) * 0.02).astype(np.float32))
        if world == 1:
            m = MoELayer(lw, max_tokens=T, device=local, profile=False, tensor_min_rows=args.tensor_min,
                         host_chunk_rows=args.host_chunk if args.host_chunk >= 0 else host_chunk_for(T),
                         gather_in_kernel=args.gather_in_kernel)
            layers.append(m), moes.append(None)
            main_sp = main_sp or m.stream
        else:
            # Expert parallel: the experts dealt to the GPUs by the load one step of this batch shows (a layer with a
            # routing bias), else interleaved; one row per (token, GPU) on the wire unless --per-assignment.
            order = ep.interleaved_order(NE, world)
            if w.get("zipf_s", 0.0) > 0 and not args.contiguous:
                probe = ep.GpuStages(lw, rank, world, max_tokens=T, device=local, order=order)
                ep.ExpertParallelMoE(probe, by_token=not args.per_assignment).forward(x_host.cuda())
                probe.sync()
                cnt = torch.from_numpy(probe.moe.read_counts().astype(np.int64)).cuda()
                dist.all_reduce(cnt)
                seen = np.zeros(NE, dtype=np.int64)
                seen[order] = cnt.cpu().numpy()          # the probe counted in its own numbering
                probe.close()
                order = ep.balanced_order(seen, world)
            st = ep.GpuStages(lw, rank, world, max_tokens=T, device=local, y_f16=True, profile=False,
                              tensor_min_rows=args.tensor_min, stream_ptr=main_sp, order=None if args.contiguous else order)
            stages.append(st), layers.append(st.moe), moes.append(ep.ExpertParallelMoE(st, by_token=not args.per_assignment))
            main_sp = main_sp or st.moe.stream
    stream = torch.cuda.ExternalStream(main_sp, device=local)
    x_dev, out_dev = x_host.cuda(), torch.empty((T, E), device="cuda")
    res, xn = (torch.empty_like(x_dev), torch.empty_like(x_dev)) if nlayers > 1 else (None, None)

    def run_layer(i, xin, xout):
        if world == 1:
            layers[i].forward_device(xin.data_ptr(), T, xout.data_ptr(), main_sp)
        else:
            moes[i].forward(xin, xout)

    from c0ven_b200.layer import rmsnorm_rows_device

    def step():
        """One pass over the batch; queued on the main stream. A stack is x <- x + moe_l(rmsnorm(x)) for every layer:
        attention replaced by the identity, the norm there only to keep 48 random layers' values bounded."""
        with torch.cuda.stream(stream):
            if nlayers == 1:
                run_layer(0, x_dev, out_dev)
                return
            res.copy_(x_dev)
            for i in range(nlayers):
                rmsnorm_rows_device(res.data_ptr(), None, T, E, 1e-6, xn.data_ptr(), main_sp)  # the library's own norm kernel
                if world == 1:   # the residual is added by the layer's combine: no kernel between the layers but the norm
                    layers[i].forward_residual_device(xn.data_ptr(), T, res.data_ptr(), res.data_ptr(), main_sp)
                else:
                    run_layer(i, xn, out_dev)
                    res.add_(out_dev)

    def step_host():
        """The same from pinned host rows to pinned host rows."""
        if world == 1 and nlayers == 1:
            layers[0].forward(x_host.numpy(), out_host.numpy())  # the C ABI's host-buffer call
            return
        if world > 1 and nlayers == 1:
            moes[0].forward_host(x_host, out_host, chunks=4 if T >= 8192 else 1)  # the expert-parallel layer's host-buffer call
            return
        with torch.cuda.stream(stream):
            x_dev.copy_(x_host, non_blocking=True)
        step()
        with torch.cuda.stream(stream):
            out_host.copy_(res if nlayers > 1 else out_dev, non_blocking=True)
        stream.synchronize()

    def sync():
        stream.synchronize()

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def kernels():
        return sum(m.stats()["kernels"] for m in layers)

    def agree(v, op):
        """A number every rank then holds: the ranks' maximum (or whatever op says)."""
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        if dist:
            dist.all_reduce(t, op=op)
        return float(t.item())

    def timed_step(i):
        flush.fill_(i & 0xFF)  # L2 flush between timed iterations, outside the timed interval
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(stream)
        step()
        e.record(stream)
        sync()
        return s.elapsed_time(e)

    # Timed steps run as a caller would run them: no per-stage timing, the shared expert beside the routed ones, small
    # steps replayed from their recorded graph. The stages are timed afterwards, in a few more steps with the timing on.
    # The `steps` steps asked for are timed first; if they hold less than MIN_TIMED_S of device time, more follow until
    # they do, so that the figure and the clock record beside it rest on half a second of work. Every step is timed by
    # its own pair of events; the figure is the median step, each step taken as its slowest rank.
    MAX = torch.distributed.ReduceOp.MAX if dist else None
    with ClockSampler([local] if world == 1 else (list(range(world)) if rank == 0 else None)) as clocks:
        for _ in range(args.warmup):
            step()
        sync()
        k0 = kernels()
        barrier()
        t_begin = time.time()
        times = [timed_step(i) for i in range(steps)]
        mean_ms = agree(sum(times) / len(times), MAX)
        extra = int(min(MAX_TIMED_STEPS, max(0, MIN_TIMED_S * 1e3 / max(mean_ms, 1e-3) - steps)) + 0.999)
        times += [timed_step(steps + i) for i in range(extra)]
        clocks.window(t_begin, time.time())
        barrier()
    launches = kernels() - k0
    tt = torch.tensor(times, device="cuda", dtype=torch.float64)
    if dist:
        dist.all_reduce(tt, op=MAX)
    ms = float(tt.median().item())
    ms_asked = float(tt[:steps].mean().item())

    for m in layers:
        m.set_profiling(True)
    for st_ in stages:
        st_.shared_beside = False  # in line, so that its stage can be timed
    step()
    sync()
    nprof = max(3, min(steps, 10))
    stage = {k: 0.0 for k in _STAGES}
    for i in range(nprof):
        flush.fill_(i & 0xFF)
        torch.cuda.synchronize()
        step()
        sync()
        for m in layers:
            for k, v in m.stage_ms().items():
                stage[k] += v / nprof
    for m in layers:
        m.set_profiling(False)
    stats = [m.stats() for m in layers]

    # End to end: pinned host rows in, pinned host rows out, the copies inside the timed region.
    for _ in range(2):
        step_host()
    barrier()
    e2e_times = []
    while True:
        t0 = time.perf_counter()
        step_host()
        torch.cuda.synchronize()
        e2e_times.append(time.perf_counter() - t0)
        if len(e2e_times) < steps:
            continue
        # Every rank stops after the same step: the decision rests on numbers every rank holds.
        total = agree(sum(e2e_times), torch.distributed.ReduceOp.MIN) if dist else sum(e2e_times)
        if total >= MIN_TIMED_S or len(e2e_times) >= MAX_TIMED_STEPS:
            break
    e2e_s = agree(statistics.median(e2e_times), MAX)

    # Expert parallel: where a step's device time goes on this rank, phase by phase (a few steps with the phases timed).
    ep_phases = None
    if world > 1 and nlayers == 1 and not args.per_assignment:
        moes[0].time_phases = True
        acc = {}
        for i in range(5):
            step()
            sync()
            if i >= 2:
                for k, v in moes[0].phase_ms.items():
                    acc[k] = acc.get(k, 0.0) + v / 3
        moes[0].time_phases = False
        ep_phases = {k: round(v, 4) for k, v in acc.items()}

    # Expert parallel: the rows each rank's experts ran in the last step (routing skew shows here: the busiest rank
    # bounds the step).
    ep_rows = None
    if world > 1:
        rows_t = torch.tensor([sum(m.expert_rows for m in moes)], device="cuda", dtype=torch.int64)
        all_rows = [torch.zeros_like(rows_t) for _ in range(world)]
        dist.all_gather(all_rows, rows_t)
        ep_rows = [int(v.item()) for v in all_rows]

    # The order things are dropped in: every tensor first (and the allocator's cached blocks with them, while the
    # streams they were used on still exist), then the layers with their streams.
    torch.cuda.synchronize()
    # (The page-locked rows too: freeing them records an event on every stream their copies ran on.)
    del x_dev, out_dev, res, xn, flush, tt, x_host, out_host
    moes.clear()
    torch.cuda.empty_cache()
    for st in stages:
        st.close()
    for m in layers:
        m.close()
    if rank != 0:
        return None
    peaks = measured_peaks()
    hit = sum(s["last_experts_hit"] for s in stats)
    tensor_rows = sum(s["last_tensor_rows"] for s in stats)
    algs = [algorithmic(w, T, s["last_experts_hit"], world) for s in stats]
    alg = {k: sum(a[k] for a in algs) for k in algs[0]}
    dom = max(("gate_up", "down"), key=lambda k: stage[k])
    dom_ms = stage[dom]
    # The routed experts' kernel family decides the bound: the stats count the shared expert's rows too when it took the
    # tile kernel (T a layer), so a step whose routed experts all ran as integer-dot rows is bandwidth-bound.
    shared_rows = T if T >= (args.tensor_min or 16) else 0
    routed_tensor_rows = sum(max(0, s["last_tensor_rows"] - shared_rows) for s in stats)
    if routed_tensor_rows * 2 > T * K * nlayers:
        achieved = alg["flops_" + dom] / (dom_ms * 1e-3) / 1e12
        # The fraction is of the burst figure (a GEMM timed alone); the sustained one (a GEMM looping under the power cap)
        # is given beside it, since the stage is timed inside steps that run back to back under that cap.
        roof = dict(bound="tensor", achieved=achieved, peak=peaks["bf16_tflops"], unit="TFLOP/s", frac=achieved / peaks["bf16_tflops"])
        if peaks.get("bf16_tflops_sustained"):
            roof.update(peak_sustained=peaks["bf16_tflops_sustained"], frac_of_sustained=achieved / peaks["bf16_tflops_sustained"])
        # What the launch must move: the hit experts' weights once, the rows in (f16), the results out (f32 h; f16 y).
        A_rows = T * K * nlayers
        roof["traffic_algorithmic"] = (alg["bytes_" + dom] + (A_rows * (E * 2 + F * 4) if dom == "gate_up" else A_rows * (F * 2 + E * 2))) if world == 1 else None
    else:
        achieved = alg["bytes_" + dom] / (dom_ms * 1e-3) / 1e9
        roof = dict(bound="hbm", achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s", frac=achieved / peaks["hbm_gbs"])
    roof.update(kernel=dom, kernel_ms=dom_ms, peak_source=peaks["source"], traffic=traffic_for(w["name"], T, dom) if world == 1 else None)
    cpu_line = None
    if world == 1 and cpu and not args.no_cpu and nlayers == 1:
        cpu_line, _ = cpu_leg(base, x_np, min(T, args.cpu_tokens))
    if world == 1:
        par = "1 GPU"
    else:
        par = (f"expert parallel x{world}: {NE // world} experts and {T} rows per GPU ({scaling} scaling), "
               + ("all-to-all of one q8 row per assignment out and one f16 result back" if args.per_assignment else
                  "all-to-all of one q8 row per (token, GPU) out and one f16 partial sum back")
               + (", contiguous expert ranges" if args.contiguous else ", experts dealt to the GPUs by load" if w.get("zipf_s", 0.0) > 0 else ", experts interleaved"))
    return dict(metric=METRIC, value=world * T / (ms * 1e-3), unit=UNIT, n_gpus=world, steps=steps, warmup=args.warmup,
                ms_per_step=ms, timed_steps=len(times), ms_per_step_mean_of_steps=ms_asked, higher_is_better=True, scaling=scaling,
                vs_baseline=None, dtype="f16" if tensor_rows > 0 else "i8", data="synthetic",
                config=static_config(w, args, world),
                run=dict(experts_hit=hit, tiles=sum(s["last_tiles"] for s in stats), parallelism=par, expert_rows_per_gpu=ep_rows,
                         ep_phase_ms=ep_phases,
                         timing=f"median of {len(times)} steps, each between its own events ({steps} asked for; more until {MIN_TIMED_S} s is timed)"),
                roofline=roof, stage_ms=stage, layer_bytes=alg["bytes_layer"], layer_flops=alg["flops_layer"],
                cpu_baseline=cpu_line, clocks=clocks.summary(),
                e2e=dict(value=world * T / e2e_s, unit=UNIT, h2d_bytes_per_step=T * E * 4, d2h_bytes_per_step=T * E * 4,
                         ms_per_step=e2e_s * 1e3, timed_steps=len(e2e_times)),
                gpu_launches=launches)


DEFAULT_WORKLOAD = "prefill32768_q4_k"   # the largest configuration one GPU holds, and the one the targets are quoted on
SECOND_WORKLOAD = "ragged3521_q4_k_zipf"  # reported beside it when the default runs on one GPU


def run_gpu(args, w):
    import torch

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import datetime

        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=180))
    line = measure(args, w, args.steps, world, rank, local, dist)
    if world == 1 and w["name"] == DEFAULT_WORKLOAD and not args.tokens and not args.layers and not args.no_second:
        second = measure(args, workload(SECOND_WORKLOAD), args.steps, world, rank, local, dist)
        line[SECOND_WORKLOAD] = {k: second[k] for k in ("value", "unit", "ms_per_step", "timed_steps", "config", "run", "roofline", "stage_ms",
                                                         "cpu_baseline", "e2e", "gpu_launches", "dtype")}
        line["gpu_launches"] += second["gpu_launches"]
    if rank == 0:
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=list(synth.CONFIGS))
    ap.add_argument("--cpu-tokens", type=int, default=2048, help="rows of the batch the CPU baseline takes per pass")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-second", action="store_true", help="the default workload alone, without the ragged batch beside it")
    ap.add_argument("--layers", type=int, default=0, help="layers instead of the workload's")
    ap.add_argument("--tokens", type=int, default=0, help="rows instead of the workload's (the sweep's points)")
    ap.add_argument("--host-chunk", type=int, default=-1,
                    help="rows of a chunk of the host-buffer call, whose copies overlap its neighbours' computation (0: never cut; default: 8192 for batches of 16384 rows and more, two halves from 2048 rows)")
    ap.add_argument("--per-assignment", action="store_true", help="expert parallel: one row per assignment on the wire (one GPU's bits) instead of one per (token, GPU)")
    ap.add_argument("--gather-in-kernel", action="store_true",
                    help="long steps: the gate/up tile kernel gathers its rows by index itself (MOE_FLAG_GATHER_IN_KERNEL)")
    ap.add_argument("--contiguous", action="store_true", help="expert parallel: GPU g holds experts [g * per, (g + 1) * per) of the layer as given")
    ap.add_argument("--tensor-min", type=int, default=0, help="rows from which an expert takes the tensor-core kernels (0: the library's default)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    w = workload(args.workload)
    if not isinstance(w["tokens"], int) and not args.tokens:
        args.tokens = w["tokens"][-2]  # a sweep's default point; --tokens picks another
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_gpu(args, w)


if __name__ == "__main__":
    main()
