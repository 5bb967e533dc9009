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
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, source="fallback")


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
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.lines, self.proc = device, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.device)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])), mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def algorithmic(w: dict, T: int, experts_hit: int) -> dict:
    """Bytes and flops the layer needs for T rows that hit `experts_hit` distinct experts."""
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


def run_reference(args, w):
    """The CPU expert path on the host's cores: the oracle port, every thread the process may use."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle

    T_full = w["tokens"]
    T = min(T_full, args.cpu_tokens)
    layer, x = build_layer(w), synth.make_input(T_full, E, seed=1)[:T]
    threads = oracle.threads()
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_step(layer, x, threads)
    times = [cpu_step(layer, x, threads) for _ in range(args.steps)]
    dt = statistics.median(times)
    v = T / dt
    sample = f"first {T} of {T_full} rows per step, median of {args.steps} steps"
    print(json.dumps(dict(metric=METRIC, value=v, unit=UNIT, n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                          ms_per_step=dt * 1e3, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="i8",
                          data="synthetic", impl="reference",
                          config=dict(workload=w["name"], rows=T_full, hidden=E, ffn=F, experts=NE, top_k=K,
                                      weights=synth.TYPE_NAMES[w["gate_type"]]),
                          cpu_baseline=dict(value=v, unit=UNIT, cores=threads, kind="port", sample=sample),
                          e2e=dict(value=v, unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0))))


def run_gpu(args, w):
    import torch

    from c0ven_b200 import MoELayer

    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    T = w["tokens"]
    layer = build_layer(w)
    x_host = torch.from_numpy(synth.make_input(T, E, seed=1 + rank)).pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    flush = torch.empty(512 << 20, dtype=torch.uint8, device="cuda")  # larger than the 126 MB L2
    if world == 1:
        gpu = MoELayer(layer, max_tokens=T, device=local, profile=False, tensor_min_rows=args.tensor_min)
        x_dev, out_dev = x_host.cuda(), torch.empty((T, E), device="cuda")

        def step():
            gpu.forward_device(x_dev.data_ptr(), T, out_dev.data_ptr())

        def step_host():
            gpu.forward(x_host.numpy(), out_host.numpy())
    else:
        # Expert parallel: every rank holds 512 / N experts and brings its own T rows (weak scaling).
        from c0ven_b200 import ep

        stages = ep.GpuStages(layer, rank, world, max_tokens=T, device=local, y_f16=True, profile=False,
                              tensor_min_rows=args.tensor_min)
        moe, gpu = ep.ExpertParallelMoE(stages), stages.moe
        x_dev, out_dev = x_host.cuda(), torch.empty((T, E), device="cuda")

        def step():
            moe.forward(x_dev, out_dev)

        def step_host():
            with torch.cuda.stream(stages.stream):
                xd = x_host.to("cuda", non_blocking=True)
                od = moe.forward(xd)
                out_host.copy_(od, non_blocking=True)
            gpu.sync()
    stream = torch.cuda.ExternalStream(gpu.stream, device=local)

    def barrier():
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    # Timed steps run as a caller would run them: no per-stage timing, the shared expert beside the routed ones, small
    # steps replayed from their recorded graph. The stages are timed afterwards, in a few more steps with the timing on.
    gpu.set_profiling(False)
    for _ in range(args.warmup):
        step()
    gpu.sync()
    k0 = gpu.stats()["kernels"]
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier()
    with ClockSampler(local) as clocks:
        for i in range(args.steps):
            flush.fill_(i & 0xFF)  # L2 flush between timed iterations, outside the timed interval
            torch.cuda.synchronize()
            with torch.cuda.stream(stream):
                starts[i].record(stream)
                step()
                ends[i].record(stream)
            gpu.sync()
        barrier()
    launches = gpu.stats()["kernels"] - k0
    gpu.set_profiling(True)
    step()
    gpu.sync()
    nprof = max(3, min(args.steps, 10))
    stage = {k: 0.0 for k in gpu.stage_ms()}
    for i in range(nprof):
        flush.fill_(i & 0xFF)
        torch.cuda.synchronize()
        step()
        gpu.sync()
        for k, v in gpu.stage_ms().items():
            stage[k] += v / nprof
    gpu.set_profiling(False)
    ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends)) / args.steps
    t = torch.tensor([ms], device="cuda")
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    st = gpu.stats()

    # End to end: host buffers (pinned) in, host buffers out, the copies inside the timed region. One GPU: the C ABI's
    # moe_layer_forward; expert parallel: the same stages with the copies on the layer's stream.
    xh = x_host.numpy()
    for _ in range(2):
        step_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step_host()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / args.steps
    t = torch.tensor([e2e_s], device="cuda")
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())

    def teardown():
        # Everything the layer's stream touched is freed and handed back to the driver while that stream still exists;
        # then the group goes, then the layer.
        nonlocal x_dev, out_dev, flush
        torch.cuda.synchronize()
        del x_dev, out_dev, flush
        if world > 1:
            stages._bufs.clear()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
            stages.close()
        else:
            gpu.close()

    if rank != 0:
        teardown()
        return
    peaks = measured_peaks()
    alg = algorithmic(w, T, st["last_experts_hit"])
    dom = max(("gate_up", "down"), key=lambda k: stage[k])
    dom_ms = stage[dom]
    tensor_path = st["last_tensor_rows"] > 0
    if tensor_path:
        achieved = alg["flops_" + dom] / (dom_ms * 1e-3) / 1e12
        roof = dict(bound="tensor", achieved=achieved, peak=peaks["bf16_tflops"], unit="TFLOP/s", frac=achieved / peaks["bf16_tflops"])
    else:
        achieved = alg["bytes_" + dom] / (dom_ms * 1e-3) / 1e9
        roof = dict(bound="hbm", achieved=achieved, peak=peaks["hbm_gbs"], unit="GB/s", frac=achieved / peaks["hbm_gbs"])
    roof.update(kernel=dom, kernel_ms=dom_ms, peak_source=peaks["source"], traffic=None)
    cpu = None
    if world == 1 and not args.no_cpu:
        from oracle import oracle

        Tc = min(T, args.cpu_tokens)
        threads = oracle.threads()
        cpu_step(layer, xh[:Tc], threads)
        dt = statistics.median([cpu_step(layer, xh[:Tc], threads) for _ in range(3)])
        cpu = dict(value=Tc / dt, unit=UNIT, cores=threads, kind="port", sample=f"first {Tc} of {T} rows, median of 3 passes")
    line = dict(metric=METRIC, value=world * T / (ms * 1e-3), unit=UNIT, n_gpus=world, steps=args.steps, warmup=args.warmup,
                ms_per_step=ms, higher_is_better=True, scaling="weak", vs_baseline=None,
                dtype="bf16" if tensor_path else "i8", data="synthetic",
                config=dict(workload=w["name"], rows=T, runs=w.get("runs"), hidden=E, ffn=F, experts=NE, top_k=K,
                            weights=synth.TYPE_NAMES[w["gate_type"]], zipf_s=w.get("zipf_s", 0.0),
                            experts_hit=st["last_experts_hit"], tiles=st["last_tiles"],
                            parallelism="1 GPU" if world == 1 else f"expert parallel x{world}: {NE // world} experts and {T} rows per GPU, "
                            "all-to-all of q8 rows out and f16 results back", l2="flushed between timed steps"),
                roofline=roof, stage_ms=stage, layer_bytes=alg["bytes_layer"], layer_flops=alg["flops_layer"],
                cpu_baseline=cpu, clocks=clocks.summary(),
                e2e=dict(value=world * T / e2e_s, unit=UNIT, h2d_bytes_per_step=T * E * 4, d2h_bytes_per_step=T * E * 4,
                         ms_per_step=e2e_s * 1e3),
                gpu_launches=launches)
    print(json.dumps(line), flush=True)
    teardown()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="ragged3521_q4_k_zipf", choices=[k for k, v in synth.CONFIGS.items() if isinstance(v["tokens"], int)])
    ap.add_argument("--cpu-tokens", type=int, default=3521, help="rows of the batch the CPU baseline takes per pass")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--tensor-min", type=int, default=0, help="rows from which an expert takes the tensor-core kernels (0: the library's default)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    w = workload(args.workload)
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_gpu(args, w)
        if int(os.environ.get("WORLD_SIZE", "1")) > 1:
            # Under torchrun, leave without the interpreter's teardown: the order in which it would drop the collectives'
            # streams and the allocator's blocks is not ours to set.
            sys.stdout.flush()
            os._exit(0)


if __name__ == "__main__":
    main()
