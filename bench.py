#!/usr/bin/env python
"""Benchmark of the BF16 GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input: one GEMM of the
workload's shape (at N > 1: replicate A from rank 0 slab by slab over NCCL while every rank
multiplies against its own N/G rows of B).  Prints ONE JSON line on rank 0.

Workloads (synthetic seeded inputs of the shapes and distributions of the baseline configs):
  c1 4096^3 | c2 4111x3967x4104 ragged | c3 16x16384x4096 decode | c4 16384^3 (default) |
  c5 8192x28672x8192 MLP up-projection | t 8192^3
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (M, N, K, sigma_a, sigma_b, dist, seed, description)
    "c1": (4096, 4096, 4096, 1.0, 1.0, "normal", 0, "BF16 GEMM M=N=K=4096"),
    "c2": (4111, 3967, 4104, 1.0, 1.0, "uniform", 1, "ragged BF16 GEMM M=4111 N=3967 K=4104"),
    "c3": (16, 16384, 4096, 1.0, 0.02, "normal", 2, "skinny decode BF16 GEMM M=16 N=16384 K=4096"),
    "c4": (16384, 16384, 16384, 1.0, 1.0, "normal", 3, "large square BF16 GEMM M=N=K=16384"),
    "c5": (8192, 28672, 8192, 1.0, 0.02, "normal", 4, "MLP up-projection BF16 GEMM M=8192 K=8192 N=28672"),
    "t": (8192, 8192, 8192, 1.0, 1.0, "normal", 5, "BF16 GEMM M=N=K=8192"),
}
L2_BYTES = 126 * 1024 * 1024
# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu
# capture on a B200; the summaries with the commands are under profiles/).  None where not captured.
NCU_TRAFFIC = {
    "c4": 9.39e9,   # profiles/gemm_pair_16384.md
    "t": 1.214e9,   # profiles/gemm_pair_8192.md
    "c3": 1.393e8,  # profiles/skinny_16x16384x4096.md
}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--slabs", type=int, default=0,
                   help="row slabs of A for the overlapped broadcast (N > 1); 0 = sizes from the makespan model")
    p.add_argument("--transport", default="auto", choices=["auto", "multimem", "chain", "nccl"],
                   help="how A reaches the other GPUs at N > 1 (auto: the copy-engine chain where symmetric memory is available, else nccl)")
    p.add_argument("--mc-stages", type=int, default=1, choices=[1, 2],
                   help="multimem transport: 2 = root scatters chunks and every GPU multicasts its own, 1 = root multicasts all")
    p.add_argument("--chain-rows", type=int, default=1024, help="chain transport: rows of A per forwarded chunk")
    p.add_argument("--chain-in-library", action="store_true",
                   help="chain transport: enqueue a step's forwarding with one library call instead of per-chunk calls")
    p.add_argument("--chain-streams", type=int, default=1, choices=[1, 2],
                   help="chain transport with --chain-in-library: streams the forwarded chunks alternate between")
    p.add_argument("--chain-fused", action="store_true",
                   help="chain transport: one gated GEMM launch per step (waits for rows inside the kernel)")
    p.add_argument("--push-ctas", type=int, default=0, help="CTAs of the multicast push kernel (0 = library default)")
    p.add_argument("--e2e-steps", type=int, default=3)
    p.add_argument("--b-layout", default="nk", choices=["nk", "kn"],
                   help="nk: B stored N x K (the bench's contract); kn: B stored K x N as the reference demo walks it (N = 1 GPU only)")
    p.add_argument("--no-pdl", action="store_true",
                   help="c3 only: do not use programmatic dependent launch with static weights for the decode kernel")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (for profiler captures)")
    p.add_argument("--force-kernel", type=int, default=0, help="kernel variant id (0 = the library's heuristic)")
    p.add_argument("--cpu-seconds", type=float, default=10.0, help="target CPU time of the cpu_baseline sample")
    return p.parse_args()


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            d = json.loads(f.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "source": "measured"}
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_uuid: str):
        self.rows = []
        self.proc = None
        self.uuid = gpu_uuid
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [r for r in self.rows if t0 <= r[0] <= t1 + 0.15] or self.rows[-3:]
        for _, line in rows:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_sample(workload: str, seconds: float, steps: int = 1, warmup: int = 0):
    """Times the CPU oracle (port of the path's numeric contract; the reference has no CPU GEMM) on a
    bounded row slab of the workload with every host thread; returns TFLOP/s and a description."""
    import numpy as np
    from oracle import oracle
    m, n, k, sa, sb, dist, seed, _ = WORKLOADS[workload]
    d = oracle.UNIFORM if dist == "uniform" else oracle.NORMAL
    b = oracle.fill_bf16(seed, 1, (n, k), d, sb)
    probe_rows = min(m, 8)
    a = oracle.fill_bf16(seed, 0, (probe_rows, k), d, sa)
    t0 = time.perf_counter()
    oracle.gemm_bf16(a, b)
    dt = max(time.perf_counter() - t0, 1e-6)
    per_row = dt / probe_rows
    rows = int(max(8, min(m, (seconds / max(steps + warmup, 1)) / per_row)))
    rows = min(m, max(8, rows // 8 * 8))
    a = oracle.fill_bf16(seed, 0, (rows, k), d, sa)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.gemm_bf16(a, b)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    flops = 2.0 * rows * n * k
    total = sum(times)
    return {
        "tflops": flops * len(times) / total / 1e12,
        "ms_per_step": 1e3 * total / len(times),
        "cores": oracle.num_threads(),
        "rows": rows,
        "sample": f"first {rows} of {m} rows of A against all of B ({n}x{k}), full K; "
                  f"{'whole workload' if rows == m else 'rate extrapolates linearly in M'}",
    }


def run_reference(args):
    """The reference arm: the path's CPU implementation on the host cores.  The reference project holds no
    runnable GEMM (it prints PTX) and no CPU matmul, so this is the CPU port, with all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    m, n, k, *_ = WORKLOADS[args.workload]
    r = cpu_sample(args.workload, seconds=40.0, steps=args.steps, warmup=args.warmup)
    unit = "TFLOP/s"
    line = {
        "impl": "reference",
        "metric": "BF16 GEMM TFLOP/s", "value": r["tflops"], "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 in, fp32 accumulate", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {WORKLOADS[args.workload][7]}", "M": m, "N": n, "K": k},
        "cpu_baseline": {"value": r["tflops"], "unit": unit, "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["tflops"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist
    import maize_b200
    from maize_b200.sharded import NShardedGemm, shard_bounds

    # NCCL prints its version banner on stdout at VERSION level; stdout must carry the JSON line only
    if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs `python -m torch.distributed.run --nproc-per-node N bench.py ...`")
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    m, n, k, sa, sb, dname, seed, desc = WORKLOADS[args.workload]
    lo, hi = shard_bounds(n, world, rank)
    ns = hi - lo
    ctx = maize_b200.Context(local_rank)
    if args.force_kernel:
        ctx.set("force_kernel", args.force_kernel)
    decode_pdl = args.workload == "c3" and not args.no_pdl
    if decode_pdl:
        # decode: B holds weights that nothing in the stream writes, so consecutive launches may overlap
        ctx.set("pdl", 1)
        ctx.set("b_static", 1)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)  # every rank draws the same A; B rows are taken from a per-rank stream

    def draw(shape, sigma, g):
        if dname == "uniform":
            return ((torch.rand(shape, device=dev, generator=g) * 2 - 1) * sigma).to(torch.bfloat16)
        return (torch.randn(shape, device=dev, generator=g) * sigma).to(torch.bfloat16)

    gen_b = torch.Generator(device=dev)
    gen_b.manual_seed(1000 + seed * 16 + rank)
    total_bytes = 2 * (m * k + n * k + m * n)
    rank_bytes = 2 * (m * k + ns * k + m * ns)
    # Inputs that fit in L2 would be served from it on back-to-back launches: rotate over enough
    # independent input sets that the bytes touched between two uses of a set exceed 4x L2.
    small = rank_bytes < 2 * L2_BYTES
    n_sets = max(1, -(-4 * L2_BYTES // rank_bytes)) if small else 1
    kn = args.b_layout == "kn"
    if kn and world != 1:
        raise SystemExit("--b-layout kn is a single-GPU measurement")
    sets = []
    for _ in range(n_sets):
        sets.append((draw((m, k), sa, gen) if rank == 0 else None, draw((k, ns) if kn else (ns, k), sb, gen_b),
                     torch.empty((m, ns), dtype=torch.bfloat16, device=dev)))
    a_root, b_shard, c_shard = sets[0]
    gemm_call = (lambda a_, b_, c_: ctx.gemm_kn(a_, b_, out=c_)) if kn else (lambda a_, b_, c_: ctx.gemm(a_, b_, out=c_))
    op = NShardedGemm(m, n, k, slabs=args.slabs, ctx=ctx, device=dev, transport=args.transport,
                      push_ctas=args.push_ctas, mc_stages=args.mc_stages, gemm_fn=gemm_call if kn else None)
    step_no = [0]

    def step():
        a_i, b_i, c_i = sets[step_no[0] % n_sets]
        step_no[0] += 1
        op.run(a_i, b_i, c_i)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    sync_all()
    ctx.poll()

    sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid)) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.25)

    launches0 = ctx.launch_count
    t_wall0 = time.time()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    sync_all()
    ms_total = e0.elapsed_time(e1)
    t_wall1 = time.time()
    launches = ctx.launch_count - launches0
    ctx.poll()
    per_rank_ms = [ms_total / args.steps]
    if world > 1:
        t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
        allt = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(allt, t)
        per_rank_ms = [round(float(x.item()) / args.steps, 4) for x in allt]
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
        lt = torch.tensor([launches], dtype=torch.int64, device=dev)
        dist.all_reduce(lt)
        launches = int(lt.item())
    if sampler:
        time.sleep(0.15)
        sampler.stop()
    ms_per_step = ms_total / args.steps
    flops = 2.0 * m * n * k
    tflops = flops / (ms_per_step * 1e-3) / 1e12

    # kernel-only time on this rank (for the roofline): one GEMM over the rank's whole shard, A resident
    a_res = a_root if rank == 0 else op.a_buffer(b_shard)
    reps = max(3, min(args.steps, 10)) * n_sets
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        _, b_i, c_i = sets[i % n_sets]
        a_i = sets[i % n_sets][0] if rank == 0 else a_res
        gemm_call(a_i, b_i, c_i)
    e1.record()
    torch.cuda.synchronize()
    kernel_ms = e0.elapsed_time(e1) / reps
    kernel_name = ctx.pick_kernel(m // len(op.slabs) if world > 1 else m, ns, k)

    # ---- end to end through the host-buffer entry point (N = 1) or pinned copies + sharded step (N > 1)
    e2e = None
    try:
        if args.no_e2e:
            raise RuntimeError("skipped by --no-e2e")
        if kn:
            raise RuntimeError("the host-buffer entry point takes B as N x K only")
        ha = torch.empty((m, k), dtype=torch.bfloat16).pin_memory() if rank == 0 else None
        hb = torch.empty((ns, k), dtype=torch.bfloat16).pin_memory()
        hc = torch.empty((m, ns), dtype=torch.bfloat16).pin_memory()
        if rank == 0:
            ha.copy_(a_root)
        hb.copy_(b_shard)
        torch.cuda.synchronize()
        h2d = hb.numel() * 2 + (ha.numel() * 2 if rank == 0 else 0)
        d2h = hc.numel() * 2

        def e2e_step():
            if world == 1:
                ctx.gemm_host(ha.data_ptr(), m, k, hb.data_ptr(), ns, k, hc.data_ptr(), m, ns)
            else:
                if rank == 0:
                    a_root.copy_(ha, non_blocking=True)
                b_shard.copy_(hb, non_blocking=True)
                op.run(a_root, b_shard, c_shard)
                hc.copy_(c_shard, non_blocking=True)

        e2e_step()
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        e1.record()
        sync_all()
        e_ms = e0.elapsed_time(e1) / args.e2e_steps
        tot = torch.tensor([e_ms, float(h2d), float(d2h)], dtype=torch.float64, device=dev)
        if world > 1:
            mx = tot.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(tot)
            e_ms, h2d, d2h = float(mx[0]), int(tot[1]), int(tot[2])
        e2e = {"value": flops / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "api": "maize_gemm_bf16_host (C ABI, pinned host buffers)" if world == 1 else
                      "pinned host copies + NShardedGemm.run"}
        ctx.poll()
        del ha, hb, hc
    except Exception as exc:  # report, never hide
        e2e = {"value": None, "unit": "TFLOP/s", "error": repr(exc)}

    if rank == 0:
        peaks = measured_peaks()
        clocks = sampler.summary(t_wall0, t_wall1) if sampler else None
        k_flops = 2.0 * m * ns * k
        hbm_bound = args.workload == "c3"
        if hbm_bound:
            k_bytes = 2.0 * (m * k + ns * k + m * ns)
            achieved = k_bytes / (kernel_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                    "peak_source": f"{peaks['source']} STREAM-style copy"}
        else:
            achieved = k_flops / (kernel_ms * 1e-3) / 1e12
            long_run = ms_total > 2000.0
            peak = peaks["bf16_tflops_sustained"] if long_run else peaks["bf16_tflops"]
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak, "traffic": None,
                    "peak_source": f"{peaks['source']} cuBLAS bf16 " + ("sustained" if long_run else "burst")}
        roof["traffic"] = NCU_TRAFFIC.get(args.workload) if world == 1 else None
        roof["kernel"] = kernel_name
        roof["kernel_ms"] = kernel_ms
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            r = cpu_sample(args.workload, seconds=args.cpu_seconds)
            cpu = {"value": r["tflops"], "unit": "TFLOP/s", "cores": r["cores"], "kind": "port",
                   "sample": r["sample"]}
        line = {
            "metric": "BF16 GEMM TFLOP/s", "value": tflops, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16 in, fp32 accumulate", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {desc}", "M": m, "N": n, "K": k,
                       "layout": "A MxK row-major, B KxN row-major, C MxN bf16" if kn else
                                 "A MxK row-major, B NxK K-major, C MxN bf16",
                       "parallelism": "single GPU" if world == 1 else
                                      f"N-sharded x{world}, A replicated from rank 0 in {len(op.slabs)} row slabs over "
                                      + {"multimem": "NVSwitch multicast (multimem.st push kernel)",
                                         "chain": "a copy-engine chain (rank r forwards to r+1 in 1024-row chunks)",
                                         "nccl": "NCCL broadcast"}[op.transport],
                       "l2": (f"rotating over {n_sets} independent input sets ({n_sets * rank_bytes >> 20} MiB > 4x L2), "
                              "back-to-back launches") if small else "inputs exceed L2 (back-to-back launches)",
                       "algorithmic_bytes": total_bytes, "ms_per_step_by_rank": per_rank_ms,
                       "launch": "programmatic dependent launch, B declared static (weights)" if decode_pdl else "plain"},
            "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
