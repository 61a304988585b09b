#!/usr/bin/env python
"""Benchmark of the BF16 GEMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input: one GEMM of the
workload's shape (at N > 1: A is replicated from rank 0 over NVLink while every rank
multiplies against its own N/G rows of B).  Prints ONE JSON line on rank 0.

Workloads (synthetic seeded inputs of the shapes and distributions of the baseline configs):
  c1 4096^3 | c2 4111x3967x4104 ragged | c3 16x16384x4096 decode | c4 16384^3 (default) |
  c5 8192x28672x8192 MLP up-projection | t 8192^3

Beside the headline the line carries: `verified` (sampled rows of every rank's C against the CPU
oracle, computed after the timed region; the run exits non-zero if they disagree), `roofline`,
`cpu_baseline`, `e2e`, and at N = 1 `cublas_same_run` (torch.matmul on the same tensors, interleaved
with this library's launches) and, on the default workload, `others` (the remaining workloads, briefly).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
# NCCL prints its version banner on stdout at VERSION level; stdout must carry the JSON line only.  Set before
# anything loads NCCL.
if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
    os.environ["NCCL_DEBUG"] = "WARN"

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
SPEC_TFLOPS, SPEC_HBM_GBS = 2250.0, 8000.0
# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu
# capture on a B200; the summaries with the commands are under profiles/).  None where not captured.
SETTLE_S = 1.0   # idle before each of the brief workloads (see brief_workload)

NCU_TRAFFIC = {
    "c4": (11.17e9, "profiles/gemm_pair_16384.md, the 256 x 512 tile with 4096-row groups (captures of the 256 x 256 kernel on the same workload: 9.3 to 18 GB)"),
    "t": (0.95e9, "profiles/gemm_wide_8192.md"),
    "c3": (1.376e8, "profiles/skinny_16x16384x4096.md"),
}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--workload", default="c4", choices=sorted(WORKLOADS))
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--slabs", type=int, default=0,
                   help="row slabs of A when the GEMM is launched per slab (N > 1, --chain-fused 0 or not the chain); "
                        "0 = sizes from the makespan model")
    p.add_argument("--transport", default="auto", choices=["auto", "multimem", "chain", "nccl"],
                   help="how A reaches the other GPUs at N > 1 (auto: the copy-engine chain where symmetric memory is available, else nccl)")
    p.add_argument("--mc-stages", type=int, default=1, choices=[1, 2],
                   help="multimem transport: 2 = root scatters chunks and every GPU multicasts its own, 1 = root multicasts all")
    p.add_argument("--chain-rows", type=int, default=2048, help="chain transport: rows of A per forwarded chunk")
    p.add_argument("--chain-streams", type=int, default=2, choices=[1, 2, 3, 4],
                   help="chain transport: streams the forwarded chunks alternate between")
    p.add_argument("--chain-fused", type=int, default=1, choices=[0, 1],
                   help="chain transport: 1 = one gated GEMM launch per step (waits for rows inside the kernel), 0 = one per slab")
    p.add_argument("--overlap-steps", action="store_true",
                   help="N > 1: give the root an event for \"A is ready\" instead of stream order, so that the replication of a "
                        "step may start while the previous step's GEMM still runs on the root (measured: no difference on 8 GPUs)")
    p.add_argument("--push-ctas", type=int, default=0, help="CTAs of the multicast push kernel (0 = library default)")
    p.add_argument("--e2e-steps", type=int, default=3)
    p.add_argument("--b-layout", default="nk", choices=["nk", "kn"],
                   help="nk: B stored N x K (the bench's contract); kn: B stored K x N as the reference demo walks it (N = 1 GPU only)")
    p.add_argument("--no-pdl", action="store_true",
                   help="ordinary launches instead of the library's default programmatic dependent launch")
    p.add_argument("--b-static", action="store_true",
                   help="declare B static (weights nothing in the stream writes): the decode kernel then prefetches B early")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (for profiler captures)")
    p.add_argument("--no-others", action="store_true", help="skip the brief runs of the other workloads and of cuBLAS")
    p.add_argument("--no-verify", action="store_true", help="skip the check against the CPU oracle (for profiler captures)")
    p.add_argument("--force-kernel", type=int, default=0, help="kernel variant id (0 = the library's heuristic)")
    p.add_argument("--repack", action="store_true", help="give the context scratch for the pitch-aligning pre-pass")
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
    """Samples the SM clock and the throttle reasons of one GPU while the timed regions run: NVML every 5 ms from a
    thread of this process (read-only queries), or `nvidia-smi -lms 100` when NVML cannot be loaded."""
    REASONS = ((0x4, "sw_power_cap"), (0x8, "hw_slowdown"), (0x20, "sw_thermal_slowdown"), (0x40, "hw_thermal_slowdown"))
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_uuid: str):
        self.rows = []  # (wall time, sm MHz, max MHz, set of active reasons)
        self.uuid = gpu_uuid
        self.proc = None
        self.thread = None
        self.stop_flag = False
        self.how = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid)
            mx = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)
            reasons_fn(handle)

            def poll():
                while not self.stop_flag:
                    try:
                        sm = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        mask = int(reasons_fn(handle))
                        self.rows.append((time.time(), sm, mx, {n for bit, n in self.REASONS if mask & bit}))
                    except Exception:
                        pass
                    time.sleep(0.005)

            self.how = "nvml, 5 ms"
            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            pass
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.how = "nvidia-smi, 100 ms"
        self.thread = threading.Thread(target=self._read_smi, daemon=True)
        self.thread.start()

    def _read_smi(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm, mx = float(parts[0]), float(parts[1])
            except ValueError:
                continue
            self.rows.append((time.time(), sm, mx, {n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")}))

    def stop(self):
        self.stop_flag = True
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()

    def summary(self, t0: float, t1: float):
        pad = 0.15 if self.proc is not None else 0.0
        rows = [r for r in self.rows if t0 <= r[0] <= t1 + pad] or self.rows[-3:]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "how": self.how}
        reasons = set()
        for r in rows:
            reasons |= r[3]
        return {"sm_mhz": statistics.median(r[1] for r in rows), "sm_max_mhz": max(r[2] for r in rows),
                "reasons": sorted(reasons), "samples": len(rows), "how": self.how}


def config_for(args, world: int):
    """The `config` object of the JSON line; a function of the command line only, so that both arms print the same."""
    m, n, k, *_rest, desc = WORKLOADS[args.workload]
    rank_bytes = 2 * (m * k + (n // world) * k + m * (n // world))
    small = rank_bytes < 2 * L2_BYTES
    n_sets = max(1, -(-4 * L2_BYTES // rank_bytes)) if small else 1
    kn = args.b_layout == "kn"
    transport = "chain" if args.transport == "auto" else args.transport
    how = {"multimem": "NVSwitch multicast (multimem.st push kernel)",
           "chain": f"a copy-engine chain (rank r forwards to r+1 in {args.chain_rows}-row chunks over {args.chain_streams} "
                    f"stream(s); {'one gated GEMM launch per step' if args.chain_fused else 'one GEMM launch per row slab'}; "
                    + ("A resident on the root, its readiness given by an event: the replication of step s+1 may start "
                       "while step s still multiplies on the root" if args.overlap_steps else
                       "the replication of a step follows the root's previous GEMM in stream order") +
                    "; landing buffers double-buffered across steps)",
           "nccl": "NCCL broadcast per row slab"}[transport]
    launch = "ordinary launches" if args.no_pdl else "programmatic dependent launch (the library's default)"
    if args.b_static:
        launch += ", B declared static (weights)"
    return {
        "workload": f"{args.workload}: {desc}", "M": m, "N": n, "K": k,
        "layout": "A MxK row-major, B KxN row-major, C MxN bf16" if kn else "A MxK row-major, B NxK K-major, C MxN bf16",
        "parallelism": "single GPU" if world == 1 else f"N-sharded x{world}, A replicated from rank 0 every step by " + how,
        "l2": (f"rotating over {n_sets} independent input sets ({n_sets * rank_bytes >> 20} MiB > 4x L2), "
               "back-to-back launches") if small else "inputs exceed L2 (back-to-back launches)",
        "algorithmic_bytes": 2 * (m * k + n * k + m * n),
        "launch": launch,
    }


def cpu_sample(workload: str, seconds: float, steps: int = 1, warmup: int = 0):
    """Times the CPU oracle (port of the path's numeric contract; the reference has no CPU GEMM) on a
    bounded row slab of the workload with every host core this process may use; returns TFLOP/s and a description."""
    from oracle import oracle
    threads = oracle.host_cores()
    oracle.set_num_threads(threads)  # a launcher may have exported OMP_NUM_THREADS=1
    m, n, k, sa, sb, dist, seed, _ = WORKLOADS[workload]
    d = oracle.UNIFORM if dist == "uniform" else oracle.NORMAL
    b = oracle.fill_bf16(seed, 1, (n, k), d, sb)
    probe_rows = min(m, 8)
    a = oracle.fill_bf16(seed, 0, (probe_rows, k), d, sa)
    t0 = time.perf_counter()
    oracle.gemm_bf16(a, b, nthreads=threads)
    dt = max(time.perf_counter() - t0, 1e-6)
    per_row = dt / probe_rows
    rows = int(max(8, min(m, (seconds / max(steps + warmup, 1)) / per_row)))
    rows = min(m, max(8, rows // 8 * 8))
    a = oracle.fill_bf16(seed, 0, (rows, k), d, sa)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.gemm_bf16(a, b, nthreads=threads)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    flops = 2.0 * rows * n * k
    total = sum(times)
    return {
        "tflops": flops * len(times) / total / 1e12,
        "ms_per_step": 1e3 * total / len(times),
        "cores": threads,
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
    r = cpu_sample(args.workload, seconds=40.0, steps=args.steps, warmup=args.warmup)
    unit = "TFLOP/s"
    line = {
        "impl": "reference",
        "metric": "BF16 GEMM TFLOP/s", "value": r["tflops"], "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16 in, fp32 accumulate", "data": "synthetic",
        "config": config_for(args, args.gpus),
        "cpu_baseline": {"value": r["tflops"], "unit": unit, "cores": r["cores"], "kind": "port",
                         "sample": r["sample"]},
        "e2e": {"value": r["tflops"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def sample_rows(m: int, count: int, seed: int, marks=()):
    """Row indices to verify: the first and last rows, rows on both sides of every mark (chunk and slab
    boundaries), and random ones."""
    import numpy as np
    picks = list(range(min(4, m))) + list(range(max(0, m - 4), m))
    for b in marks:
        picks += [x for x in (b - 1, b) if 0 <= x < m]
    rng = np.random.default_rng(seed)
    picks += [int(x) for x in rng.integers(0, m, max(count - len(picks), 8))]
    return np.unique(np.array(picks, dtype=np.int64))


def check_rows(a_rows, b_host, got_rows, k: int, threads: int):
    """Sampled rows of C against the CPU oracle, with the two bounds of the parity tests: the path's tolerance
    1e-2 * sqrt(K) * max|a| * max|b| + one bf16 ulp, and the tight bug-catching bound 1e-4 * sqrt(K) * max|a| * max|b|
    + one bf16 ulp.  Returns (ok, max abs error, path bound)."""
    import numpy as np
    from oracle import oracle
    ref = oracle.gemm_bf16(a_rows, b_host, nthreads=threads)
    ma, mb = oracle.max_abs_bf16(a_rows), oracle.max_abs_bf16(b_host)
    ok, err, bound, _bad = oracle.check(got_rows, ref, k, ma, mb)
    g = oracle.bf16_to_f32(got_rows).astype(np.float64)
    r = oracle.bf16_to_f32(ref).astype(np.float64)
    tight = np.abs(r) * 2.0 ** -7 + 1e-4 * math.sqrt(max(k, 1)) * ma * mb
    ok = bool(ok) and bool(np.all(np.abs(g - r) <= tight))
    return ok, float(err), float(bound)


def to_u16(t):
    import numpy as np
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def time_loop(fn, reps: int):
    """Average milliseconds of `reps` back-to-back calls, CUDA events on the current stream, with wall-clock
    marks for the clock sampler."""
    import torch
    torch.cuda.synchronize()
    w0 = time.time()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        fn(i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps, w0, time.time()


def draw(shape, sigma, dname, dev, gen):
    import torch
    if dname == "uniform":
        return ((torch.rand(shape, device=dev, generator=gen) * 2 - 1) * sigma).to(torch.bfloat16)
    return (torch.randn(shape, device=dev, generator=gen) * sigma).to(torch.bfloat16)


def brief_workload(ctx, name: str, dev, peaks, sampler, reps: int, b_static: bool = False, cublas: bool = True,
                   kn: bool = False):
    """One of the other workloads on one GPU: warm up, time `reps` launches (rotating over input sets when the
    inputs fit in L2), the same with torch.matmul, and check sampled rows against the CPU oracle."""
    import torch
    from oracle import oracle
    m, n, k, sa, sb, dname, seed, desc = WORKLOADS[name]
    gen = torch.Generator(device=dev)
    gen.manual_seed(7000 + seed)
    nbytes = 2 * (m * k + n * k + m * n)
    n_sets = max(1, -(-4 * L2_BYTES // nbytes)) if nbytes < 2 * L2_BYTES else 1
    sets = [(draw((m, k), sa, dname, dev, gen), draw((n, k), sb, dname, dev, gen),
             torch.empty((m, n), dtype=torch.bfloat16, device=dev)) for _ in range(n_sets)]
    # kn: the same B handed over as K x N row-major (the reference demo's layout), through maize_gemm_bf16_kn
    sets_kn = [b.t().contiguous() for _, b, _ in sets] if kn else None
    ctx.set("b_static", 1 if b_static else 0)
    # The loops before this one leave the part at the low clock its power controller chose for them (1.2 GHz after
    # seconds of 16384^3), and that clock lasts longer than a short workload's whole loop: idle first, so that every
    # workload is measured from the same state (the idle is outside every timed region and is reported).
    torch.cuda.synchronize()
    time.sleep(SETTLE_S)
    try:
        def ours(i):
            a, b, c = sets[i % n_sets]
            if kn:
                ctx.gemm_kn(a, sets_kn[i % n_sets], out=c)
            else:
                ctx.gemm(a, b, out=c)
        for i in range(3):
            ours(i)
        total = max(reps, 3) * n_sets if n_sets > 1 else max(reps, 3)
        ms, w0, w1 = time_loop(ours, total)
        ctx.poll()
    finally:
        ctx.set("b_static", 0)
    out = {"workload": f"{name}: {desc}", "kernel": ctx.last_kernel or ctx.pick_kernel(m, n, k), "ms": ms,
           "idle_before_s": SETTLE_S,
           "launch": "library defaults, B declared static (weights)" if b_static else
                     ("library defaults, B stored K x N" if kn else "library defaults"),
           "clocks": sampler.summary(w0, w1) if sampler else None}
    if name == "c3":
        gbs = nbytes / (ms * 1e-3) / 1e9
        out.update(value=gbs, unit="GB/s", roofline={"bound": "hbm", "frac": gbs / peaks["hbm_gbs"], "peak": peaks["hbm_gbs"],
                                                     "frac_of_spec_8TBs": gbs / SPEC_HBM_GBS})
    else:
        tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
        out.update(value=tf, unit="TFLOP/s", roofline={"bound": "tensor", "frac": tf / peaks["bf16_tflops"],
                                                       "peak": peaks["bf16_tflops"], "frac_of_spec_2250": tf / SPEC_TFLOPS})
    if cublas:
        c2 = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
        torch.cuda.synchronize()
        time.sleep(SETTLE_S)

        def lib(i):
            a, b, _ = sets[i % n_sets]
            if kn:
                torch.matmul(a, sets_kn[i % n_sets], out=c2)
            else:
                torch.matmul(a, b.t(), out=c2)
        for i in range(3):
            lib(i)
        ms_lib, _, _ = time_loop(lib, total)
        out["cublas_ms"] = ms_lib
        del c2
    # sampled rows of the last launch's output against the oracle
    a, b, c = sets[(total - 1) % n_sets]
    rows = sample_rows(m, 16, seed)
    idx = torch.from_numpy(rows).to(dev)
    ok, err, bound = check_rows(to_u16(a[idx]), to_u16(b), to_u16(c[idx]), k, oracle.host_cores())
    out["verified"] = {"rows": int(len(rows)), "max_err": err, "bound": bound, "ok": ok}
    del sets, sets_kn, a, b, c
    torch.cuda.empty_cache()
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return

    import torch
    import torch.distributed as dist
    import maize_b200
    from maize_b200.sharded import NShardedGemm, shard_bounds
    from oracle import oracle

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
    host_threads = max(1, oracle.host_cores() // world)
    oracle.set_num_threads(host_threads)

    m, n, k, sa, sb, dname, seed, desc = WORKLOADS[args.workload]
    lo, hi = shard_bounds(n, world, rank)
    ns = hi - lo
    ctx = maize_b200.Context(local_rank)
    if args.force_kernel:
        ctx.set("force_kernel", args.force_kernel)
    if args.repack:
        ctx.set("repack_bytes", (m + ns) * ((k + 63) // 64 * 64) * 2)
    if args.no_pdl:
        ctx.set("pdl", 0)
    if args.b_static:
        # B holds weights that nothing in the stream writes
        ctx.set("b_static", 1)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)  # every rank draws the same A; B rows are taken from a per-rank stream
    gen_b = torch.Generator(device=dev)
    gen_b.manual_seed(1000 + seed * 16 + rank)
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
        sets.append((draw((m, k), sa, dname, dev, gen) if rank == 0 else None,
                     draw((k, ns) if kn else (ns, k), sb, dname, dev, gen_b),
                     torch.empty((m, ns), dtype=torch.bfloat16, device=dev)))
    a_root, b_shard, c_shard = sets[0]
    gemm_call = (lambda a_, b_, c_: ctx.gemm_kn(a_, b_, out=c_)) if kn else (lambda a_, b_, c_: ctx.gemm(a_, b_, out=c_))
    op = NShardedGemm(m, n, k, slabs=args.slabs, ctx=ctx, device=dev, transport=args.transport,
                      push_ctas=args.push_ctas, mc_stages=args.mc_stages, gemm_fn=gemm_call if kn else None,
                      chain_rows=args.chain_rows, chain_streams=args.chain_streams, chain_fused=bool(args.chain_fused))
    # --overlap-steps: A is resident on the root before the timed region (as `value` is defined); its readiness is
    # an event recorded once here, so that the replication of a step need not wait for the previous step's GEMM
    a_ready = None
    if world > 1 and rank == 0 and args.overlap_steps:
        a_ready = torch.cuda.Event()
        a_ready.record()
    step_no = [0]

    def step(_i=0):
        a_i, b_i, c_i = sets[step_no[0] % n_sets]
        step_no[0] += 1
        op.run(a_i, b_i, c_i, a_ready=a_ready)

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
    sync_all()
    t_wall0 = time.time()
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
    last_set = (step_no[0] - 1) % n_sets
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
    ms_per_step = ms_total / args.steps
    flops = 2.0 * m * n * k
    tflops = flops / (ms_per_step * 1e-3) / 1e12
    clocks_headline = sampler.summary(t_wall0, t_wall1) if sampler else None

    # ---- verification, outside the timed region: sampled rows of this rank's C (the last timed step's output)
    # against the CPU oracle fed with the ROOT's rows of A (sent with a plain NCCL broadcast, not with the path
    # under test) and this rank's B
    verified = None
    if not args.no_verify and not kn:
        marks = list(range(0, m, args.chain_rows)) + [lo_ for lo_, _ in op.slabs]
        rows = sample_rows(m, 64, seed, marks)
        idx = torch.from_numpy(rows).to(dev)
        a_rows = sets[last_set][0][idx].contiguous() if rank == 0 else \
            torch.empty((len(rows), k), dtype=torch.bfloat16, device=dev)
        if world > 1:
            dist.broadcast(a_rows, src=0)
        ok, err, bound = check_rows(to_u16(a_rows), to_u16(sets[last_set][1]), to_u16(sets[last_set][2][idx]), k, host_threads)
        v = torch.tensor([0.0 if ok else 1.0, err, bound], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(v, op=dist.ReduceOp.MAX)
        verified = {"rows": int(len(rows)), "cols_per_rank": ns, "ranks": world, "max_err": float(v[1]),
                    "bound": float(v[2]), "ok": bool(float(v[0]) == 0.0),
                    "checker": "CPU oracle on sampled rows of every rank's C shard (the path's tolerance and the tight bound of the parity tests)"}

    # ---- kernel time for the roofline.  N = 1: a step IS one launch of the dominant kernel, so the roofline uses the
    # timed step loop itself; a second, identical loop is recorded beside it with its own clock samples.
    # N > 1: one GEMM over the rank's whole shard with A resident.
    a_res = a_root if rank == 0 else op.a_buffer(b_shard)

    def kernel_only(i):
        _, b_i, c_i = sets[i % n_sets]
        a_i = sets[i % n_sets][0] if rank == 0 else a_res
        gemm_call(a_i, b_i, c_i)

    reps = max(3, min(args.steps, 10)) * n_sets
    repeat_ms, rw0, rw1 = time_loop(kernel_only, reps)
    repeat = {"ms": repeat_ms, "reps": reps, "clocks": sampler.summary(rw0, rw1) if sampler else None}
    kernel_ms = ms_per_step if world == 1 else repeat_ms
    kernel_name = ctx.last_kernel or ctx.pick_kernel(m, ns, k)   # what the kernel-only loop just launched

    # ---- cuBLAS through torch.matmul on the same tensors, interleaved with this library's launches (N = 1)
    cublas = None
    others = None
    peaks = measured_peaks()
    if world == 1 and not args.no_others and not kn and args.workload != "c3":
        c_lib = torch.empty((m, ns), dtype=torch.bfloat16, device=dev)

        def lib_call(i):
            a_i, b_i, _ = sets[i % n_sets]
            torch.matmul(a_i, b_i.t(), out=c_lib)
        for i in range(3):
            lib_call(i)
        runs = []
        loop_reps = max(args.steps, 3) * n_sets
        for who in ("ours", "cublas", "ours", "cublas"):
            ms_, w0_, w1_ = time_loop(kernel_only if who == "ours" else lib_call, loop_reps)
            ck = sampler.summary(w0_, w1_) if sampler else {}
            runs.append({"who": who, "ms": ms_, "tflops": flops / (ms_ * 1e-3) / 1e12, "sm_mhz": ck.get("sm_mhz"),
                         "ms_x_ghz": ms_ * ck["sm_mhz"] / 1e3 if ck.get("sm_mhz") else None})
        cublas = {"api": "torch.matmul(a, b.T, out=...) (cuBLAS), same tensors, same process, loops interleaved",
                  "value": statistics.mean(r["tflops"] for r in runs if r["who"] == "cublas"),
                  "ours_value": statistics.mean(r["tflops"] for r in runs if r["who"] == "ours"), "unit": "TFLOP/s",
                  "reps_per_loop": loop_reps, "runs": runs}
        del c_lib
    if world == 1 and not args.no_others and args.workload == "c4" and not kn:
        others = []
        for name, static, b_kn in (("c1", False, False), ("c2", False, False), ("c3", False, False), ("c3", True, False),
                                   ("c3", False, True), ("c5", False, False), ("t", False, False)):
            try:
                others.append(brief_workload(ctx, name, dev, peaks, sampler, reps=max(args.steps, 5), b_static=static,
                                             cublas=not static, kn=b_kn))
            except Exception as exc:  # report, never hide
                others.append({"workload": name, "error": repr(exc)})

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
                op.run(a_root, b_shard, c_shard)  # A arrives on this stream: stream order says when it is ready
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
        if world == 1 and not args.b_static:
            # the same call with B declared static (weights): B stays on the device between calls, only A goes up
            ctx.set("b_static", 1)
            try:
                e2e_step()
                e_ms2, _, _ = time_loop(lambda i: e2e_step(), args.e2e_steps)
                e2e["b_resident"] = {"value": flops / (e_ms2 * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms2,
                                     "h2d_bytes_per_step": int(ha.numel() * 2), "d2h_bytes_per_step": int(d2h),
                                     "note": "\"b_static\" set: B (weights) is uploaded once and re-used, A and C cross PCIe every step"}
            finally:
                ctx.set("b_static", 0)
            ctx.poll()
        del ha, hb, hc
    except Exception as exc:  # report, never hide
        e2e = {"value": None, "unit": "TFLOP/s", "error": repr(exc)}

    if sampler:
        sampler.stop()
    failed = verified is not None and not verified["ok"]
    if rank == 0:
        k_flops = 2.0 * m * ns * k
        hbm_bound = args.workload == "c3"
        if hbm_bound:
            k_bytes = 2.0 * (m * k + ns * k + m * ns)
            achieved = k_bytes / (kernel_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": None,
                    "peak_source": f"{peaks['source']} STREAM-style copy", "frac_of_spec_8TBs": achieved / SPEC_HBM_GBS}
        else:
            achieved = k_flops / (kernel_ms * 1e-3) / 1e12
            long_run = ms_total > 2000.0
            peak = peaks["bf16_tflops_sustained"] if long_run else peaks["bf16_tflops"]
            roof = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak, "traffic": None,
                    "peak_source": f"{peaks['source']} cuBLAS bf16 " + ("sustained" if long_run else "burst"),
                    "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"],
                    "frac_of_spec_2250": achieved / SPEC_TFLOPS}
        if world == 1 and args.workload in NCU_TRAFFIC:
            roof["traffic"] = NCU_TRAFFIC[args.workload][0]
            roof["traffic_source"] = "one ncu capture of this kernel on this workload, " + NCU_TRAFFIC[args.workload][1]
        roof["kernel"] = kernel_name
        roof["kernel_ms"] = kernel_ms
        roof["kernel_ms_source"] = "the timed step loop (one launch per step)" if world == 1 else \
            "a loop of whole-shard launches with A resident, after the timed region"
        roof["repeat_loop"] = repeat
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
            "config": config_for(args, world), "ms_per_step_by_rank": per_rank_ms,
            "transport": op.transport if world > 1 else None,
            "verified": verified, "roofline": roof, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches,
            "clocks": clocks_headline, "cublas_same_run": cublas, "others": others,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        sys.stderr.write(f"bench: verification against the CPU oracle FAILED: {verified}\n")
        sys.exit(3)


if __name__ == "__main__":
    main()
