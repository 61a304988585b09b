"""Performance diagnostics of the GEMM kernels, on cuda:0.

    python -m maize_b200.diag roles  --shape 8192,8192,8192 --kernels 1,5,6 [--flags 0,1,2]
    python -m maize_b200.diag sweep  --shape 16384,16384,16384 --kernel 6 --group-rows 2048,3072,4096 --flags 0,4,12
    python -m maize_b200.diag launch --shape 16,256,64 [--kernel 7] [--flags 2] [--reps 3]
    python -m maize_b200.diag pitch  --shape 4111,3967,4104 [--pad 56,1] [--reps 24]

``roles``  prints, per kernel variant and diagnostic flag, the time, the busiest CTA's cycle count, the
           effective SM clock and the share of its life each role spent blocked (the library's own cycle
           counters, ``maize_ctx_set("profile", 1)``).
``sweep``  launches one GEMM per (group_rows, debug_flags) pair, for capture under ``ncu --metrics ...``.
``launch`` launches one shape a few times, for ``ncu --metrics gpu__time_duration.sum``.
``pitch``  times one shape with the operand pitch (lda = ldb) and the C pitch (ldc) as given and padded by
           ``--pad`` elements, in the four combinations: tells a slow epilogue (C rows that are not 16-byte
           aligned) from slow loads (operand rows whose pitch is not a multiple of 128 bytes).

Diagnostic flags (``maize_ctx_set("debug_flags", f)``; results are WRONG when set, and the library takes them
only while its per-CTA cycle accounting, "profile", is on): 1 = every load fetches tile (0, 0) so all operand
traffic hits in L2, 2 = no loads at all, 4 = A loaded with an evict-last L2 hint, 8 = B loaded with evict-first
(4 and 8: pair kernels only).  ``--set key=value`` (repeatable) passes any other tunable to the context, e.g.
``--set serpentine=1 --set tail_split=0``.
"""
from __future__ import annotations

import argparse
import json
import statistics


def _ints(text):
    return [int(x) for x in text.split(",") if x != ""]


def main():
    import torch
    import maize_b200

    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("mode", choices=["roles", "sweep", "launch", "pitch"])
    ap.add_argument("--shape", default="8192,8192,8192", help="M,N,K")
    ap.add_argument("--kernels", default="1,5,6")
    ap.add_argument("--kernel", type=int, default=0)
    ap.add_argument("--flags", default="0")
    ap.add_argument("--group-rows", default="2048")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--pad", default="56,1", help="pitch mode: elements added to lda = ldb and to ldc")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE", help="context tunable (repeatable)")
    args = ap.parse_args()

    m, n, k = _ints(args.shape)
    torch.cuda.set_device(0)
    ctx = maize_b200.Context(0)
    for item in args.set:
        key, value = item.split("=", 1)
        ctx.set(key, int(value))

    def set_flags(flags):
        # the library honours the switches only while profiling is on
        ctx.set("profile", 1 if flags else 0)
        ctx.set("debug_flags", flags)

    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    c = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)

    def timed(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            ctx.gemm(a, b, out=c)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    if args.mode == "roles":
        for kern in _ints(args.kernels):
            for flags in _ints(args.flags):
                ctx.set("force_kernel", kern)
                set_flags(flags)
                timed(3)
                ms = timed(args.reps)
                ctx.set("profile", 1)
                ms_prof = timed(1)
                prof = ctx.read_profile()
                ctx.set("profile", 0)
                if not prof:
                    print(json.dumps({"kernel": kern, "flags": flags, "ms": round(ms, 4), "note": "no role counters"}))
                    continue
                pair = "2cta" in ctx.pick_kernel(m, n, k)
                lead = [p for i, p in enumerate(prof) if not pair or i % 2 == 0]
                cyc = max(p["cta_cycles"] for p in prof)

                def share(rows, key):
                    return round(statistics.mean(p[key] / max(p["cta_cycles"], 1) for p in rows), 3)

                print(json.dumps({
                    "kernel": ctx.pick_kernel(m, n, k), "flags": flags, "ms": round(ms, 4),
                    "tflops": round(2.0 * m * n * k / ms / 1e9, 1), "cta_cycles_max": cyc,
                    "eff_sm_mhz": round(cyc / (ms_prof * 1e3)),
                    "mma_wait_data": share(lead, "mma_wait_full"),
                    "mma_wait_accumulator": share(lead, "mma_wait_acc_empty"),
                    "producer_wait_stage": share(prof, "producer_wait_empty"),
                    "epilogue_wait_accumulator": share(prof, "epilogue_wait_acc_full"),
                    "epilogue_drain": share(prof, "epilogue_drain")}), flush=True)
    elif args.mode == "pitch":
        pad_ab, pad_c = _ints(args.pad)
        sets = 4  # rotate over independent operands so that a set has left L2 before it is used again
        for dab, dc in ((0, 0), (0, pad_c), (pad_ab, 0), (pad_ab, pad_c)):
            lda, ldc = k + dab, n + dc
            ops = [(torch.randn(m, lda, device="cuda").bfloat16(), torch.randn(n, lda, device="cuda").bfloat16(),
                    torch.empty(m, ldc, device="cuda", dtype=torch.bfloat16)) for _ in range(sets)]

            def run(reps):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for i in range(reps):
                    x, w, y = ops[i % sets]
                    ctx.gemm(x[:, :k], w[:, :k], out=y[:, :n])
                e1.record()
                torch.cuda.synchronize()
                return e0.elapsed_time(e1) / reps

            run(4)
            ms = run(args.reps)
            print(json.dumps({"lda=ldb": lda, "ldc": ldc, "ms": round(ms, 4),
                              "tflops": round(2.0 * m * n * k / ms / 1e9, 1)}), flush=True)
            del ops
    elif args.mode == "sweep":
        ctx.set("force_kernel", args.kernel)
        for g in _ints(args.group_rows):
            for flags in _ints(args.flags):
                ctx.set("group_rows", g)
                set_flags(flags)
                ms = timed(1)
                print(json.dumps({"group_rows": g, "flags": flags, "ms": round(ms, 4)}), flush=True)
    else:
        ctx.set("force_kernel", args.kernel)
        for flags in _ints(args.flags):
            set_flags(flags)
            ms = timed(args.reps)
            print(json.dumps({"kernel": ctx.pick_kernel(m, n, k), "flags": flags, "ms_per_launch": round(ms, 4)}),
                  flush=True)
    set_flags(0)
    ctx.set("force_kernel", 0)
    ctx.poll()


if __name__ == "__main__":
    main()
