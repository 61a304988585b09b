"""Writes the golden fixtures of tests/golden/: seeded inputs and the expected bf16 product.

The expected output is computed HERE by an independent numpy restatement of the contract
(an explicit ascending-k fp32 running sum over whole matrices, one RNE rounding), not by the
C oracle, so the fixtures pin the oracle rather than echo it.  The reference project has no
numeric test, fixture or runnable GEMM for this path, so nothing of it is used.

    python tests/golden/make_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle import oracle as o  # noqa: E402  (input generator only)

CASES = [
    # m, n, k, seed, dist_a, scale_a, dist_b, scale_b
    (48, 40, 64, 100, 0, 1.0, 0, 1.0),
    (130, 75, 520, 101, 1, 1.0, 1, 1.0),     # ragged like config 2, U(-1, 1)
    (16, 96, 1024, 102, 0, 1.0, 0, 0.02),    # decode-like, small weights
    (1, 8, 8, 103, 0, 1.0, 0, 1.0),
    (257, 129, 72, 104, 0, 1.0, 0, 1.0),
]


def f32(x):
    return (x.astype(np.uint32) << 16).view(np.float32)


def rne(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((u + (0x7FFF + ((u >> 16) & 1))) >> 16).astype(np.uint16)


def product(a, b):
    af, bf = f32(a), f32(b)
    acc = np.zeros((a.shape[0], b.shape[0]), dtype=np.float32)
    for k in range(a.shape[1]):  # ascending k, one fp32 rounding per step; products are exact
        acc = acc + np.outer(af[:, k], bf[:, k]).astype(np.float32)
    return rne(acc)


def main():
    index = {"cases": []}
    for i, (m, n, k, seed, da, sa, db, sb) in enumerate(CASES):
        a = o.fill_bf16(seed, 0, (m, k), da, sa)
        b = o.fill_bf16(seed, 1, (n, k), db, sb)
        name = f"case{i}_{m}x{n}x{k}.npz"
        np.savez_compressed(HERE / name, a=a, b=b, c=product(a, b))
        index["cases"].append(dict(file=name, m=m, n=n, k=k, seed=seed, dist_a=da, scale_a=sa, dist_b=db, scale_b=sb))
    (HERE / "index.json").write_text(json.dumps(index, indent=1) + "\n")
    print("wrote", len(CASES), "cases")


if __name__ == "__main__":
    main()
