"""The diagnostics tool `python -m maize_b200.diag` (the commands quoted in profiles/ use it): every mode runs on a
small shape and prints one JSON object per line with the fields the profiles quote."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _diag(*args):
    r = subprocess.run([sys.executable, "-m", "maize_b200.diag", *map(str, args)], cwd=ROOT, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    return [json.loads(line) for line in r.stdout.splitlines() if line.startswith("{")]


def test_roles_and_launch_modes():
    rows = _diag("roles", "--shape", "1024,1024,1024", "--kernels", "1,6", "--flags", "0,1", "--reps", 2)
    assert len(rows) == 4
    for row in rows:
        assert row["ms"] > 0 and row["cta_cycles_max"] > 0 and 0 <= row["mma_wait_data"] <= 1
    rows = _diag("launch", "--shape", "16,256,64", "--kernel", 7, "--reps", 2)
    assert len(rows) == 1 and "skinny" in rows[0]["kernel"]


def test_pitch_and_sweep_modes():
    rows = _diag("pitch", "--shape", "1031,1000,1032", "--pad", "56,1", "--reps", 4, "--set", "repack_bytes=0")
    assert [r["lda=ldb"] for r in rows] == [1032, 1032, 1088, 1088] and all(r["ms"] > 0 for r in rows)
    rows = _diag("sweep", "--shape", "2048,2048,512", "--kernel", 6, "--group-rows", "1024,2048", "--flags", "0",
                 "--set", "serpentine=1")
    assert [r["group_rows"] for r in rows] == [1024, 2048]
