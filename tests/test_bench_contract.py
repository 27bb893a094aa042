"""bench.py prints exactly one JSON line on stdout, whatever libraries write there; the reference arm reports why it
cannot run."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_prints_one_json_line():
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                          capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    assert out["impl"] == "reference" and "unavailable" in out and "\n" not in out["unavailable"]


def test_stdout_is_reserved_for_the_result():
    code = (
        "import os, sys; sys.argv = ['bench.py']; sys.path.insert(0, %r); import bench; bench.claim_stdout();"
        "os.write(1, b'banner from a library\\n'); print('a stray print'); bench.emit('{\"ok\": 1}')" % str(ROOT)
    )
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=120, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout == '{"ok": 1}\n'
    assert "banner from a library" in proc.stderr and "a stray print" in proc.stderr


import pytest


@pytest.mark.gpu
def test_bench_line_has_the_anchor_and_correctness_keys():
    """One GPU, reduced token count: the line carries the oracle verdict and the comm-only figures next to the
    contract's keys (the NCCL comm-only arm needs at least two ranks and is checked on multi-GPU runs)."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--tokens", "512", "--steps", "3", "--warmup", "3"],
                          capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-3000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    out = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "clocks", "gpu_launches", "e2e", "phases_us", "verified",
                "value_comm_only"):
        assert key in out, key
    assert out["verified"] is True and out["gpu_launches"] > 0
    assert out["e2e"]["h2d_bytes_per_step"] > 0 and out["e2e"]["d2h_bytes_per_step"] > 0
