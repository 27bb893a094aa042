"""Collectives through the NVSwitch multicast object on real GPUs (two or more): numerics of all-reduce,
reduce-scatter, all-gather and broadcast against an fp32 sum, for bf16, fp16 and fp32.  The ranks run as child
processes of the tool that also times them; every rank leaves together, after a barrier."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from conftest import free_port

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def test_nvls_collectives_numerics():
    n = min(torch.cuda.device_count(), 4)
    if n < 2:
        pytest.skip("needs two GPUs behind an NVSwitch")
    env = dict(os.environ, TILEXR_WAIT_TIMEOUT_MS="5000", PYTHONPATH=str(ROOT))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), "-m", "tilexr_b200.tools.nvls_perf", "--check-only"]
    proc = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-4000:]
    lines = [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert lines, proc.stdout[-2000:] + proc.stderr[-2000:]
    verdict = json.loads(lines[-1])
    if verdict.get("nvls") == "unavailable":
        pytest.skip("no multicast object on this system: " + verdict.get("why", ""))
    assert verdict == {"nvls": "ok", "world": n, "numerics": "pass", "rows": []}
