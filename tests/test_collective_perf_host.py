"""The collective sweep tool on a host-memory communicator: three gloo ranks, every plain collective over a few sizes,
checked against the pattern, with the CSV the device sweep writes."""
import csv
import os
import pathlib
import subprocess
import sys

import torch

from conftest import free_port
from tilexr_b200.tools import collective_perf as cp

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_expected_outputs_of_the_pattern():
    world, n = 3, 12
    ins = [cp.pattern(s, n) for s in range(world)]
    assert ins[0].dtype == torch.float32 and not torch.equal(ins[0], ins[1]) and float(ins[0].abs().max()) <= 125
    assert torch.equal(cp.expected_host("all_gather", world, 1, n), torch.cat(ins))
    assert torch.equal(cp.expected_host("all_reduce", world, 2, n), ins[0] + ins[1] + ins[2])
    assert torch.equal(cp.expected_host("reduce_scatter", world, 1, n), (ins[0] + ins[1] + ins[2])[4:8])
    assert torch.equal(cp.expected_host("all_to_all", world, 2, n), torch.cat([i[8:12] for i in ins]))
    assert torch.equal(cp.expected_host("broadcast", world, 2, n), ins[0])
    assert cp.message_elems("reduce_scatter", 4096, 3, 4) == (1023, 341)
    assert cp.message_elems("all_gather", 4096, 3, 4) == (1024, 3072)


def test_host_sweep_between_three_processes(tmp_path):
    out = tmp_path / "sweep.csv"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nproc-per-node", "3", "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           "-m", "tilexr_b200.tools.collective_perf", "--comm-mode", "host", "--op", "all", "--min-bytes", "1024", "--max-bytes", "1048576",
           "--step-factor", "32", "--iters", "3", "--warmup-iters", "1", "--buffer-mb", "32", "--csv", str(out)]
    env = dict(os.environ, PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    rows = list(csv.DictReader(open(out)))
    assert {x["op"] for x in rows} == set(cp.OPS)
    assert len(rows) == 5 * 3                                            # 1 KB, 32 KB, 1 MB per op
    assert all(int(x["errors"]) == 0 and int(x["ranks"]) == 3 and float(x["avg_us"]) > 0 for x in rows)
    # a message that does not fit a pair's slice of the window ends that op's sweep instead of failing the launch
    cmd[cmd.index("--max-bytes") + 1] = str(256 << 20)
    cmd[cmd.index("--min-bytes") + 1] = str(8 << 20)
    cmd[cmd.index("--op") + 1] = "all_gather"
    r = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert list(csv.DictReader(open(out))) == []
