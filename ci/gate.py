#!/usr/bin/env python3
"""Hardware gate of the CI: build, wait for idle GPUs, run the GPU suite, report collisions.

Steps and exit codes (the reference's NPU gate, scripts/ci/gate.py and docs/CI.md, uses the same taxonomy):

    0    everything passed
    20   the native build failed
    21   not enough idle GPUs appeared within the wait budget
    22   a test command failed
    23   collision: another process showed up on a gated GPU while the suite ran (result not trusted)
    130  interrupted

GPUs are only READ through NVML (memory in use, compute processes); the gate changes no setting of any GPU.
`--nvml fake:<json file>` replaces NVML with a scripted sequence of device states, which is how the gate's logic
is tested without hardware.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from typing import Dict, List, Optional, Sequence

EXIT_OK, EXIT_BUILD, EXIT_NO_DEVICES, EXIT_TESTS, EXIT_COLLISION, EXIT_INTERRUPTED = 0, 20, 21, 22, 23, 130


class Nvml:
    """Read-only view of the GPUs: [{index, used_mib, pids}]."""

    def __init__(self):
        import pynvml

        pynvml.nvmlInit()
        self.nv = pynvml

    def snapshot(self) -> List[Dict[str, object]]:
        nv = self.nv
        out = []
        for i in range(nv.nvmlDeviceGetCount()):
            h = nv.nvmlDeviceGetHandleByIndex(i)
            mem = nv.nvmlDeviceGetMemoryInfo(h)
            try:
                pids = sorted(p.pid for p in nv.nvmlDeviceGetComputeRunningProcesses(h))
            except nv.NVMLError:
                pids = []
            out.append({"index": i, "used_mib": int(mem.used >> 20), "pids": pids})
        return out


class FakeNvml:
    """Plays back `states` (a list of snapshots); the last one repeats."""

    def __init__(self, path: str):
        self.states = json.loads(open(path).read())
        self.calls = 0

    def snapshot(self) -> List[Dict[str, object]]:
        s = self.states[min(self.calls, len(self.states) - 1)]
        self.calls += 1
        return s


def idle_devices(snapshot: Sequence[Dict[str, object]], max_used_mib: int, own_pids: Sequence[int] = ()) -> List[int]:
    own = set(own_pids)
    return [int(d["index"]) for d in snapshot
            if int(d["used_mib"]) <= max_used_mib and not (set(d["pids"]) - own)]


def wait_for_idle(nvml, want: int, max_used_mib: int, budget_s: float, poll_s: float, sleep=time.sleep, now=time.time) -> Optional[List[int]]:
    deadline = now() + budget_s
    while True:
        idle = idle_devices(nvml.snapshot(), max_used_mib)
        if len(idle) >= want:
            return idle[:want]
        if now() >= deadline:
            return None
        sleep(poll_s)


def foreign_pids(snapshot: Sequence[Dict[str, object]], devices: Sequence[int], own_pids: Sequence[int]) -> Dict[int, List[int]]:
    own = set(own_pids)
    hits = {}
    for d in snapshot:
        if int(d["index"]) in devices:
            other = sorted(set(d["pids"]) - own)
            if other:
                hits[int(d["index"])] = other
    return hits


def descendants(root: int) -> List[int]:
    """PIDs of `root` and its children, read from /proc (no pattern matching on command lines)."""
    kids: Dict[int, List[int]] = {}
    for name in os.listdir("/proc"):
        if name.isdigit():
            try:
                with open(f"/proc/{name}/stat") as f:
                    fields = f.read().rsplit(")", 1)[1].split()
                kids.setdefault(int(fields[1]), []).append(int(name))
            except (OSError, IndexError, ValueError):
                continue
    out, todo = [], [root]
    while todo:
        p = todo.pop()
        out.append(p)
        todo.extend(kids.get(p, []))
    return out


def run_suite(commands: Sequence[str], devices: Sequence[int], nvml, poll_s: float, log) -> int:
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=",".join(str(d) for d in devices))
    for cmd in commands:
        log(f"[gate] run: {cmd}")
        proc = subprocess.Popen(cmd, shell=True, env=env)
        collided = {}
        while proc.poll() is None:
            time.sleep(poll_s)
            hits = foreign_pids(nvml.snapshot(), devices, descendants(proc.pid))
            if hits:
                collided = hits
        if collided:
            log(f"[gate] collision: foreign processes on gated GPUs {collided}")
            return EXIT_COLLISION
        if proc.returncode != 0:
            log(f"[gate] command failed with {proc.returncode}: {cmd}")
            return EXIT_TESTS
    return EXIT_OK


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--max-used-mib", type=int, default=1024, help="a GPU with more memory in use is not idle")
    ap.add_argument("--wait-s", type=float, default=3600)
    ap.add_argument("--poll-s", type=float, default=10)
    ap.add_argument("--nvml", default="real")
    ap.add_argument("--skip-build", action="store_true")
    ap.add_argument("--build", default=f"{sys.executable} -m tilexr_b200._build")
    ap.add_argument("--suite", action="append", default=None, help="command of the hardware suite (repeatable)")
    args = ap.parse_args(argv)
    log = lambda m: print(m, flush=True)
    suite = args.suite or [
        f"{sys.executable} -m pytest tests -q -m gpu",
        f"{sys.executable} bench.py --steps 20 --warmup 5",
    ]
    try:
        if not args.skip_build:
            log(f"[gate] build: {args.build}")
            if subprocess.call(args.build, shell=True) != 0:
                return EXIT_BUILD
        nvml = FakeNvml(args.nvml.split(":", 1)[1]) if args.nvml.startswith("fake:") else Nvml()
        devices = wait_for_idle(nvml, args.gpus, args.max_used_mib, args.wait_s, args.poll_s)
        if devices is None:
            log(f"[gate] fewer than {args.gpus} idle GPUs within {args.wait_s:.0f} s")
            return EXIT_NO_DEVICES
        log(f"[gate] gated GPUs: {devices}")
        return run_suite(suite, devices, nvml, args.poll_s, log)
    except KeyboardInterrupt:
        return EXIT_INTERRUPTED


if __name__ == "__main__":
    sys.exit(main())
