#!/usr/bin/env python3
"""Hardware gate of the CI: build, wait for idle GPUs, run the GPU suite, report collisions.

Steps and exit codes (the reference's NPU gate, scripts/ci/gate.py and docs/CI.md, uses the same taxonomy):

    0    everything passed
    20   the native build failed
    21   not enough idle GPUs appeared within the wait budget
    22   a test command failed
    23   collision: another process showed up on a gated GPU while the suite ran (result not trusted)
    24   obsolete: the checked-out source is not the commit this run was asked to gate (`--expect-sha`)
    25   infrastructure: a command outlived its time limit, or left processes behind on the gated GPUs
    130  interrupted (SIGINT / SIGTERM): the running command's process group is ended first

Every command runs in a session of its own, so that what it started can be ended as one process group (by its id, never by
a pattern) when it runs out of time or the gate is cancelled; after the suite the gate checks that nothing of it is left on
the gated GPUs.  `--report FILE` writes what happened phase by phase (command, seconds, exit code, failure class) as JSON;
the same summary is printed.  Variables that look like credentials are not passed on to the commands.

GPUs are only READ through NVML (memory in use, compute processes); the gate changes no setting of any GPU.
`--nvml fake:<json file>` replaces NVML with a scripted sequence of device states, which is how the gate's logic
is tested without hardware.
"""
from __future__ import annotations

import argparse
import json
import os
import signal
import subprocess
import sys
import time
from typing import Dict, List, Optional, Sequence

EXIT_OK, EXIT_BUILD, EXIT_NO_DEVICES, EXIT_TESTS, EXIT_COLLISION, EXIT_INTERRUPTED = 0, 20, 21, 22, 23, 130
EXIT_OBSOLETE, EXIT_INFRASTRUCTURE = 24, 25
FAILURE_CLASS = {EXIT_OK: "none", EXIT_BUILD: "code", EXIT_TESTS: "code", EXIT_NO_DEVICES: "resource", EXIT_COLLISION: "resource",
                 EXIT_OBSOLETE: "obsolete", EXIT_INFRASTRUCTURE: "infrastructure", EXIT_INTERRUPTED: "cancelled"}
SECRET_MARKS = ("TOKEN", "SECRET", "PASSWORD", "PASSWD", "CREDENTIAL", "PRIVATE_KEY", "API_KEY")


class Cancelled(Exception):
    """SIGINT or SIGTERM reached the gate."""


def child_environment(environ=None, devices: Sequence[int] = ()) -> Dict[str, str]:
    """The environment of a gated command: the caller's without anything that looks like a credential, and with the gated
    GPUs as the only visible ones."""
    src = os.environ if environ is None else environ
    env = {k: v for k, v in src.items() if not any(mark in k.upper() for mark in SECRET_MARKS)}
    if devices:
        env["CUDA_VISIBLE_DEVICES"] = ",".join(str(d) for d in devices)
    return env


def verify_sha(source: str, expected: str, run_git=None) -> Optional[str]:
    """None when `source` is checked out at `expected` (a full or abbreviated commit id), else what is wrong."""
    if run_git is None:
        def run_git(path):
            return subprocess.run(["git", "-C", path, "rev-parse", "HEAD"], capture_output=True, text=True, check=True).stdout.strip()
    want = expected.strip().lower()
    if len(want) < 7 or any(c not in "0123456789abcdef" for c in want):
        return f"not a commit id: {expected!r}"
    try:
        head = run_git(source).strip().lower()
    except (OSError, subprocess.CalledProcessError) as exc:
        return f"cannot read the head of {source}: {exc}"
    return None if head.startswith(want) else f"{source} is at {head[:12]}, this run gates {want[:12]}"


def end_process_group(pgid: int, grace_s: float = 5.0, sleep=time.sleep, reap=lambda: None) -> bool:
    """SIGTERM, then after `grace_s` SIGKILL, to exactly the process group `pgid`.  True when the group is gone.  `reap` is
    called while waiting (the caller's `Popen.poll`): an ended child that nobody has waited for still counts as a member."""
    def alive() -> bool:
        reap()
        try:
            os.killpg(pgid, 0)
            return True
        except ProcessLookupError:
            return False
        except PermissionError:
            return True

    for sig, wait in ((signal.SIGTERM, grace_s), (signal.SIGKILL, 2.0)):
        if not alive():
            return True
        try:
            os.killpg(pgid, sig)
        except ProcessLookupError:
            return True
        waited = 0.0
        while alive() and waited < wait:
            sleep(0.05)
            waited += 0.05
    return not alive()


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


def run_command(cmd: str, env: Dict[str, str], devices: Sequence[int], nvml, poll_s: float, timeout_s: float, log, cancelled=lambda: False) -> Dict[str, object]:
    """One command in a session of its own.  Returns its phase record: seconds, exit code, collisions seen, whether it was
    ended for running out of time, and what it left behind."""
    t0 = time.time()
    proc = subprocess.Popen(cmd, shell=True, env=env, start_new_session=True)
    pgid = proc.pid                                   # the leader of the new session leads its process group too
    rec: Dict[str, object] = {"command": cmd, "collisions": {}, "timed_out": False, "cancelled": False, "leftover_pids": []}
    while proc.poll() is None:
        time.sleep(poll_s)
        if cancelled():
            rec["cancelled"] = True
            break
        if timeout_s > 0 and time.time() - t0 > timeout_s:
            rec["timed_out"] = True
            break
        if devices:
            hits = foreign_pids(nvml.snapshot(), devices, descendants(proc.pid))
            if hits:
                rec["collisions"] = {str(k): v for k, v in hits.items()}
    if proc.poll() is None:
        log(f"[gate] ending process group {pgid} ({'cancelled' if rec['cancelled'] else 'out of time'})")
        end_process_group(pgid, reap=proc.poll)
        proc.wait()
    else:
        # the command itself returned: whatever it started and did not wait for is ended with its group
        left = [p for p in descendants(proc.pid) if p != proc.pid]
        try:
            os.killpg(pgid, 0)
            group_alive = True
        except (ProcessLookupError, PermissionError):
            group_alive = False
        if group_alive:
            rec["leftover_pids"] = left or [pgid]
            end_process_group(pgid, reap=proc.poll)
    rec["exit_code"] = proc.returncode
    rec["seconds"] = round(time.time() - t0, 3)
    return rec


def classify(rec: Dict[str, object], build: bool = False) -> int:
    if rec["cancelled"]:
        return EXIT_INTERRUPTED
    if rec["collisions"]:
        return EXIT_COLLISION
    if rec["timed_out"] or rec["leftover_pids"]:
        return EXIT_INFRASTRUCTURE
    if rec["exit_code"] != 0:
        return EXIT_BUILD if build else EXIT_TESTS
    return EXIT_OK


def run_suite(commands: Sequence[str], devices: Sequence[int], nvml, poll_s: float, log, timeout_s: float = 0.0, phases: Optional[list] = None,
              cancelled=lambda: False) -> int:
    env = child_environment(None, devices)
    for cmd in commands:
        log(f"[gate] run: {cmd}")
        rec = run_command(cmd, env, devices, nvml, poll_s, timeout_s, log, cancelled)
        code = classify(rec)
        rec.update(phase="suite", result=code)
        if phases is not None:
            phases.append(rec)
        if code == EXIT_COLLISION:
            log(f"[gate] collision: foreign processes on gated GPUs {rec['collisions']}")
        elif code == EXIT_INFRASTRUCTURE:
            log(f"[gate] infrastructure: timed out={rec['timed_out']}, left behind {rec['leftover_pids']}: {cmd}")
        elif code == EXIT_TESTS:
            log(f"[gate] command failed with {rec['exit_code']}: {cmd}")
        if code != EXIT_OK:
            return code
    return EXIT_OK


def format_report(report: Dict[str, object]) -> str:
    lines = [f"[gate] result {report['exit_code']} ({report['failure_class']}) on GPUs {report.get('devices')}"]
    for ph in report["phases"]:
        lines.append(f"[gate]   {ph['phase']}: {ph.get('seconds', 0):.1f} s, exit {ph.get('exit_code')}, result {ph['result']}: {str(ph.get('command', ''))[:100]}")
    return "\n".join(lines)


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
    ap.add_argument("--timeout-s", type=float, default=0.0, help="time limit of every command (0: none)")
    ap.add_argument("--expect-sha", default="", help="the commit this run gates; another head in --source ends the run as obsolete")
    ap.add_argument("--source", default=".", help="the checked-out tree (for --expect-sha)")
    ap.add_argument("--report", default="", help="file for the JSON report")
    args = ap.parse_args(argv)
    log = lambda m: print(m, flush=True)
    suite = args.suite or [
        f"{sys.executable} -m pytest tests -q -m gpu",
        f"{sys.executable} bench.py --steps 20 --warmup 5",
    ]
    report: Dict[str, object] = {"phases": [], "devices": None, "started": time.time()}
    state = {"cancelled": False}

    def on_signal(signum, frame):
        state["cancelled"] = True

    previous = {}
    for sig in (signal.SIGINT, signal.SIGTERM):
        try:
            previous[sig] = signal.signal(sig, on_signal)
        except ValueError:                             # not the main thread (tests): signals stay as they are
            pass
    cancelled = lambda: state["cancelled"]

    def finish(code: int) -> int:
        report["exit_code"] = code
        report["failure_class"] = FAILURE_CLASS.get(code, "infrastructure")
        report["seconds"] = round(time.time() - report["started"], 3)
        log(format_report(report))
        if args.report:
            with open(args.report, "w") as f:
                json.dump(report, f, indent=1)
        for sig, handler in previous.items():
            signal.signal(sig, handler)
        return code

    try:
        if args.expect_sha:
            problem = verify_sha(args.source, args.expect_sha)
            report["phases"].append({"phase": "source", "command": f"head of {args.source}", "result": EXIT_OBSOLETE if problem else EXIT_OK, "detail": problem or ""})
            if problem:
                log(f"[gate] obsolete: {problem}")
                return finish(EXIT_OBSOLETE)
        nvml = FakeNvml(args.nvml.split(":", 1)[1]) if args.nvml.startswith("fake:") else None
        if not args.skip_build:
            log(f"[gate] build: {args.build}")
            rec = run_command(args.build, child_environment(), (), nvml, min(args.poll_s, 1.0), args.timeout_s, log, cancelled)
            code = classify(rec, build=True)
            rec.update(phase="build", result=code)
            report["phases"].append(rec)
            if code != EXIT_OK:
                return finish(code)
        if nvml is None:
            nvml = Nvml()
        devices = wait_for_idle(nvml, args.gpus, args.max_used_mib, args.wait_s, args.poll_s)
        if cancelled():
            return finish(EXIT_INTERRUPTED)
        if devices is None:
            log(f"[gate] fewer than {args.gpus} idle GPUs within {args.wait_s:.0f} s")
            report["phases"].append({"phase": "wait", "command": f"{args.gpus} idle GPUs", "result": EXIT_NO_DEVICES})
            return finish(EXIT_NO_DEVICES)
        log(f"[gate] gated GPUs: {devices}")
        report["devices"] = devices
        return finish(run_suite(suite, devices, nvml, args.poll_s, log, args.timeout_s, report["phases"], cancelled))
    except KeyboardInterrupt:
        return finish(EXIT_INTERRUPTED)


if __name__ == "__main__":
    sys.exit(main())
