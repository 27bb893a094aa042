"""The CI hardware gate against a scripted NVML: idle detection, wait budget, collision detection, exit codes."""
import importlib.util
import json
import pathlib
import sys

ROOT = pathlib.Path(__file__).resolve().parent.parent
spec = importlib.util.spec_from_file_location("gate", ROOT / "ci" / "gate.py")
gate = importlib.util.module_from_spec(spec)
spec.loader.exec_module(gate)


def _dev(i, used=10, pids=()):
    return {"index": i, "used_mib": used, "pids": list(pids)}


def test_idle_devices_skip_busy_memory_and_foreign_processes():
    snap = [_dev(0), _dev(1, used=5000), _dev(2, pids=[77]), _dev(3, pids=[5])]
    assert gate.idle_devices(snap, 1024) == [0]
    assert gate.idle_devices(snap, 1024, own_pids=[5]) == [0, 3]


def test_wait_for_idle_polls_until_enough_or_gives_up(tmp_path):
    states = [[_dev(0, pids=[9]), _dev(1)], [_dev(0, pids=[9]), _dev(1)], [_dev(0), _dev(1)]]
    p = tmp_path / "nvml.json"
    p.write_text(json.dumps(states))
    clock = {"t": 0.0}
    sleep = lambda s: clock.__setitem__("t", clock["t"] + s)
    assert gate.wait_for_idle(gate.FakeNvml(str(p)), 2, 1024, budget_s=100, poll_s=10, sleep=sleep, now=lambda: clock["t"]) == [0, 1]
    assert clock["t"] == 20
    clock["t"] = 0.0
    busy = tmp_path / "busy.json"
    busy.write_text(json.dumps([[_dev(0, pids=[9])]]))
    assert gate.wait_for_idle(gate.FakeNvml(str(busy)), 1, 1024, budget_s=30, poll_s=10, sleep=sleep, now=lambda: clock["t"]) is None


def test_gate_exit_codes(tmp_path):
    idle = tmp_path / "idle.json"
    idle.write_text(json.dumps([[_dev(0), _dev(1)]]))
    base = ["--nvml", f"fake:{idle}", "--gpus", "2", "--poll-s", "0.05", "--wait-s", "1"]
    ok = f"{sys.executable} -c pass"
    assert gate.main(base + ["--skip-build", "--suite", ok]) == gate.EXIT_OK
    assert gate.main(base + ["--build", f"{sys.executable} -c 'raise SystemExit(3)'", "--suite", ok]) == gate.EXIT_BUILD
    assert gate.main(base + ["--skip-build", "--suite", f"{sys.executable} -c 'raise SystemExit(1)'"]) == gate.EXIT_TESTS
    assert gate.main(["--nvml", f"fake:{idle}", "--gpus", "4", "--poll-s", "0.05", "--wait-s", "0.2", "--skip-build", "--suite", ok]) == gate.EXIT_NO_DEVICES
    # a stranger appears on a gated GPU while the suite runs
    collide = tmp_path / "collide.json"
    collide.write_text(json.dumps([[_dev(0), _dev(1)], [_dev(0, pids=[999999]), _dev(1)]]))
    slow = f"{sys.executable} -c 'import time; time.sleep(0.5)'"
    assert gate.main(["--nvml", f"fake:{collide}", "--gpus", "2", "--poll-s", "0.05", "--wait-s", "1", "--skip-build", "--suite", slow]) == gate.EXIT_COLLISION


def test_time_limit_leftovers_source_check_report_and_environment(tmp_path):
    """A command that outlives its limit is ended as a process group; one that returns but leaves a child behind is an
    infrastructure failure and the child is ended too; another head than the gated commit makes the run obsolete; the
    report lists the phases; credentials do not reach the commands (reference: scripts/ci/control/gate.py:30-52, 699-745,
    1039-1068)."""
    import os
    import subprocess
    import time

    idle = tmp_path / "idle.json"
    idle.write_text(json.dumps([[_dev(0)]]))
    base = ["--nvml", f"fake:{idle}", "--gpus", "1", "--poll-s", "0.05", "--wait-s", "1", "--skip-build"]
    report = tmp_path / "report.json"
    sleeper = f"{sys.executable} -c 'import time; time.sleep(30)'"
    t0 = time.time()
    assert gate.main(base + ["--suite", sleeper, "--timeout-s", "0.3", "--report", str(report)]) == gate.EXIT_INFRASTRUCTURE
    assert time.time() - t0 < 15
    rep = json.loads(report.read_text())
    assert rep["failure_class"] == "infrastructure" and rep["phases"][-1]["timed_out"] and rep["devices"] == [0]
    # returns at once, leaves a sleeping child in its session
    pidfile = tmp_path / "child.pid"
    script = tmp_path / "leaver.py"
    script.write_text("import subprocess, sys\n"
                      "p = subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(30)'])\n"
                      f"open(r'{pidfile}', 'w').write(str(p.pid))\n")
    leaver = f"{sys.executable} {script}"
    assert gate.main(base + ["--suite", leaver, "--report", str(report)]) == gate.EXIT_INFRASTRUCTURE
    child = int(pidfile.read_text())
    rep = json.loads(report.read_text())
    assert rep["phases"][-1]["leftover_pids"]
    time.sleep(0.3)
    try:
        os.kill(child, 0)
        state = open(f"/proc/{child}/stat").read().rsplit(")", 1)[1].split()[0]
        assert state == "Z"                               # at most a zombie waiting for its reaper: it was ended
    except (ProcessLookupError, FileNotFoundError):
        pass
    # the source check
    assert gate.verify_sha("x", "zzzz") is not None and gate.verify_sha("x", "abc1234", run_git=lambda p: "abc1234ffff") is None
    assert "is at" in gate.verify_sha("x", "abc1234", run_git=lambda p: "def5678aaaa")
    repo = tmp_path / "repo"
    repo.mkdir()
    subprocess.run(["git", "init", "-q", str(repo)], check=True)
    subprocess.run(["git", "-C", str(repo), "-c", "user.email=a@b", "-c", "user.name=n", "commit", "-q", "--allow-empty", "-m", "x"], check=True)
    head = subprocess.run(["git", "-C", str(repo), "rev-parse", "HEAD"], capture_output=True, text=True, check=True).stdout.strip()
    ok = f"{sys.executable} -c pass"
    assert gate.main(base + ["--suite", ok, "--expect-sha", head[:10], "--source", str(repo)]) == gate.EXIT_OK
    assert gate.main(base + ["--suite", ok, "--expect-sha", "0" * 40, "--source", str(repo), "--report", str(report)]) == gate.EXIT_OBSOLETE
    assert json.loads(report.read_text())["failure_class"] == "obsolete"
    # environment of the commands
    env = gate.child_environment({"PATH": "/bin", "GITHUB_TOKEN": "t", "MY_SECRET_THING": "s", "Api_Key": "k", "HOME": "/h"}, [2, 5])
    assert env == {"PATH": "/bin", "HOME": "/h", "CUDA_VISIBLE_DEVICES": "2,5"}
    # cancellation ends the running command and reports 130
    flag = {"n": 0}

    def cancelled():
        flag["n"] += 1
        return flag["n"] > 2

    rec = gate.run_command(sleeper, gate.child_environment(), (), None, 0.05, 0.0, lambda m: None, cancelled)
    assert rec["cancelled"] and gate.classify(rec) == gate.EXIT_INTERRUPTED and rec["seconds"] < 15
