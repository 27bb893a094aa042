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
