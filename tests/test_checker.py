"""Protocol checker: clean protocols pass for every op, scheduler and rank count; each injected
single-step fault is reported as the finding class it stands for."""
import json
import subprocess
from pathlib import Path

import pytest

from tilexr_b200.tools import checker

OPS = ["allgather", "allreduce", "alltoall", "ep_dispatch", "ep_combine"]


@pytest.mark.parametrize("op", OPS)
@pytest.mark.parametrize("scheduler", ["serial", "round_robin"])
@pytest.mark.parametrize("ranks,servers", [(2, 1), (4, 2), (8, 2)])
def test_clean_protocols_pass(op, scheduler, ranks, servers):
    rep = checker.run_case(op=op, rank_size=ranks, server_count=servers, count=ranks * 96, tile_elems=64, launches=4,
                           moe_expert_num=ranks * 2, bs=6, h=8, top_k=3, scheduler=scheduler)
    assert rep["passed"], rep["summary"]
    assert rep["findings"] == []


@pytest.mark.parametrize("injection,expected", [
    ("inject_read_before_copy", "READ_BEFORE_COPY"),
    ("inject_stale_magic", "FLAG_STALE_MAGIC"),
    ("inject_missing_flag", "FLAG_NO_PRODUCER"),
    ("inject_peer_user_read", "DIRECT_PEER_USER_BUFFER"),
    ("inject_pipe_wait", "PIPE_WAIT_NO_PRODUCER"),
    ("inject_deadlock", "DEADLOCK"),
    ("inject_corrupt_output", "OUTPUT_MISMATCH"),
])
def test_each_injection_is_found(injection, expected):
    rep = checker.run_case(op="allgather", rank_size=2, count=512, tile_elems=128, **{injection: True})
    assert not rep["passed"]
    assert expected in rep["findings"], rep["summary"]


def test_reuse_guard_is_required():
    rep = checker.run_case(op="allgather", rank_size=2, count=256, launches=4, inject_skip_reuse_guard=True)
    assert "BUFFER_LIFETIME" in rep["findings"]


def test_ep_injections():
    rep = checker.run_case(op="ep_dispatch", rank_size=2, moe_expert_num=4, inject_missing_flag=True)
    assert "FLAG_NO_PRODUCER" in rep["findings"] and "EVENT_COVERAGE_GAP" in rep["findings"]
    rep = checker.run_case(op="ep_dispatch", rank_size=2, moe_expert_num=4, inject_read_before_copy=True)
    assert "READ_BEFORE_COPY" in rep["findings"]
    rep = checker.run_case(op="ep_combine", rank_size=2, moe_expert_num=4, inject_missing_flag=True)
    assert "FLAG_NO_PRODUCER" in rep["findings"]


def test_trace_round_trip_and_tampering():
    rep = checker.run_case(op="allgather", rank_size=2, count=256, tile_elems=128)
    trace = rep["events_jsonl"]
    assert checker.check_trace(trace) == []
    # drop every flag store of rank 0: rank 1's waits lose their producer
    lines = [l for l in trace.splitlines() if not ('"FlagStore"' in l and '"rank": 0,' in l and '"slot": 0,' in l)]
    kinds = {f[0] for f in checker.check_trace("\n".join(lines))}
    assert "FLAG_NO_PRODUCER" in kinds
    assert {f[0] for f in checker.check_trace("not json\n")} == {"UNSUPPORTED_API"}


def test_unsupported_case():
    rep = checker.run_case(op="gather", rank_size=2)
    assert rep["findings"] == ["UNSUPPORTED_API"]


def test_cli_writes_reports(tmp_path):
    from tilexr_b200 import _build

    exe = _build.build_checker_cli(verbose=False)  # rebuilt when checker sources are newer
    assert exe.exists()
    r = subprocess.run([str(exe), "--op", "allreduce", "--ranks", "4", "--count", "1024", "--launches", "3", "--out", str(tmp_path)],
                       capture_output=True, text=True)
    assert r.returncode == 0 and "RESULT: PASS" in r.stdout
    report = json.loads((tmp_path / "checker_report.json").read_text())
    assert report["passed"] is True and report["rank_size"] == 4
    assert (tmp_path / "summary.txt").exists() and (tmp_path / "events.jsonl").exists()
    r = subprocess.run([str(exe), "--op", "allgather", "--inject-deadlock"], capture_output=True, text=True)
    assert r.returncode == 1 and "FATAL DEADLOCK" in r.stdout
    r = subprocess.run([str(exe), "--trace", str(tmp_path / "events.jsonl")], capture_output=True, text=True)
    assert r.returncode == 0


def test_installed_traces_are_recorded_judged_and_covered(tmp_path):
    """An installed trace: host kernels run between two real processes under the recorder, the checker judges the events and
    the manifest's event coverage is met; a recording that lost one kind of event fails the coverage check (reference:
    tools/checker/installed_traces/*_trace_manifest.json, `--verify-installed-traces`)."""
    import json

    from tilexr_b200.tools import checker

    names = {m["name"] for m in checker.load_manifests()}
    assert {"host_all_gather", "host_all_reduce", "host_ep_dispatch_combine", "host_moonep_stages"} <= names
    for m in checker.load_manifests():
        assert m["recipe"] in checker.RECIPES and m["ranks"] >= 2 and m["required_event_coverage"]
    rows = checker.verify_installed_traces("host_all_reduce", keep_dir=str(tmp_path))
    assert len(rows) == 1 and rows[0]["ok"] and rows[0]["events"] > 10 and rows[0]["findings"] == []
    manifest = checker.load_manifests("host_all_reduce")[0]
    paths = [str(tmp_path / "host_all_reduce" / f"rank{r}.jsonl") for r in range(2)]
    assert checker.missing_coverage(manifest, paths) == []
    # rank 1's recorder "lost" its waits
    lines = [l for l in open(paths[1]) if json.loads(l)["kind"] != "FlagWait"]
    open(paths[1], "w").writelines(lines)
    gaps = checker.missing_coverage(manifest, paths)
    assert gaps and all(g["rank"] == 1 and g["kind"] == "FlagWait" and g["have"] == 0 for g in gaps)
    with pytest.raises(ValueError):
        checker.load_manifests("no_such_trace")
    with pytest.raises(ValueError):
        checker.record_installed_trace("no_such_recipe", 2, str(tmp_path / "x"))
    # the MoonEP stages by plan between three processes: two plans over the same windows
    rows = checker.verify_installed_traces("host_moonep_stages")
    assert len(rows) == 1 and rows[0]["ok"] and rows[0]["ranks"] == 3 and rows[0]["findings"] == [], rows


def test_zero_copy_gather_needs_the_entry_meeting():
    """Tiles that go straight into the peers' own output tensors: clean with the entry meeting (several ranks, several launches,
    both schedulers), and a BUFFER_LIFETIME finding when one producer writes without having waited for its peer's entry."""
    for ranks, sched in ((2, "round_robin"), (4, "serial"), (4, "round_robin")):
        rep = checker.run_case(op="allgather", rank_size=ranks, count=512, tile_elems=128, launches=3, zero_copy=True, scheduler=sched)
        assert rep["passed"] and rep["outputs_match"], rep["summary"]
    rep = checker.run_case(op="allgather", rank_size=2, count=512, tile_elems=128, zero_copy=True, inject_skip_entry_meeting=True)
    assert not rep["passed"] and "BUFFER_LIFETIME" in rep["findings"], rep["summary"]
    assert "entered this launch" in rep["summary"]
    # the window path has no such meeting and needs none
    assert checker.run_case(op="allgather", rank_size=2, count=512, tile_elems=128, launches=3)["passed"]
    cli = Path(__file__).resolve().parent.parent / "tilexr_b200" / "bin" / "tilexr_checker"
    if cli.exists():
        ok = subprocess.run([str(cli), "--op", "allgather", "--ranks", "2", "--zero-copy"], capture_output=True, text=True)
        bad = subprocess.run([str(cli), "--op", "allgather", "--ranks", "2", "--zero-copy", "--inject-skip-entry-meeting"], capture_output=True, text=True)
        assert ok.returncode == 0 and bad.returncode != 0 and "BUFFER_LIFETIME" in bad.stdout


def test_two_writers_of_the_same_bytes_are_reported():
    """AMBIGUOUS_SOURCE: ranks 0 and 2 both store into overlapping bytes of rank 1's window in one launch; slices that only
    touch, other launches and other regions are fine."""
    import json

    from tilexr_b200.tools import checker

    def ev(i, kind, rank, peer, offset=0, nbytes=0, magic=1, slot=0, role="comm_data"):
        return {"id": i, "kind": kind, "rank": rank, "peer": peer, "block": 0, "role": role, "slot": slot, "pipe": -1, "magic": magic,
                "offset": offset, "bytes": nbytes, "satisfied": 1, "source": "test"}

    def run(copies):
        events = [ev(1, "RankStart", 0, -1, role="none"), ev(2, "RankStart", 2, -1, role="none")]
        events += [ev(10 + i, "Copy", *c) for i, c in enumerate(copies)]
        events += [ev(90, "RankEnd", 0, -1, role="none"), ev(91, "RankEnd", 2, -1, role="none")]
        return [f[0] for f in checker.check_trace("\n".join(json.dumps(e) for e in events) + "\n")]

    assert run([(0, 1, 0, 128), (2, 1, 128, 128)]) == []                               # the slices touch and do not overlap
    assert run([(0, 1, 0, 128), (2, 1, 64, 128)]) == ["AMBIGUOUS_SOURCE"]
    assert run([(0, 1, 0, 256), (0, 1, 300, 8), (2, 1, 200, 8)]) == ["AMBIGUOUS_SOURCE"]   # inside an earlier, longer store
    assert run([(0, 1, 0, 128), (2, 1, 64, 128, 2)]) == []                             # another launch (the other half of the window)
    assert run([(0, 1, 0, 128), (2, 1, 64, 128, 1, 5)]) == []                          # another region
    assert run([(0, 1, 0, 128), (0, 1, 64, 128)]) == []                                # one writer may store twice
    assert run([(0, 1, 0, 128), (2, 1, 64, 128), (2, 1, 100, 8), (0, 1, 90, 8)]) == ["AMBIGUOUS_SOURCE"]   # one finding per pair of writers and owner


def test_shared_slice_injection_is_found_in_the_modelled_all_gather():
    from tilexr_b200.tools import checker

    good = checker.run_case(op="allgather", rank_size=3, count=512, tile_elems=128)
    assert good["passed"], good["summary"]
    rep = checker.run_case(op="allgather", rank_size=3, count=512, tile_elems=128, inject_shared_slice=True)
    assert not rep["passed"] and "AMBIGUOUS_SOURCE" in rep["findings"], rep["summary"]
    # with two ranks there is no third writer: the switch changes nothing
    assert checker.run_case(op="allgather", rank_size=2, count=512, tile_elems=128, inject_shared_slice=True)["passed"]
