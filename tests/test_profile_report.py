"""The profile aggregator on synthetic per-launch traces."""
import json

from tilexr_b200.tools import profile_report

STAGES = [{"id": i, "name": n, "category": 0} for i, n in enumerate(
    ["kernel_total", "chunk_total", "post_sync", "local_input_to_ipc", "flag_poll_wait", "peer_ipc_to_output", "chunk_barrier"])]


def _trace(rank, launch, start, dur, wait):
    recs = [
        {"rank": rank, "core": 0, "stage": 0, "count": 1, "sum": dur, "min": dur, "max": dur, "firstStart": start, "lastEnd": start + dur, "bytes": 1 << 20},
        {"rank": rank, "core": 0, "stage": 3, "count": 4, "sum": dur - wait, "min": 1, "max": 9, "firstStart": start, "lastEnd": start + dur - wait, "bytes": 1 << 20},
        {"rank": rank, "core": 1, "stage": 4, "count": 4, "sum": wait, "min": 1, "max": wait, "firstStart": start, "lastEnd": start + dur, "bytes": 0},
    ]
    return {"schema": "tilexr-perf-trace-v1", "op": "TileXRAllGather", "opType": 3, "dataType": 11, "rank": rank, "rankSize": 2,
            "launchId": launch, "messageBytes": 1 << 20, "blocks": 2, "ticksPerUs": 1000, "incomplete": False, "incompleteReason": "",
            "stages": STAGES, "records": recs}


def test_aggregator_outputs(tmp_path):
    for rank in range(2):
        for launch in range(3):
            d = tmp_path / f"rank{rank}" / f"launch{launch}"
            d.mkdir(parents=True)
            (d / "trace.json").write_text(json.dumps(_trace(rank, launch, 1000 * launch, 50_000 + 10_000 * rank, 30_000)))
    (tmp_path / "rank1" / "launch9").mkdir()
    (tmp_path / "rank1" / "launch9" / "trace.json").write_text("{broken")
    assert profile_report.main([str(tmp_path), "--align"]) == 0
    out = tmp_path / "report"
    index = json.loads((out / "trace_index.json").read_text())
    assert len(index) == 7 and sum("error" in e for e in index) == 1
    good = [e for e in index if "error" not in e]
    assert abs(good[0]["span_us"] - 50.0) < 1e-6 and good[0]["algbw_GBps"] > 20
    text = (out / "analysis.md").read_text()
    assert "slowest: rank 1" in text and "flag_poll_wait" in text and "unreadable trace" in text
    pf = json.loads((out / "perfetto_trace.json").read_text())
    slices = [e for e in pf["traceEvents"] if e["ph"] == "X"]
    assert len(slices) == 18 and min(e["ts"] for e in slices) == 0
    assert "<table>" in (out / "report.html").read_text()


def test_groups_diagnostics_and_prompt(tmp_path):
    """Launches grouped across ranks (span, skew, slowest rank), input problems named (a rank that did not record a launch, a
    launch missing from the sampling pattern, an inconsistent record, a trace without keys), the assistant prompt."""
    for rank in range(2):
        for launch in (0, 2, 4):
            if rank == 1 and launch == 4:
                continue                                  # rank 1 did not record launch 4
            d = tmp_path / f"rank{rank}" / f"launch{launch}"
            d.mkdir(parents=True)
            (d / "trace.json").write_text(json.dumps(_trace(rank, launch, 100_000 * launch + 5_000 * rank, 50_000 + 10_000 * rank, 30_000)))
    bad = _trace(0, 6, 600_000, 50_000, 30_000)
    bad["records"][1]["lastEnd"] = bad["records"][1]["firstStart"] - 10          # ends before it starts
    (tmp_path / "rank0" / "launch6").mkdir()
    (tmp_path / "rank0" / "launch6" / "trace.json").write_text(json.dumps(bad))
    (tmp_path / "rank0" / "launch7").mkdir()
    (tmp_path / "rank0" / "launch7" / "trace.json").write_text(json.dumps({"op": "TileXRAllGather"}))
    assert profile_report.main([str(tmp_path), "--measured-iters", "10", "--sample-every", "2", "--ai-prompt"]) == 0
    out = tmp_path / "report"
    groups = json.loads((out / "launch_groups.json").read_text())
    g0 = [g for g in groups if g["launchId"] == 0][0]
    assert g0["ranks"] == [0, 1] and g0["missing_ranks"] == [] and g0["slowest_rank"] == 1
    assert abs(g0["start_skew_us"] - 5.0) < 1e-6 and abs(g0["group_span_us"] - 65.0) < 1e-6 and abs(g0["end_skew_us"] - 15.0) < 1e-6
    kinds = {}
    for d in json.loads((out / "diagnostics.json").read_text()):
        kinds.setdefault(d["kind"], []).append(d)
    assert any("[1]" in d["detail"] and d["launchId"] == 4 for d in kinds["missing_rank"])
    assert any("ends before it starts" in d["detail"] for d in kinds["inconsistent"])
    assert any("missing keys" in d["detail"] for d in kinds["inconsistent"])
    assert any("[8]" in d["detail"] for d in kinds["missing_launch"])              # 0, 2, 4, 6 recorded; 8 is not
    text = (out / "analysis.md").read_text()
    assert "## Launches across ranks" in text and "## Problems with the input" in text
    prompt = (out / "ai_prompt.md").read_text()
    assert prompt.startswith("# Question") and "missing_rank" in prompt and "| TileXRAllGather |" in prompt
    index = json.loads((out / "trace_index.json").read_text())
    stage = [e for e in index if "error" not in e][0]["stages"]["local_input_to_ipc"]
    assert stage["GBps_per_block_time"] > 0
    assert profile_report.sanitize(_trace(0, 0, 0, 50_000, 30_000)) == [] and profile_report.expected_launch_ids(7, 3) == [0, 3, 6]


def test_clock_offsets_between_hosts_are_estimated_and_removed(tmp_path):
    """Four ranks on two hosts; host 1's timer runs 5 ms ahead.  Every launch ends on all ranks within a few microseconds, so
    the estimate recovers the 5 ms and the Perfetto slices of both hosts line up."""
    skew_ticks = 5_000_000                                    # 5000 us at 1000 ticks per us
    for rank in range(4):
        for launch in range(5):
            d = tmp_path / f"rank{rank}" / f"launch{launch}"
            d.mkdir(parents=True)
            start = 100_000 * launch + 500 * rank + (skew_ticks if rank >= 2 else 0)
            dur = 60_000 - 500 * rank + 700 * (launch % 2) * (rank % 2)          # ends within a microsecond or two of each other
            t = _trace(rank, launch, start, dur, 20_000)
            t["rankSize"] = 4
            (d / "trace.json").write_text(json.dumps(t))
    assert profile_report.main([str(tmp_path), "--ranks-per-host", "2"]) == 0
    out = tmp_path / "report"
    offsets = json.loads((out / "clock_offsets.json").read_text())
    assert set(offsets) == {"0", "1"} and offsets["0"]["offset_us"] == 0.0 and offsets["0"]["launches"] == 5
    assert abs(offsets["1"]["offset_us"] - 5000.0) < 2.0 and offsets["1"]["launches"] == 5 and offsets["1"]["spread_us"] < 2.0
    pf = json.loads((out / "perfetto_trace.json").read_text())
    first = {}
    for e in pf["traceEvents"]:
        if e["ph"] == "X" and e["args"]["launch"] == 3 and e["name"] == "kernel_total":
            first[e["pid"]] = e["ts"]
    assert len(first) == 4 and max(first.values()) - min(first.values()) < 5.0          # 5000 us apart before the correction
    # without the option nothing is shifted and no offsets file is written
    assert profile_report.main([str(tmp_path), "--out", str(tmp_path / "plain")]) == 0
    assert not (tmp_path / "plain" / "clock_offsets.json").exists()
    assert profile_report.estimate_clock_offsets([], 2) == {} and profile_report.estimate_clock_offsets([{"error": "x"}], 0) == {}
