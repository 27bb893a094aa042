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
