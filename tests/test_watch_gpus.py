"""The read-only GPU watcher on recorded samples: rows, CSV, the per-GPU summary and the verdict on throttle reasons."""
import csv
import io
import json

from tilexr_b200.tools import watch_gpus as wg


def _gpu(i, util, mhz, reasons=(), pids=(), power=700.0):
    return {"index": i, "util_pct": util, "mem_used_mib": 1000 * (i + 1), "mem_total_mib": 183359, "sm_mhz": mhz, "sm_max_mhz": 1965, "power_w": power,
            "reasons": list(reasons), "pids": list(pids)}


def test_watch_rows_csv_and_summary(tmp_path):
    samples = [[_gpu(0, 0, 345, ["gpu_idle"]), _gpu(1, 0, 345, ["gpu_idle"])],
               [_gpu(0, 99, 1965, [], [41]), _gpu(1, 98, 1320, ["sw_power_cap"], [42], 995.0)],
               [_gpu(0, 99, 1905, [], [41]), _gpu(1, 97, 1100, ["sw_power_cap", "hw_thermal_slowdown"], [42], 990.0)]]
    f = tmp_path / "s.json"
    f.write_text(json.dumps(samples))
    clock = {"t": 0.0}
    out = io.StringIO()
    got = wg.watch(wg.FakeReader(str(f)), 0.5, 3, None, out=out, sleep=lambda s: clock.__setitem__("t", clock["t"] + s), now=lambda: clock["t"])
    lines = out.getvalue().strip().splitlines()
    assert len(got) == 3 and len(lines) == 6 and "gpu1:  98%" in lines[3] and "[sw_power_cap]" in lines[3] and "pids [42]" in lines[3]
    summary = {s["index"]: s for s in wg.summarize(got)}
    assert summary[0]["sm_mhz_median_under_load"] == 1965 and summary[0]["sm_mhz_min_under_load"] == 1905 and not summary[0]["rejects_measurement"]
    assert summary[1]["rejects_measurement"] and "hw_thermal_slowdown" in summary[1]["reasons"] and summary[1]["power_w_max"] == 995.0
    # CSV, one GPU only
    path = tmp_path / "c.csv"
    assert wg.main(["--nvml", f"fake:{f}", "--interval", "0", "--count", "3", "--gpus", "1", "--csv", str(path)]) == 0
    rows = list(csv.reader(open(path)))
    assert rows[0] == list(wg.FIELDS) and len(rows) == 4 and all(r[1] == "1" for r in rows[1:]) and rows[3][8] == "sw_power_cap|hw_thermal_slowdown"
    assert wg.decode_reasons(0b1000101) == ["gpu_idle", "sw_power_cap", "hw_thermal_slowdown"] and wg.decode_reasons(0) == []
