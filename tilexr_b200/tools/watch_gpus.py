"""Watch the GPUs of a node while a job runs: utilisation, memory, SM clock against its maximum, power, the reasons the
clock is held back, and who is on the device (the reference ships shell watchers for its NPUs: scripts/watch.sh).

Everything is READ through NVML; no clock, power limit or mode of any GPU is touched.  One line per GPU and sample, as a
table or as CSV (`--csv FILE`), which is the form `bench.py` and the perf tools cite beside a number.

    python -m tilexr_b200.tools.watch_gpus --interval 1 --count 30
    python -m tilexr_b200.tools.watch_gpus --csv clocks.csv --interval 0.2 --count 100 --gpus 0,1
"""
from __future__ import annotations

import argparse
import csv
import json
import sys
import time
from typing import Dict, List, Optional, Sequence

# names of the bits of NVML's "clocks event reasons" word, lowest bit first (nvml.h)
REASON_BITS = ("gpu_idle", "applications_clocks_setting", "sw_power_cap", "hw_slowdown", "sync_boost", "sw_thermal_slowdown",
               "hw_thermal_slowdown", "hw_power_brake_slowdown", "display_clock_setting")
BAD_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "hw_power_brake_slowdown")
FIELDS = ("time", "index", "util_pct", "mem_used_mib", "mem_total_mib", "sm_mhz", "sm_max_mhz", "power_w", "reasons", "pids")


def decode_reasons(word: int) -> List[str]:
    return [name for bit, name in enumerate(REASON_BITS) if word & (1 << bit)]


class NvmlReader:
    """One sample = a list of dicts with FIELDS[1:]."""

    def __init__(self):
        import pynvml

        pynvml.nvmlInit()
        self.nv = pynvml

    def sample(self, gpus: Optional[Sequence[int]] = None) -> List[Dict[str, object]]:
        nv = self.nv
        out = []
        for i in range(nv.nvmlDeviceGetCount()):
            if gpus is not None and i not in gpus:
                continue
            h = nv.nvmlDeviceGetHandleByIndex(i)

            def get(fn, *a, default=0):
                try:
                    return fn(h, *a)
                except nv.NVMLError:
                    return default

            mem = get(nv.nvmlDeviceGetMemoryInfo, default=None)
            util = get(nv.nvmlDeviceGetUtilizationRates, default=None)
            reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
            procs = get(nv.nvmlDeviceGetComputeRunningProcesses, default=[])
            out.append({"index": i, "util_pct": 0 if util is None else int(util.gpu),
                        "mem_used_mib": 0 if mem is None else int(mem.used >> 20), "mem_total_mib": 0 if mem is None else int(mem.total >> 20),
                        "sm_mhz": int(get(nv.nvmlDeviceGetClockInfo, nv.NVML_CLOCK_SM)), "sm_max_mhz": int(get(nv.nvmlDeviceGetMaxClockInfo, nv.NVML_CLOCK_SM)),
                        "power_w": round(get(nv.nvmlDeviceGetPowerUsage) / 1000.0, 1), "reasons": decode_reasons(int(get(reasons_fn))),
                        "pids": sorted(p.pid for p in procs)})
        return out


class FakeReader:
    """Plays back samples from a JSON file (a list of samples); the last one repeats."""

    def __init__(self, path: str):
        self.samples = json.loads(open(path).read())
        self.calls = 0

    def sample(self, gpus: Optional[Sequence[int]] = None) -> List[Dict[str, object]]:
        s = self.samples[min(self.calls, len(self.samples) - 1)]
        self.calls += 1
        return [d for d in s if gpus is None or d["index"] in gpus]


def summarize(samples: Sequence[Sequence[Dict[str, object]]]) -> List[Dict[str, object]]:
    """Per GPU over all samples: median and lowest SM clock under load (utilisation above 50 %), the maximum clock, the
    highest power, every reason seen, and whether a reason that invalidates a measurement was among them."""
    per: Dict[int, List[Dict[str, object]]] = {}
    for s in samples:
        for d in s:
            per.setdefault(int(d["index"]), []).append(d)
    out = []
    for idx, rows in sorted(per.items()):
        busy = sorted(int(r["sm_mhz"]) for r in rows if int(r["util_pct"]) > 50) or sorted(int(r["sm_mhz"]) for r in rows)
        seen = sorted({name for r in rows for name in r["reasons"]})
        out.append({"index": idx, "samples": len(rows), "sm_mhz_median_under_load": busy[len(busy) // 2], "sm_mhz_min_under_load": busy[0],
                    "sm_max_mhz": max(int(r["sm_max_mhz"]) for r in rows), "power_w_max": max(float(r["power_w"]) for r in rows),
                    "reasons": seen, "rejects_measurement": any(name in BAD_REASONS for name in seen)})
    return out


def format_row(t: float, d: Dict[str, object]) -> str:
    return (f"{t:8.1f}s gpu{d['index']}: {d['util_pct']:3d}% {d['mem_used_mib']:7d}/{d['mem_total_mib']} MiB  {d['sm_mhz']:4d}/{d['sm_max_mhz']} MHz "
            f"{d['power_w']:6.1f} W  [{','.join(d['reasons']) or '-'}]  pids {d['pids'] or '-'}")


def watch(reader, interval: float, count: int, gpus: Optional[Sequence[int]], csv_path: str = "", out=sys.stdout, sleep=time.sleep,
          now=time.time) -> List[List[Dict[str, object]]]:
    samples = []
    writer = None
    fh = None
    if csv_path:
        fh = open(csv_path, "w", newline="")
        writer = csv.writer(fh)
        writer.writerow(FIELDS)
    t0 = now()
    try:
        for n in range(count):
            s = reader.sample(gpus)
            samples.append(s)
            t = now() - t0
            for d in s:
                if writer is not None:
                    writer.writerow([f"{t:.3f}", d["index"], d["util_pct"], d["mem_used_mib"], d["mem_total_mib"], d["sm_mhz"], d["sm_max_mhz"], d["power_w"],
                                     "|".join(d["reasons"]), "|".join(str(p) for p in d["pids"])])
                else:
                    print(format_row(t, d), file=out)
            if n + 1 < count:
                sleep(interval)
    except KeyboardInterrupt:
        pass
    finally:
        if fh is not None:
            fh.close()
    return samples


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--interval", type=float, default=1.0)
    p.add_argument("--count", type=int, default=10)
    p.add_argument("--gpus", default="", help="comma-separated indices (default: all)")
    p.add_argument("--csv", default="")
    p.add_argument("--nvml", default="real", help="fake:<json file> plays back recorded samples")
    p.add_argument("--summary", action="store_true", help="print a per-GPU summary as JSON at the end")
    a = p.parse_args(argv)
    gpus = [int(x) for x in a.gpus.split(",") if x.strip()] or None
    reader = FakeReader(a.nvml.split(":", 1)[1]) if a.nvml.startswith("fake:") else NvmlReader()
    samples = watch(reader, a.interval, a.count, gpus, a.csv)
    if a.summary:
        print(json.dumps(summarize(samples)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
