"""What the compiler made of every kernel, without a GPU: registers, spills, stack, static shared memory and barriers per
entry function, from `ptxas -v` on the library's `.cu` sources with the flags of the in-tree build; and from those, how many
blocks of a given size fit on an SM.  (The reference inspects its kernels off the hardware with a vendor simulator:
op-simulator/README.md.  Nothing is disassembled here; the figures are the ones `ptxas` prints.)

    python -m tilexr_b200.tools.kernel_report                              # every source, a table per file
    python -m tilexr_b200.tools.kernel_report csrc/gemm/gemm_tcgen05_pair.cu --threads 192 --dynamic-smem 221184
    python -m tilexr_b200.tools.kernel_report --json report.json --fail-on-spills

A spill in a hot kernel is a finding (`--fail-on-spills` makes it the exit status: a host check for CI).  Kernel names are
shortened to the function name; `--full-names` keeps the demangled signature.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import json
import re
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path
from typing import Dict, List, Optional, Sequence

# sm_100a, per SM (the CUDA occupancy rules for compute capability 10.0)
REGISTERS_PER_SM = 65536
MAX_THREADS_PER_SM = 2048
MAX_BLOCKS_PER_SM = 32
SHARED_PER_SM = 228 * 1024            # of which 1 KB per resident block is the system's
SHARED_PER_BLOCK_MAX = 227 * 1024
REGISTER_ALLOC_UNIT = 8               # registers per thread are rounded up to a multiple of 8, allocated per warp

_ENTRY = re.compile(r"Compiling entry function '([^']+)' for '([^']+)'")
_STACK = re.compile(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads")
_USED = re.compile(r"Used (\d+) registers(.*)")
_BARRIERS = re.compile(r"used (\d+) barriers")
_SMEM = re.compile(r"(\d+) bytes smem")
_CMEM = re.compile(r"(\d+) bytes cmem\[(\d+)\]")


def parse_ptxas(text: str) -> List[Dict[str, object]]:
    """One record per entry function of a `ptxas -v` log (device functions that ptxas lists without an entry line are skipped)."""
    out: List[Dict[str, object]] = []
    cur: Optional[Dict[str, object]] = None
    for line in text.splitlines():
        m = _ENTRY.search(line)
        if m:
            cur = {"mangled": m.group(1), "arch": m.group(2), "registers": 0, "stack_bytes": 0, "spill_store_bytes": 0, "spill_load_bytes": 0,
                   "barriers": 0, "static_smem_bytes": 0, "const_bytes": 0}
            out.append(cur)
            continue
        if cur is None:
            continue
        m = _STACK.search(line)
        if m:
            cur["stack_bytes"], cur["spill_store_bytes"], cur["spill_load_bytes"] = (int(g) for g in m.groups())
            continue
        m = _USED.search(line)
        if m:
            cur["registers"] = int(m.group(1))
            rest = m.group(2)
            b = _BARRIERS.search(rest)
            cur["barriers"] = int(b.group(1)) if b else 0
            s = _SMEM.search(rest)
            cur["static_smem_bytes"] = int(s.group(1)) if s else 0
            cur["const_bytes"] = sum(int(c.group(1)) for c in _CMEM.finditer(rest))
            cur = None                                   # "Used ..." closes an entry's block
    return out


def demangle(names: Sequence[str]) -> List[str]:
    tool = shutil.which("c++filt")
    if tool is None or not names:
        return list(names)
    r = subprocess.run([tool], input="\n".join(names) + "\n", capture_output=True, text=True)
    got = r.stdout.splitlines()
    return got if r.returncode == 0 and len(got) == len(names) else list(names)


def short_name(demangled: str) -> str:
    """`TileXR::(anonymous namespace)::Kernel<true, 2>(Args const*)` -> `Kernel<true, 2>`."""
    depth, cut = 0, len(demangled)
    for i, ch in enumerate(demangled):                   # the parameter list opens at the first '(' outside template brackets
        if ch == "<":
            depth += 1
        elif ch == ">":
            depth -= 1
        elif ch == "(" and depth == 0 and not demangled.startswith("(anonymous namespace)", i):
            cut = i
            break
    head = demangled[:cut].strip()
    depth, start = 0, 0
    for i in range(len(head) - 1):                       # the last "::" outside template brackets
        if head[i] == "<":
            depth += 1
        elif head[i] == ">":
            depth -= 1
        elif depth == 0 and head[i:i + 2] == "::":
            start = i + 2
    name = head[start:]
    return name.split(" ")[-1] if "<" not in name else name[name.rfind(" ", 0, name.find("<")) + 1:]


def blocks_per_sm(registers: int, threads: int, static_smem: int, dynamic_smem: int = 0) -> Dict[str, object]:
    """Resident blocks of `threads` threads per SM and which resource sets the limit."""
    if threads <= 0 or threads > 1024:
        raise ValueError("threads per block must be in 1..1024")
    warps = (threads + 31) // 32
    regs_per_thread = max(REGISTER_ALLOC_UNIT, (registers + REGISTER_ALLOC_UNIT - 1) // REGISTER_ALLOC_UNIT * REGISTER_ALLOC_UNIT)
    by_regs = REGISTERS_PER_SM // (regs_per_thread * 32 * warps)
    by_threads = MAX_THREADS_PER_SM // (warps * 32)
    smem = static_smem + dynamic_smem
    if smem > SHARED_PER_BLOCK_MAX:
        return {"blocks": 0, "limit": "shared memory per block", "warps_per_sm": 0, "occupancy": 0.0}
    limits = {"registers": by_regs, "threads": by_threads, "blocks": MAX_BLOCKS_PER_SM}
    if smem > 0:
        limits["shared memory"] = SHARED_PER_SM // (smem + 1024)
    which = min(limits, key=lambda k: limits[k])
    n = limits[which]
    return {"blocks": n, "limit": which, "warps_per_sm": n * warps, "occupancy": n * warps * 32 / MAX_THREADS_PER_SM}


def compile_report(source: Path, nvcc: str, flags: Sequence[str], includes: Sequence[Path]) -> List[Dict[str, object]]:
    with tempfile.TemporaryDirectory() as tmp:
        cmd = [nvcc, *flags, "-Xptxas", "-v", *[f"-I{i}" for i in includes], "-c", str(source), "-o", str(Path(tmp) / "out.o")]
        r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{source}: nvcc failed\n{r.stderr[-2000:]}")
    rows = parse_ptxas(r.stderr + r.stdout)
    for row, name in zip(rows, demangle([str(x["mangled"]) for x in rows])):
        row["name"] = name
        row["kernel"] = short_name(name)
        row["source"] = str(source)
    return rows


def render(rows: Sequence[Dict[str, object]], threads: int = 0, dynamic_smem: int = 0, full_names: bool = False) -> str:
    lines = []
    by_file: Dict[str, List[Dict[str, object]]] = {}
    for r in rows:
        by_file.setdefault(str(r["source"]), []).append(r)
    for src, group in by_file.items():
        lines.append(f"### {src}\n")
        head = "| kernel | registers | spill st / ld (B) | stack (B) | static smem (B) | barriers |"
        sep = "|---|---|---|---|---|---|"
        if threads:
            head += f" blocks/SM at {threads} threads | limit |"
            sep += "---|---|"
        lines += [head, sep]
        for r in sorted(group, key=lambda x: -int(x["registers"])):
            cell = f"| `{r['name'] if full_names else r['kernel']}` | {r['registers']} | {r['spill_store_bytes']} / {r['spill_load_bytes']} | {r['stack_bytes']} | {r['static_smem_bytes']} | {r['barriers']} |"
            if threads:
                o = blocks_per_sm(int(r["registers"]), threads, int(r["static_smem_bytes"]), dynamic_smem)
                cell += f" {o['blocks']} | {o['limit']} |"
            lines.append(cell)
        lines.append("")
    return "\n".join(lines)


def spilling(rows: Sequence[Dict[str, object]]) -> List[Dict[str, object]]:
    return [r for r in rows if int(r["spill_store_bytes"]) or int(r["spill_load_bytes"])]


def main(argv=None) -> int:
    from .. import _build

    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("sources", nargs="*", help="`.cu` files (default: every source of the library)")
    p.add_argument("--threads", type=int, default=0, help="also print the resident blocks per SM for blocks of this many threads")
    p.add_argument("--dynamic-smem", type=int, default=0, help="dynamic shared memory per block, for the blocks-per-SM column")
    p.add_argument("--json", default="")
    p.add_argument("--full-names", action="store_true")
    p.add_argument("--fail-on-spills", action="store_true")
    p.add_argument("--jobs", type=int, default=4)
    a = p.parse_args(argv)
    sources = [Path(s) for s in a.sources] or _build._sources()[1]
    with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, a.jobs)) as pool:
        per_file = list(pool.map(lambda s: compile_report(s, _build.NVCC, _build.NVCC_FLAGS, _build.INCLUDES), sources))
    rows = [r for group in per_file for r in group]
    for r in rows:
        try:
            r["source"] = str(Path(str(r["source"])).resolve().relative_to(_build.ROOT))
        except ValueError:
            pass
    print(render(rows, a.threads, a.dynamic_smem, a.full_names))
    bad = spilling(rows)
    print(f"{len(rows)} kernels in {len(sources)} files; {len(bad)} with spills" + ("" if not bad else ": " + ", ".join(sorted({str(r['kernel']) for r in bad}))))
    if a.json:
        with open(a.json, "w") as f:
            json.dump(rows, f, indent=1)
    return 1 if (a.fail_on_spills and bad) else 0


if __name__ == "__main__":
    sys.exit(main())
