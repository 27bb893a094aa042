"""Architectural invariants checked on the source text (the reference keeps the same kind of
guards: tests/comm/unit/test_tilexr_source_guards.cpp, tests/collectives/unit/
test_tilexr_collectives_kernel_ownership.cpp)."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"


def _sources(*suffixes):
    return [p for p in CSRC.rglob("*") if p.suffix in suffixes]


def test_no_batched_copy_calls_anywhere():
    # the batched async copy entry points of the runtime and driver are never used: one copy per call instead
    batched_copy = "Memcpy" + "Batch" + "Async"
    for p in _sources(".cu", ".cuh", ".h", ".cpp", ".inc"):
        assert batched_copy not in p.read_text(), p


def test_operator_libraries_do_not_reach_into_the_core_runtime():
    # collectives / ep / gemm / moonep consume the C API and the launch service only
    for sub in ("collectives", "ep", "gemm", "moonep", "hostsim"):
        for p in (CSRC / sub).glob("*"):
            if p.suffix in (".cu", ".cpp", ".cuh", ".h"):
                text = p.read_text()
                assert '#include "comm.h"' not in text and "sock_exchange.h" not in text, p


def test_every_device_spin_is_bounded():
    # a `while`/`for(;;)` that polls memory must sit next to a deadline or poll-count check
    pattern = re.compile(r"(for \(;;\)|while \([^)]*ld_(acquire|relaxed|vec16_volatile)[^)]*\))")
    for p in _sources(".cu", ".cuh"):
        text = p.read_text()
        for m in pattern.finditer(text):
            window = text[m.start(): m.start() + 900]
            if m.group(0).startswith("for") and not re.search(r"ld_(acquire|relaxed|vec16_volatile)|MbarTryWait", window[:500]):
                continue      # a host or integer loop, not a memory poll
            assert ("deadline" in window or "budget" in window or "polls" in window), f"{p}: unbounded spin near offset {m.start()}"


def test_no_trap_or_device_assert():
    for p in _sources(".cu", ".cuh"):
        text = p.read_text()
        assert "__trap" not in text, p
        assert not re.search(r"(?<!static_)assert\(", text), p


def test_kernels_target_blackwell_features_where_claimed():
    gemm = (CSRC / "gemm" / "gemm_tcgen05.cu").read_text()
    for needle in ("tcgen05.mma", "tcgen05.alloc", "tcgen05.ld", "tcgen05.commit", "cp.async.bulk.tensor.2d"):
        assert needle in gemm
    assert "wgmma" not in gemm and "mma.sync" not in gemm
    # the fused kernels touch peer memory in the same kernel as the tensor-core tiles
    assert "peerBase[" in gemm and "WaitFlagGE" in gemm


def test_public_headers_cite_the_reference():
    for name in ("tilexr_api.h", "tilexr_collectives.h", "tilexr_ep.h", "tilexr_moonep.h", "tilexr_perf_trace.h"):
        assert "src/" in (CSRC / "include" / name).read_text(), name


def test_no_build_note_names_in_sources():
    banned = ("SURVEY", "VERDICT", "ADVICE.md", "DESIGN.md", "BASELINE.md", "gpurun", "/root/")
    for p in list(_sources(".cu", ".cuh", ".h", ".cpp", ".inc")) + list((ROOT / "tilexr_b200").rglob("*.py")):
        text = p.read_text()
        for b in banned:
            assert b not in text, f"{p} mentions {b}"


def test_no_bulk_load_with_cluster_multicast():
    # a TMA or bulk LOAD with cluster multicast may reach a peer's memory through a tensor map; none is used anywhere.
    # (tcgen05.commit's multicast is an mbarrier arrive, not a load, and is allowed.)
    for p in _sources(".cu", ".cuh", ".h", ".cpp", ".inc"):
        for line in p.read_text().splitlines():
            if "multicast::cluster" in line:
                assert "tcgen05.commit" in line and "cp.async" not in line, f"{p}: {line.strip()}"


def test_kernels_that_touch_a_peers_own_tensors_meet_it_first():
    # the MoonEP kernels that write or read a peer's registered tensors (not its window) call the entry meeting before they do
    text = (CSRC / "moonep" / "moonep_kernels.cu").read_text()
    bodies = {name: text[text.index(f"__device__ void {name}("):] for name in ("MoonDispatchBody", "MoonPrefetchBody", "MoonReduceGradBody")}
    for name, body in bodies.items():
        body = body[: body.index("\n}\n")]
        meet = body.find("MeetPeersOnEntry(")
        touch = body.find("peerBase[")
        assert meet >= 0 and touch >= 0 and meet < touch, name
    # the zero-copy push of the collectives announces and waits as well
    coll = (CSRC / "collectives" / "coll_kernels.cu").read_text()
    assert "READY_SLOT" in coll and coll.index("READY_SLOT") < coll.index("PeerOut(a, peer")
