"""The device headers compile for the host (their PTX wrappers have host stand-ins), which is how the CPU plumbing runs
the same protocol code.  Layout constants and helpers of the data-as-flag transport, and a send -> check -> receive
round trip of both packed formats on host memory.  (Reference: tests/data_as_flag/unit: 512 / 480 / 32 bytes,
flag at offset 480, eight floats of 1.0, block counts 0 -> 0, 480 -> 1, 481 -> 2.)"""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent

PROGRAM = r'''
#include <cstdio>
#include <cstring>
#include <vector>
#include "device/tilexr_data_as_flag.cuh"
using namespace tilexr;
static_assert(DATA_AS_FLAG_BLOCK_BYTES == 512 && DATA_AS_FLAG_PAYLOAD_BYTES == 480 && DATA_AS_FLAG_FLAG_BYTES == 32, "block");
static_assert(DATA_AS_FLAG_FLAG_OFFSET == 480 && DATA_AS_FLAG_FLAG_FLOATS == 8, "flag");
int main()
{
    if (DataAsFlagBlockCount(0) != 0 || DataAsFlagBlockCount(480) != 1 || DataAsFlagBlockCount(481) != 2) return 1;
    if (DataAsFlagPackedBytes(481) != 1024 || Ll16UnitCount(13) != 2 || Ll16PackedBytes(24) != 32) return 2;
    CommArgs args;
    std::memset(&args, 0, sizeof(args));
    args.extraFlag = TileXR::TILEXR_FLAG_HOST_MEMORY;
    args.waitTimeoutNs = 1000000;
    args.rankSize = 1;
    std::vector<unsigned char> window(TILEXR_WIN_DATA_OFFSET, 0);      // control block and flag planes of rank 0
    args.peerMems[0] = window.data();
    args.peerMemBytes = window.size();
    Waiter w = MakeWaiter(&args, 7, 0);
    const uint64_t n = 1008;                      // whole 16-byte vectors and 12-byte units, not whole 480-byte blocks
    auto nosync = [] {};
    std::vector<unsigned char> src(n + 16), packed(DataAsFlagPackedBytes(n) + 64, 0), out(n + 16, 0);
    for (uint64_t i = 0; i < n; ++i) src[i] = static_cast<unsigned char>(i * 7 + 3);
    if (DataAsFlagCheck(packed.data(), DataAsFlagBlockCount(n), w.epoch)) return 3;      // nothing has arrived yet
    DataAsFlagSend(packed.data(), src.data(), n, w.epoch, 0, 1, nosync);
    if (!DataAsFlagCheck(packed.data(), DataAsFlagBlockCount(n), w.epoch)) return 4;
    if (!DataAsFlagCheckAndRecv(w, out.data(), packed.data(), n, 0, 0, 1, nosync)) return 5;
    if (std::memcmp(out.data(), src.data(), n) != 0) return 6;
    std::vector<unsigned char> ll(Ll16PackedBytes(n) + 64, 0), out2(n + 16, 0);
    Ll16Send(ll.data(), src.data(), n, w.epoch, 0, 1);
    if (!Ll16Recv(w, out2.data(), ll.data(), n, 0, 0, 1)) return 7;
    if (std::memcmp(out2.data(), src.data(), n) != 0) return 8;
    // a batch that never arrives: the bounded wait gives up and says so
    std::vector<unsigned char> empty(Ll16PackedBytes(n) + 64, 0);
    Waiter w2 = MakeWaiter(&args, 9, 0);
    if (Ll16Recv(w2, out2.data(), empty.data(), n, 0, 0, 1)) return 9;
    if (w2.ok()) return 10;
    std::puts("ok");
    return 0;
}
'''


def test_data_as_flag_layout_and_round_trip_on_the_host(tmp_path):
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    src = tmp_path / "daf.cpp"
    src.write_text(PROGRAM)
    exe = tmp_path / "daf"
    proc = subprocess.run(["g++", "-std=c++17", "-O1", f"-I{ROOT / 'csrc' / 'include'}", str(src), "-o", str(exe)],
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0 and run.stdout.strip() == "ok", (run.returncode, run.stdout, run.stderr)


UDMA_PROGRAM = r'''
#include <cstdio>
#include <cstring>
#include <vector>
#include "device/tilexr_udma.cuh"
using namespace tilexr;
int main()
{
    // two ranks whose registered regions live in this process; the program plays rank 0
    constexpr uint64_t BYTES = 4096;
    std::vector<unsigned char> region0(BYTES, 0), region1(BYTES, 0);
    uint8_t *peers[2] = {region0.data(), region1.data()};
    TileXR::TileXRRegistry reg;
    std::memset(&reg, 0, sizeof(reg));
    reg.magic = TILEXR_REGISTRY_MAGIC;
    reg.rankSize = 2;
    reg.regionCount = 1;
    reg.regions[0].bytes = BYTES;
    reg.regions[0].localBase = peers[0];
    reg.regions[0].peerBase = peers;
    CommArgs args;
    std::memset(&args, 0, sizeof(args));
    args.rank = 0;
    args.rankSize = 2;
    args.extraFlag = TileXR::TILEXR_FLAG_HOST_MEMORY;
    if (UDMAEnabled(&args) || UDMAQpCount(&args) != 0) return 1;                   // no registry, no verbs
    args.extraFlag |= TileXR::TILEXR_FLAG_RMA;
    args.registryPtr = &reg;
    if (!UDMAEnabled(&args) || !UDMARegistryEnabled(&args) || UDMAQpCount(&args) == 0) return 2;
    if (!UDMARankValid(&args, 1) || UDMARankValid(&args, 0) || UDMARankValid(&args, 2)) return 3;   // a peer, never itself
    std::vector<unsigned char> src(512), back(512, 0);
    for (size_t i = 0; i < src.size(); ++i) src[i] = static_cast<unsigned char>(i * 5 + 1);
    if (UDMAPutNbiOnQp<unsigned char>(&args, 1, 0, src.data(), 1024, 512) != TILEXR_UDMA_STATUS_SUCCESS) return 4;
    UDMAQuiet(&args, 1);
    if (std::memcmp(region1.data() + 1024, src.data(), 512) != 0) return 5;
    if (UDMAGetNbiOnQp<unsigned char>(&args, 1, 3, back.data(), 1024, 512) != TILEXR_UDMA_STATUS_SUCCESS) return 6;
    if (UDMAQuietStatus(&args, 1) != TILEXR_UDMA_STATUS_SUCCESS || std::memcmp(back.data(), src.data(), 512) != 0) return 7;
    // payload, then the signal word
    if (UDMAPutSignalNbiOnQp<unsigned char>(&args, 1, 1, src.data(), 2048, 256, 4088, 77) != TILEXR_UDMA_STATUS_SUCCESS) return 8;
    uint64_t word = 0;
    std::memcpy(&word, region1.data() + 4088, 8);
    if (word != 77 || std::memcmp(region1.data() + 2048, src.data(), 256) != 0) return 9;
    // refused before a byte moves: range, rank, lane, signal alignment, signal range
    std::memset(region1.data(), 0, BYTES);
    if (UDMAPutNbiOnQp<unsigned char>(&args, 1, 0, src.data(), 4000, 512) != TILEXR_UDMA_STATUS_INVALID) return 10;
    if (UDMAPutNbiOnQp<unsigned char>(&args, 0, 0, src.data(), 0, 16) != TILEXR_UDMA_STATUS_INVALID) return 11;
    if (UDMAPutNbiOnQp<unsigned char>(&args, 1, 99, src.data(), 0, 16) != TILEXR_UDMA_STATUS_INVALID) return 12;
    if (UDMAPutSignalNbiOnQp<unsigned char>(&args, 1, 0, src.data(), 0, 16, 4, 1) != TILEXR_UDMA_STATUS_INVALID) return 13;
    if (UDMAPutSignalNbiOnQp<unsigned char>(&args, 1, 0, src.data(), 0, 16, 4096, 1) != TILEXR_UDMA_STATUS_INVALID) return 14;
    if (UDMAGetNbiOnQp<unsigned char>(&args, 1, 0, back.data(), 4090, 16) != TILEXR_UDMA_STATUS_INVALID) return 15;
    for (uint64_t i = 0; i < BYTES; ++i) {
        if (region1[i] != 0) return 16;
    }
    if (SDMAEnabled(&args)) return 17;
    args.extraFlag |= TileXR::TILEXR_FLAG_LOCAL_COPY;
    if (!SDMAEnabled(&args)) return 18;
    std::puts("ok");
    return 0;
}
'''


def test_reference_named_verbs_on_the_host(tmp_path):
    """The reference's device verb names (UDMAPutNbi, UDMAGetNbi, UDMAPutSignalNbi, UDMAQuiet, ...) over the registered-memory
    verbs: round trips between two regions, and every bad rank, lane or range refused before a byte moves.
    (Reference: src/include/tilexr_udma.h:748-1046.)"""
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    src = tmp_path / "udma.cpp"
    src.write_text(UDMA_PROGRAM)
    exe = tmp_path / "udma"
    proc = subprocess.run(["g++", "-std=c++17", "-O1", f"-I{ROOT / 'csrc' / 'include'}", str(src), "-o", str(exe)],
                          capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr[-3000:]
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0 and run.stdout.strip() == "ok", (run.returncode, run.stdout, run.stderr)
