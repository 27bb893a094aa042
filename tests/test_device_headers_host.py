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
