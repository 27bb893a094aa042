"""The compiler's resource figures per kernel: the parser of `ptxas -v`, the occupancy arithmetic, and one real compile."""
import pathlib
import shutil

import pytest

from tilexr_b200.tools import kernel_report as kr

ROOT = pathlib.Path(__file__).resolve().parents[1]

LOG = """ptxas info    : 0 bytes gmem
ptxas info    : Compiling entry function '_Z3fooPf' for 'sm_100a'
ptxas info    : Function properties for _Z3fooPf
    16 bytes stack frame, 8 bytes spill stores, 12 bytes spill loads
ptxas info    : Used 40 registers, used 2 barriers, 2048 bytes smem, 364 bytes cmem[0], 8 bytes cmem[2]
ptxas info    : Compile time = 1.0 ms
ptxas info    : Function properties for _Z6helperv
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Compiling entry function '_Z3barv' for 'sm_100a'
ptxas info    : Function properties for _Z3barv
    0 bytes stack frame, 0 bytes spill stores, 0 bytes spill loads
ptxas info    : Used 255 registers
"""


def test_parser_reads_entries_and_skips_device_functions():
    rows = kr.parse_ptxas(LOG)
    assert [r["mangled"] for r in rows] == ["_Z3fooPf", "_Z3barv"]
    foo, bar = rows
    assert (foo["registers"], foo["barriers"], foo["static_smem_bytes"], foo["const_bytes"]) == (40, 2, 2048, 372)
    assert (foo["stack_bytes"], foo["spill_store_bytes"], foo["spill_load_bytes"]) == (16, 8, 12)
    assert (bar["registers"], bar["barriers"], bar["static_smem_bytes"], bar["stack_bytes"]) == (255, 0, 0, 0)
    for r in rows:
        r.update(source="x.cu", name=r["mangled"], kernel=r["mangled"])
    assert [r["mangled"] for r in kr.spilling(rows)] == ["_Z3fooPf"]
    text = kr.render(rows, threads=256)
    assert "| `_Z3barv` | 255 | 0 / 0 | 0 | 0 | 0 | 1 | registers |" in text
    assert text.index("_Z3barv") < text.index("_Z3fooPf")              # most registers first


def test_short_names():
    assert kr.short_name("TileXR::(anonymous namespace)::Kernel_single(TileXR::Args)") == "Kernel_single"
    assert kr.short_name("void TileXR::Gemm<true, 2, (Mode)1>(TileXR::GemmArgs const*)") == "Gemm<true, 2, (Mode)1>"
    assert kr.short_name("_Z3fooPf") == "_Z3fooPf"
    assert kr.short_name("plain(float*)") == "plain"


def test_blocks_per_sm():
    assert kr.blocks_per_sm(64, 512, 0) == {"blocks": 2, "limit": "registers", "warps_per_sm": 32, "occupancy": 0.5}
    assert kr.blocks_per_sm(32, 512, 0)["blocks"] == 4 and kr.blocks_per_sm(32, 512, 0)["occupancy"] == 1.0
    assert kr.blocks_per_sm(33, 512, 0)["blocks"] == 3                   # 33 registers are allocated as 40
    o = kr.blocks_per_sm(128, 192, 32, dynamic_smem=216 * 1024)
    assert o["blocks"] == 1 and o["limit"] == "shared memory"
    assert kr.blocks_per_sm(32, 128, 0, dynamic_smem=228 * 1024)["blocks"] == 0
    assert kr.blocks_per_sm(16, 32, 0) == {"blocks": 32, "limit": "blocks", "warps_per_sm": 32, "occupancy": 0.5}
    with pytest.raises(ValueError):
        kr.blocks_per_sm(32, 2048, 0)


@pytest.mark.skipif(shutil.which("nvcc") is None and not pathlib.Path("/usr/local/cuda/bin/nvcc").exists(), reason="needs nvcc")
def test_report_of_a_real_source(capsys, tmp_path):
    out = tmp_path / "r.json"
    assert kr.main([str(ROOT / "csrc" / "collectives" / "ar_quant.cu"), "--threads", "256", "--json", str(out), "--fail-on-spills"]) == 0
    text = capsys.readouterr().out
    assert "TileXRAllReduceQuantKernel_single" in text and "2 kernels in 1 files; 0 with spills" in text
    import json

    rows = json.loads(out.read_text())
    assert {r["kernel"] for r in rows} == {"TileXRAllReduceQuantKernel_single", "TileXRAllReduceQuantKernel_emulated"}
    assert all(r["arch"] == "sm_100a" and 32 <= r["registers"] <= 255 and r["source"] == "csrc/collectives/ar_quant.cu" for r in rows)
