"""The public C API headers compile as C11 (the reference checks the same for its MoonEP ABI header with a `.c`
translation unit, tests/moonep/unit), and the ABI structs keep their sizes between C and C++."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
INCLUDE = ROOT / "csrc" / "include"
C_HEADERS = ["tilexr_api.h", "tilexr_collectives.h", "tilexr_collectives_perf.h", "tilexr_comm_args.h", "tilexr_ep.h", "tilexr_ep_plan.h",
             "tilexr_fused.h", "tilexr_hostsim.h", "tilexr_moonep.h", "tilexr_moonep_planner.h", "tilexr_moonep_combine_v2.h", "tilexr_moonep_trace.h",
             "tilexr_noalloc.h", "tilexr_perf_trace.h", "tilexr_probes.h", "tilexr_types.h"]


@pytest.mark.parametrize("header", C_HEADERS)
def test_header_compiles_as_c(header, tmp_path):
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    src = tmp_path / "unit.c"
    src.write_text(f'#include "{header}"\nint main(void) {{ return 0; }}\n')
    proc = subprocess.run(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", f"-I{INCLUDE}", str(src)], capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr[-2000:]


def test_plan_structs_have_one_size_in_c_and_cpp(tmp_path):
    if shutil.which("gcc") is None or shutil.which("g++") is None:
        pytest.skip("needs gcc and g++")
    body = ('#include <stdio.h>\n#include "tilexr_ep_plan.h"\n#include "tilexr_moonep.h"\n'
            'int main(void) { printf("%zu %zu %zu %zu %zu\\n", sizeof(TileXRMoonEPPlanConfig), sizeof(TileXRMoonEPPlanMetadataV2), '
            'sizeof(TileXRMoonEPPlanDesc), sizeof(TileXRMoonEPStageTables), sizeof(TileXRMoonEpPlanV1)); return 0; }\n')
    sizes = []
    for compiler, name, std in (("gcc", "a.c", "-std=c11"), ("g++", "a.cpp", "-std=c++17")):
        src = tmp_path / name
        src.write_text(body)
        exe = tmp_path / (name + ".out")
        subprocess.run([compiler, std, f"-I{INCLUDE}", str(src), "-o", str(exe)], check=True, capture_output=True)
        sizes.append(subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.strip())
    assert sizes[0] == sizes[1], sizes
