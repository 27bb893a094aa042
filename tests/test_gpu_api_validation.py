"""Argument validation of the C entry points on a one-rank GPU communicator, called through ctypes like a C program would:
a bad argument is refused with TILEXR_ERROR_PARA_CHECK_FAIL before anything is launched, and the communicator works
afterwards (reference: tests/collectives/unit/test_tilexr_collectives_stub_behavior.cpp:30-58, the host validation tests of
tests/ep/unit and tests/moonep/unit)."""
import ctypes
import pathlib

import pytest
import torch

from conftest import require_cuda

pytestmark = pytest.mark.gpu
LIB = pathlib.Path(__file__).resolve().parent.parent / "tilexr_b200" / "lib" / "libtilexr.so"
PARA_CHECK_FAIL = -3
FP32, BF16, INT128, SUM = 4, 11, 12, 0


def _p(x):
    return ctypes.c_void_p(x)


def test_bad_arguments_are_refused_before_any_launch(port):
    require_cuda()
    import tilexr_b200 as txr

    lib = ctypes.CDLL(str(LIB))
    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{port}", buffer_mb=16, device=0)
    h = _p(comm.handle)
    x = torch.arange(1024, dtype=torch.float32, device="cuda")
    y = torch.zeros_like(x)
    a, b, none = _p(x.data_ptr()), _p(y.data_ptr()), _p(None)
    n = ctypes.c_int64
    stream = _p(torch.cuda.current_stream().cuda_stream)
    bad = [
        lib.TileXRAllGather(none, b, n(16), FP32, h, stream),                 # null buffer
        lib.TileXRAllGather(a, b, n(0), FP32, h, stream),                     # empty message
        lib.TileXRAllGather(a, b, n(-4), FP32, h, stream),
        lib.TileXRAllGather(a, b, n(16), 99, h, stream),                      # unknown element type
        lib.TileXRAllReduce(a, b, n(16), INT128, SUM, h, stream),             # a type that cannot be reduced
        lib.TileXRAllReduce(a, b, n(16), FP32, 7, h, stream),                 # unknown reduce operation
        lib.TileXRReduceScatter(a, none, n(16), FP32, SUM, h, stream),
        lib.TileXRBroadcast(a, n(16), FP32, 1, h, stream),                    # root outside the communicator
        lib.TileXRBroadcast(a, n(16), FP32, -1, h, stream),
        lib.TileXRAllToAll(a, b, n(1 << 62), FP32, h, stream),                # the byte count overflows
        lib.TileXRAllToAll(a, a, n(16), FP32, h, stream),                     # an all-to-all cannot run in place
    ]
    assert bad == [PARA_CHECK_FAIL] * len(bad), bad
    # the GEMM entry: shapes that the tensor maps cannot describe, types it does not multiply
    m = torch.zeros(256, 256, dtype=torch.bfloat16, device="cuda")
    pa = _p(m.data_ptr())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ps = _p(status.data_ptr())
    gemm_bad = [
        lib.TileXRMatmul(pa, pa, pa, n(256), n(256), n(0), BF16, ps, stream),
        lib.TileXRMatmul(pa, pa, pa, n(256), n(256), n(252), BF16, ps, stream),      # K not a multiple of 8 elements
        lib.TileXRMatmul(pa, pa, pa, n(256), n(250), n(256), BF16, ps, stream),
        lib.TileXRMatmul(pa, pa, pa, n(256), n(256), n(256), FP32, ps, stream),
        lib.TileXRMatmul(_p(m.data_ptr() + 2), pa, pa, n(128), n(128), n(128), BF16, ps, stream),   # not 16-byte aligned
        lib.TileXRMatmul(none, pa, pa, n(256), n(256), n(256), BF16, ps, stream),
    ]
    assert gemm_bad == [PARA_CHECK_FAIL] * len(gemm_bad), gemm_bad
    # expert parallelism: the routing does not fit the experts, or the experts do not fit the ranks
    from tilexr_b200.ops import ep

    tokens = torch.randn(8, 256, device="cuda").to(torch.bfloat16)
    ids = torch.zeros(8, 2, dtype=torch.int32, device="cuda")
    for kwargs in (dict(num_experts=4, top_k=8, expert_ids=torch.zeros(8, 8, dtype=torch.int32, device="cuda")),     # more routes than experts
                   dict(num_experts=0, top_k=2, expert_ids=ids),
                   dict(num_experts=4, top_k=2, expert_ids=ids, quant_mode=77),
                   dict(num_experts=4, top_k=2, expert_ids=ids, max_recv_rows=0)):
        with pytest.raises(RuntimeError):
            ep.dispatch(comm, tokens, **kwargs)
    # nothing was launched and nothing is stuck: the same communicator still works
    torch.cuda.synchronize()
    assert comm.device_status() == 0
    assert lib.TileXRAllReduce(a, b, n(1024), FP32, SUM, h, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(y, x)
    d = ep.dispatch(comm, tokens, num_experts=4, top_k=2, expert_ids=ids)
    torch.cuda.synchronize()
    assert comm.device_status() == 0 and int(d.expert_token_nums.sum()) == 16
    comm.destroy()
