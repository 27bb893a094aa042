"""The allocation-free single-GPU dispatch entry point, called through its exported C symbol.

Some callers of this library cannot allocate device memory at the moment they need a MoE token
permutation (a server that gave all free memory to its cache pool, a plugin inside another
framework's step, code that cannot afford cudaMalloc's device-wide synchronisation).  For them
`TileXRMoeLocalDispatchNoAlloc` keeps its scratch counters in an array inside the library image.
This test checks it against the communicator-based dispatch on a one-rank communicator, twice in
a row, because the second call runs on the scratch contents the first one left behind.
"""
import ctypes

import pytest
import torch

from conftest import free_port, require_cuda

pytestmark = pytest.mark.gpu


def _outputs(x, ids, experts):
    bs, h = x.shape
    k = ids.shape[1]
    return (torch.empty(bs * k, h, dtype=x.dtype, device=x.device), torch.empty(bs * k, 4, dtype=torch.int32, device=x.device),
            torch.empty(experts, dtype=torch.int64, device=x.device), torch.empty(experts, dtype=torch.int32, device=x.device))


def _call(lib, x, ids, experts, outputs=None):
    bs, h = x.shape
    k = ids.shape[1]
    expand, assist, nums, counts = outputs if outputs is not None else _outputs(x, ids, experts)
    dtype_code = 11 if x.dtype == torch.bfloat16 else 3
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.TileXRMoeLocalDispatchNoAlloc(
        ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(ids.data_ptr()), ctypes.c_int64(bs), ctypes.c_int64(h), ctypes.c_int64(k),
        ctypes.c_int64(experts), ctypes.c_void_p(expand.data_ptr()), ctypes.c_void_p(assist.data_ptr()),
        ctypes.c_void_p(nums.data_ptr()), ctypes.c_void_p(counts.data_ptr()), ctypes.c_int(dtype_code), ctypes.c_void_p(stream))
    return rc, expand, assist, nums, counts


def test_no_alloc_dispatch_matches_communicator_dispatch():
    require_cuda()
    import tilexr_b200 as txr
    from tilexr_b200.ops import ep

    lib = ctypes.CDLL(txr.LIB_PATH)
    lib.TileXRMoeLocalDispatchNoAlloc.restype = ctypes.c_int
    lib.TileXRMoeLocalDispatchNoAllocStatus.restype = ctypes.c_int
    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{free_port()}", buffer_mb=64, device=0)
    g = torch.Generator().manual_seed(42)
    for (bs, h, k, experts) in [(200, 512, 4, 32), (1000, 256, 2, 8)]:       # two calls in a row, different shapes
        x = torch.randn(bs, h, generator=g).to(torch.bfloat16).cuda()
        ids = torch.randint(0, experts, (bs, k), generator=g, dtype=torch.int32)
        ids[3, 1] = -1                                                         # an inactive route
        ids = ids.cuda()
        ref = ep.dispatch(comm, x, expert_ids=ids, num_experts=experts, top_k=k, max_recv_rows=bs * k)
        rc, expand, assist, nums, counts = _call(lib, x, ids, experts)
        assert rc == 0
        torch.cuda.synchronize()
        status = ctypes.c_int(-1)
        assert lib.TileXRMoeLocalDispatchNoAllocStatus(ctypes.byref(status)) == 0 and status.value == 0
        assert comm.device_status() == 0
        n = int(ref.recv_total.item())
        assert n == bs * k - 1
        assert torch.equal(expand[:n], ref.expand_x[:n])                       # rows are copies: exact
        assert torch.equal(assist[:n], ref.assist[:n])
        assert torch.equal(nums, ref.expert_token_nums)
        assert torch.equal(counts, ref.send_counts)
    # the property the entry point exists for: with the outputs in place, a call takes no device memory, neither
    # from the driver nor from torch's pool, and the results are those of the call before
    outputs = _outputs(x, ids, experts)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    stop.record()
    torch.cuda.synchronize()
    free_before, allocated_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    reserved_before = torch.cuda.memory_reserved()
    start.record()
    for _ in range(10):
        rc, expand2, *_ = _call(lib, x, ids, experts, outputs)
        assert rc == 0
    stop.record()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert torch.cuda.memory_allocated() == allocated_before and torch.cuda.memory_reserved() == reserved_before
    assert torch.equal(expand2[:n], expand[:n])
    print(f"no-alloc dispatch {bs} x {h} top-{k}: {start.elapsed_time(stop) * 100:.1f} us per call")
    # sizes beyond the built-in scratch are refused, nothing is launched
    rc, *_ = _call(lib, x, ids, 4096)
    assert rc == -3
    comm.destroy()
