"""The C entry points without a GPU, called through ctypes like a C program would: no communicator, a host-memory
communicator (whose collectives are the CPU ones of tilexr_hostsim.h), and host-only queries that must work anywhere.
Modelled on the reference's stub-behaviour tests (tests/collectives/unit/test_tilexr_collectives_stub_behavior.cpp:30-58,
tests/sdma/unit, tests/moonep/unit host validation)."""
import ctypes
import os
import pathlib

import pytest
import torch
import torch.distributed as dist

from conftest import free_port

LIB = pathlib.Path(__file__).resolve().parent.parent / "tilexr_b200" / "lib" / "libtilexr.so"
NOT_INITIALIZED, PARA_CHECK_FAIL, NOT_SUPPORT = -1, -3, -6
FP32, SUM = 4, 0


@pytest.fixture(scope="module")
def lib():
    import tilexr_b200  # noqa: F401  (loads the library's dependencies first)

    return ctypes.CDLL(str(LIB))


def _p(x):
    return ctypes.c_void_p(x)


def test_calls_without_a_communicator_say_so(lib):
    buf = (ctypes.c_float * 16)()
    a = ctypes.addressof(buf)
    none = _p(None)
    assert lib.TileXRAllGather(_p(a), _p(a), ctypes.c_int64(4), FP32, none, none) == NOT_INITIALIZED
    assert lib.TileXRAllToAll(_p(a), _p(a), ctypes.c_int64(4), FP32, none, none) == NOT_INITIALIZED
    assert lib.TileXRAllReduce(_p(a), _p(a), ctypes.c_int64(4), FP32, SUM, none, none) == NOT_INITIALIZED
    assert lib.TileXRReduceScatter(_p(a), _p(a), ctypes.c_int64(4), FP32, SUM, none, none) == NOT_INITIALIZED
    assert lib.TileXRBroadcast(_p(a), ctypes.c_int64(4), FP32, 0, none, none) == NOT_INITIALIZED
    size, cap = ctypes.c_uint64(7), ctypes.c_int64(7)
    assert lib.TileXRMoonEpPlannerGetWorkspaceSizeV2(none, ctypes.c_int64(8), ctypes.c_int64(2), ctypes.c_int64(4), ctypes.byref(size),
                                                     ctypes.byref(cap)) == NOT_INITIALIZED
    assert size.value == 0 and cap.value == 0                       # outputs are cleared before anything can fail
    assert lib.TileXRMoonEpPlannerGetWorkspaceSizeV2(none, ctypes.c_int64(8), ctypes.c_int64(2), ctypes.c_int64(4), None, None) == PARA_CHECK_FAIL


def test_host_memory_communicator_refuses_the_cuda_entry_points_and_serves_host_queries(lib):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(free_port())
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        import tilexr_b200 as txr

        comm = txr.init_from_torch_distributed(host_memory=True, buffer_mb=16)
        h = _p(comm.handle)
        x = torch.ones(64)
        a = _p(x.data_ptr())
        none = _p(None)
        for call in (lambda: lib.TileXRAllGather(a, a, ctypes.c_int64(4), FP32, h, none),
                     lambda: lib.TileXRAllReduce(a, a, ctypes.c_int64(4), FP32, SUM, h, none),
                     lambda: lib.TileXRReduceScatter(a, a, ctypes.c_int64(4), FP32, SUM, h, none),
                     lambda: lib.TileXRBroadcast(a, ctypes.c_int64(4), FP32, 0, h, none),
                     lambda: lib.TileXRAllToAll(a, a, ctypes.c_int64(4), FP32, h, none)):
            assert call() == NOT_SUPPORT
        # the older planner call's size query is host arithmetic: it works on any communicator
        size, cap = ctypes.c_uint64(0), ctypes.c_int64(0)
        assert lib.TileXRMoonEpPlannerGetWorkspaceSizeV2(h, ctypes.c_int64(64), ctypes.c_int64(4), ctypes.c_int64(8), ctypes.byref(size),
                                                         ctypes.byref(cap)) == 0
        assert cap.value == 256 and size.value > 0 and size.value % 64 == 0
        assert lib.TileXRMoonEpPlannerGetWorkspaceSizeV2(h, ctypes.c_int64(0), ctypes.c_int64(4), ctypes.c_int64(8), ctypes.byref(size),
                                                         ctypes.byref(cap)) == PARA_CHECK_FAIL
        # ... but the planner kernel itself needs a GPU communicator, and says so before touching an argument
        one = ctypes.c_int32(0)
        ws = (ctypes.c_uint8 * 4096)()
        addr = (ctypes.addressof(ws) + 63) // 64 * 64
        p1 = _p(ctypes.addressof(one))
        ret = lib.TileXRMoonEpPlannerV2(p1, p1, h, ctypes.c_int64(64), ctypes.c_int64(4), ctypes.c_int64(8), _p(addr), ctypes.c_uint64(1 << 30), p1, p1,
                                        p1, p1, p1, ctypes.c_uint64(1), none)
        assert ret == NOT_SUPPORT
        assert lib.TileXRMoonEpPlannerV2(p1, p1, h, ctypes.c_int64(64), ctypes.c_int64(4), ctypes.c_int64(8), _p(addr), ctypes.c_uint64(1 << 30), p1,
                                         p1, p1, p1, p1, ctypes.c_uint64(0), none) == PARA_CHECK_FAIL          # waitIterations must be non-zero
        comm.destroy()
    finally:
        dist.destroy_process_group()


def test_symmetric_allocator_plumbing_without_a_gpu(lib, tmp_path):
    """What the runtime-owned symmetric memory needs from the host, checked without a GPU: the support query answers "no" on a
    machine without a driver (the caller then takes cudaMalloc + CUDA IPC), and a descriptor passed through the allocator's own
    Unix-socket hand-over arrives as a descriptor of the same file, with its header; nobody listening is an error, not a hang."""
    vmm, mc = ctypes.c_int(7), ctypes.c_int(7)
    assert lib.TileXRVmmQuerySupport(0, ctypes.byref(vmm), ctypes.byref(mc)) == 0
    if not torch.cuda.is_available():
        assert (vmm.value, mc.value) == (0, 0)
    assert lib.TileXRVmmQuerySupport(0, None, None) == PARA_CHECK_FAIL
    path = tmp_path / "payload.bin"
    path.write_bytes(b"rank memory stands in here")
    fd = os.open(path, os.O_RDONLY)
    try:
        tag = ctypes.c_uint64(0x7E57000000000000 | os.getpid())
        got = ctypes.c_int(-1)
        assert lib.TileXRVmmDescriptorSelfTest(tag, 3, fd, 5, 1, ctypes.byref(got)) == 0
        assert got.value >= 0 and got.value != fd
        try:
            assert os.fstat(got.value).st_ino == os.fstat(fd).st_ino              # the same open file, another descriptor
            assert os.pread(got.value, 100, 0) == b"rank memory stands in here"
        finally:
            os.close(got.value)
        assert lib.TileXRVmmDescriptorNobodyThere(ctypes.c_uint64(tag.value + 1), 0, fd) == 0
        assert lib.TileXRVmmDescriptorSelfTest(tag, 3, fd, 5, 1, None) == PARA_CHECK_FAIL
    finally:
        os.close(fd)
