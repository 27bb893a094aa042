"""Device primitives through the probe kernels: registered-memory put / get / signal, the TMA
local-copy pipeline, device-side range validation, and a wait that runs out of budget."""
import pytest
import torch

from conftest import require_cuda

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def txr():
    require_cuda()
    import tilexr_b200

    return tilexr_b200


def test_put_signal_and_get_between_emulated_ranks(txr):
    C = txr._C
    ranks = 4
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=16)
    info = world[0].physical_info()
    assert info["link"] == "same_device" and info["compute_capability"][0] >= 10 and info["sm_count"] > 0 and not info["nvls_bound"]
    n = 1 << 20
    region = world.symm_empty((n,), torch.int32)
    handles = [0] * ranks      # first registration on every rank
    src = [torch.arange(n, dtype=torch.int32, device="cuda") + 1000 * r for r in range(ranks)]
    blocks = 8
    for call in range(1, 3):
        world.run(lambda c, r: C.put_signal_probe(c, handles[r], 0, src[r], 5, blocks * call, blocks))
        world.check()
    for r in range(ranks):
        assert torch.equal(region[(r + 1) % ranks], src[r])          # rank r wrote into rank r+1
    got = [torch.empty(n, dtype=torch.int32, device="cuda") for _ in range(ranks)]
    world.run(lambda c, r: C.get_probe(c, handles[r], 0, got[r], blocks))
    world.check()
    for r in range(ranks):
        assert torch.equal(got[r], region[(r + 1) % ranks])
    # device-side registry validation: a range past the end of the region is refused, not accessed
    res = world.run(lambda c, r: C.range_check_probe(c, handles[r], n * 4 - 8, 64))
    world.check()
    assert all(int(x.item()) == 4 for x in res)                      # RMA_OUT_OF_RANGE
    res = world.run(lambda c, r: C.range_check_probe(c, 7, 0, 64))
    world.check()
    assert all(int(x.item()) == 2 for x in res)                      # RMA_BAD_HANDLE
    world.destroy()


@pytest.mark.parametrize("nbytes", [64, 4096, 1 << 20, (1 << 20) + 48])
def test_local_copy_probe_and_copy_engine(txr, port, nbytes):
    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{port}", buffer_mb=16, device=0)
    src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros_like(src)
    txr._C.local_copy_probe(comm, dst, src, 4)
    dst2 = torch.zeros_like(src)
    txr._C.local_copy_async(comm, dst2, src)
    torch.cuda.synchronize()
    assert comm.device_status() == 0
    assert torch.equal(dst, src) and torch.equal(dst2, src)
    comm.destroy()


def test_wait_that_nobody_satisfies_times_out_cleanly(txr, port):
    """Failure detection on the device: a flag nothing sets, a short budget, a status the host
    reads; the context stays usable afterwards."""
    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{port}", buffer_mb=16, device=0)
    comm.set_wait_timeout_ms(200)
    txr._C.signal_wait_probe(comm, 9, 1)
    torch.cuda.synchronize()
    assert comm.device_status() == 1                                  # TILEXR_DEV_WAIT_TIMEOUT
    d = comm.dfx()
    assert d[3] == 0xDEAD and d[6] == 9 and d[7] == 1                 # failed, slot 9, expected value 1
    comm.reset_status()
    x = torch.ones(1000, device="cuda")
    y = txr.profile_probe(comm, x)
    torch.cuda.synchronize()
    assert comm.device_status() == 0 and torch.equal(x, y)
    comm.destroy()


def test_data_as_flag_round_trip_and_a_withheld_block(txr):
    """16-byte units that carry their launch epoch (payload and flag in one transaction) between the ranks of an emulated
    world; then one block of every rank sends nothing, its counterpart's wait runs out of a 200 ms budget, the kernel ends
    by itself, the host reads the status, and the communicator works again after a reset."""
    ranks, n = 4, 30000                                              # 120000 bytes: 10000 units over 8 blocks
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=16)
    g = torch.Generator().manual_seed(12)
    src = [torch.randint(-2 ** 31, 2 ** 31 - 1, (n,), generator=g, dtype=torch.int64).to(torch.int32).cuda() for _ in range(ranks)]
    for _ in range(3):                                               # both halves of the low-latency plane, and the reuse guard
        dst = [torch.zeros(n, dtype=torch.int32, device="cuda") for _ in range(ranks)]
        world.run(lambda c, r: txr._C.data_as_flag_probe(c, src[r], dst[r], -1, 8))
        world.check()
        for r in range(ranks):
            assert torch.equal(dst[r], src[(r - 1) % ranks])
    for r in range(ranks):
        world[r].set_wait_timeout_ms(200)
    dst = [torch.zeros(n, dtype=torch.int32, device="cuda") for _ in range(ranks)]
    world.run(lambda c, r: txr._C.data_as_flag_probe(c, src[r], dst[r], 3, 8))
    torch.cuda.synchronize()
    statuses = [world[r].device_status() for r in range(ranks)]
    assert all(s in (1, 2) for s in statuses), statuses              # wait timeout, or aborted by a peer that timed out first
    assert all(world[r].dfx()[3] == 0xDEAD for r in range(ranks))
    # the blocks that did get their units delivered them
    per_block = ((n + 7) // 8 + 2) // 3 * 3
    assert torch.equal(dst[1][:3 * per_block], src[0][:3 * per_block])
    for r in range(ranks):
        world[r].reset_status()
    dst = [torch.zeros(n, dtype=torch.int32, device="cuda") for _ in range(ranks)]
    world.run(lambda c, r: txr._C.data_as_flag_probe(c, src[r], dst[r], -1, 8))
    world.check()
    assert all(torch.equal(dst[r], src[(r - 1) % ranks]) for r in range(ranks))
    world.destroy()


def test_reference_named_verbs_between_emulated_ranks(txr):
    """Kernels written against the reference's device verbs (UDMAPutSignalNbi, UDMAGetNbi, UDMAQuiet; its
    src/include/tilexr_udma.h:748-1046) run on the registered-memory verbs: every warp puts its share into the next rank's
    region with a signal word behind it, waits for its own word, and gets the share back; a put that leaves the region is
    refused on the device."""
    ranks, blocks = 4, 4
    world = txr.init_emulated_world(ranks, device=0, buffer_mb=16)
    n = 1 << 18                                         # payload bytes
    words = blocks * 16                                 # one signal word per warp of the launch
    region = world.symm_empty((n + words * 8,), torch.uint8)
    for r in range(ranks):
        region[r].zero_()
    src = [torch.randint(0, 255, (n,), dtype=torch.uint8, device="cuda") for _ in range(ranks)]
    dst = [torch.zeros(n, dtype=torch.uint8, device="cuda") for _ in range(ranks)]
    for _ in range(2):                                  # the second launch waits for a later epoch in the same words
        world.run(lambda c, r: txr._C.named_verbs_probe(c, src[r], dst[r], n, blocks))
        world.check()
    for r in range(ranks):
        assert torch.equal(region[(r + 1) % ranks][:n], src[r])
        assert torch.equal(dst[r], src[r])
    world.destroy()
