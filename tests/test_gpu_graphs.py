"""CUDA-graph capture of library launches on one GPU (a communicator of world size one): the flag epochs
live on the device, so a replayed launch is a fresh launch."""
import pytest
import torch

from conftest import free_port

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def txr():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import tilexr_b200

    return tilexr_b200


def test_moe_step_replays_from_a_cuda_graph(txr):
    from tilexr_b200.ops import ep

    comm = txr.init_process(0, 1, comm_id=f"127.0.0.1:{free_port()}", buffer_mb=64, device=0)
    bs, h, E, K = 96, 1024, 16, 4
    g = torch.Generator().manual_seed(5)
    x_static = torch.randn(bs, h, generator=g).to(torch.bfloat16).cuda()
    lg_static = torch.randn(bs, E, generator=g).cuda()

    def step():
        d = ep.dispatch(comm, x_static, gate_logits=lg_static, num_experts=E, top_k=K, quant_mode=ep.QUANT_FP8_1X128,
                        score_func=1)
        rows = txr.quant.fp8_dequant_1x128(d.expand_x, d.dynamic_scales, torch.bfloat16)
        return ep.combine(comm, rows, d, expert_scales=d.topk_weights)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        eager = step().clone()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = step()
    launches = txr.launch_count()
    for it in range(4):
        graph.replay()
    torch.cuda.synchronize()
    assert txr.launch_count() == launches            # replays do not go through the host launch path
    assert comm.device_status() == 0
    assert torch.equal(y_static, eager)
    x_static.copy_(torch.randn(bs, h, generator=g).to(torch.bfloat16))
    graph.replay()
    want = step()                                     # eager again, after the replays
    torch.cuda.synchronize()
    assert comm.device_status() == 0
    assert torch.equal(y_static, want)
    comm.destroy()
