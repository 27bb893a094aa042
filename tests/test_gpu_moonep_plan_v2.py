"""Second-generation MoonEP planner kernel against its CPU oracle on an emulated world (R ranks on one GPU, one
cooperative launch): bit-equal tables on every rank, the agreed status, and a rank with a wrong histogram table."""
import numpy as np
import pytest
import torch

import tilexr_b200 as txr
from tilexr_b200 import _C
from test_moonep_plan_v2_cpu import make_routing, plan_all, PLAN_OK, TPE

pytestmark = pytest.mark.gpu
KEYS = ("dst", "cu_seqlens", "experts_to_copy", "remote_stats", "remote_experts", "expert_targets", "status")


def run_kernel(world, topk, tpe, gids, B, nvs, padding=1, limit=0, tpe_of=None):
    dev_topk = [torch.from_numpy(topk[r]).cuda() for r in range(len(world))]
    dev_tpe = [torch.from_numpy(tpe if tpe_of is None else tpe_of(r)).cuda() for r in range(len(world))]
    dev_gid = torch.tensor(gids, dtype=torch.int32).cuda()
    out = world.run(lambda c, rank: _C.moonep_plan_v2(c, dev_topk[rank], dev_tpe[rank], dev_gid, B, nvs, padding, limit))
    world.check()
    return out


@pytest.mark.parametrize("R,S,K,E,B,skew", [(4, 32, 4, 32, 8, None), (8, 64, 8, 64, 8, 0.5), (8, 128, 8, 256, 32, None)])
def test_kernel_matches_oracle(R, S, K, E, B, skew):
    world = txr.init_emulated_world(R, device=0, buffer_mb=16)
    try:
        topk, tpe = make_routing(R, S, K, E, seed=7 + R, skew=skew)
        nvs = R * S * K if skew else S * K + (E + B) * 8
        gids = list(range(R))
        ref = plan_all(topk, tpe, gids, B, nvs, padding=8)
        got = run_kernel(world, topk, tpe, gids, B, nvs, padding=8)
        for r in range(R):
            for key in KEYS:
                assert torch.equal(got[r][key].cpu(), ref[r][key]), (r, key, got[r]["status"].tolist(), ref[r]["status"].tolist())
        # a second call reuses the windows with the next epoch
        again = run_kernel(world, topk, tpe, gids, B, nvs, padding=8)
        assert all(torch.equal(again[r]["dst"], got[r]["dst"]) for r in range(R))
    finally:
        world.destroy()


def test_wrong_table_on_one_rank_is_seen_by_all():
    R, S, K, E, B = 4, 16, 2, 16, 4
    world = txr.init_emulated_world(R, device=0, buffer_mb=16)
    try:
        topk, tpe = make_routing(R, S, K, E, seed=2)
        nvs = S * K + E + B
        bad = tpe.copy()
        a, b = int(np.argmax(bad[1])), int(np.argmin(bad[1]))
        bad[1, a] -= 1
        bad[1, b] += 1          # rank 2 was handed a table whose row of rank 1 is not what rank 1 counted
        got = run_kernel(world, topk, tpe, list(range(R)), B, nvs, tpe_of=lambda r: bad if r == 2 else tpe)
        assert [int(g["status"][0]) for g in got] == [TPE] * R
        ok = run_kernel(world, topk, tpe, list(range(R)), B, nvs)
        assert [int(g["status"][0]) for g in ok] == [PLAN_OK] * R
    finally:
        world.destroy()
