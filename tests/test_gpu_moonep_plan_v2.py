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


@pytest.mark.parametrize("R,S,K,E,skew", [(4, 32, 4, 32, None), (8, 64, 8, 64, 0.5)])
def test_older_call_shape_plans_like_the_configured_call(R, S, K, E, skew):
    """TileXRMoonEpPlannerV2 (one workspace, no configuration; reference src/include/tilexr_moonep_planner.h:18-25) is the
    topology-aware planner with experts-per-rank slots, s * k rows per rank, padding 1 and server-local global ids."""
    world = txr.init_emulated_world(R, device=0, buffer_mb=16)
    try:
        topk, tpe = make_routing(R, S, K, E, seed=11 + R, skew=skew)
        ref = plan_all(topk, tpe, list(range(R)), E // R, S * K, padding=1)
        dev_topk = [torch.from_numpy(topk[r]).cuda() for r in range(R)]
        dev_tpe = torch.from_numpy(tpe).cuda()
        got = world.run(lambda c, rank: _C.moonep_planner_v2_compat(c, dev_topk[rank], dev_tpe))
        world.check()
        for r in range(R):
            assert got[r]["dispatched_capacity"] == S * K
            for key in ("dst", "cu_seqlens", "experts_to_copy", "remote_stats"):
                assert torch.equal(got[r][key].cpu(), ref[r][key]), (r, key)
            assert int(got[r]["planner_status"].item()) == int(ref[r]["status"][0])
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


def test_v2_plan_drives_dispatch_and_combine():
    """The stage tables of a V2 plan (skewed routing, foreign experts in slots) through dispatch and combine."""
    R, S, K, E, B, pad, h = 8, 48, 4, 64, 8, 8, 256
    world = txr.init_emulated_world(R, device=0, buffer_mb=64)
    try:
        topk, tpe = make_routing(R, S, K, E, seed=31, skew=0.4)
        nvs = 2 * S * K + (E + B) * pad
        n = S * K
        got = run_kernel(world, topk, tpe, list(range(R)), B, nvs, padding=pad)
        assert int(got[0]["status"][0]) == PLAN_OK and int(got[0]["status"][6]) > 0      # experts moved
        plans = [g["stage_plan"] for g in got]
        assert all(int(p["status"].item()) == 0 for p in plans)
        # dst_local is the inverse of the decoded destinations; rows outside it lie in the zero-fill ranges
        for rank in range(R):
            dl = plans[rank]["dst_local"].cpu()
            filled = 0
            for src in range(R):
                for i, raw in enumerate(plans[src]["dst"].cpu().tolist()):
                    if raw // nvs == rank:
                        assert int(dl[raw % nvs]) == src * n + i
                        filled += 1
            assert int((dl >= 0).sum()) == filled == n
            zero = torch.zeros(nvs, dtype=torch.bool)
            for lo, count in plans[rank]["zero_fill_ranges"].cpu().tolist():
                assert 0 <= lo and count >= 0 and lo + count <= nvs
                zero[lo:lo + count] = True
            assert torch.equal(zero, dl < 0)
        g = torch.Generator().manual_seed(5)
        hidden = [torch.randn(S, h, generator=g).to(torch.bfloat16).cuda() for _ in range(R)]
        weights = [torch.rand(S, K, generator=g).cuda() for _ in range(R)]
        rows = world.symm_empty((nvs, h), torch.bfloat16)
        wrow = world.symm_empty((nvs,), torch.float32)
        for x in rows:
            x.fill_(7.0)
        world.run(lambda c, rank: _C.moonep_dispatch(c, plans[rank], hidden[rank], weights[rank], rows[rank], wrow[rank]))
        world.check()
        for rank in range(R):
            dl = plans[rank]["dst_local"].cpu()
            rows_cpu = rows[rank].cpu()
            for slot in range(nvs):
                v = int(dl[slot])
                if v < 0:
                    assert torch.all(rows_cpu[slot] == 0)
                else:
                    src, route = divmod(v, n)
                    assert torch.equal(rows_cpu[slot], hidden[src].cpu()[route // K])
        outs = [torch.empty(S, h, dtype=torch.bfloat16, device="cuda") for _ in range(R)]
        wout = [torch.empty(S, K, dtype=torch.float32, device="cuda") for _ in range(R)]
        world.run(lambda c, rank: _C.moonep_combine(c, plans[rank], rows[rank], wrow[rank], outs[rank], wout[rank]))
        world.check()
        for rank in range(R):
            want = (hidden[rank].float() * K).to(torch.bfloat16)
            assert torch.allclose(outs[rank].float(), want.float(), rtol=1e-2, atol=1e-2)
            assert torch.equal(wout[rank], weights[rank])
    finally:
        world.destroy()
