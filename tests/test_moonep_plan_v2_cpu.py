"""Second-generation MoonEP planner on the CPU oracle (the same algorithm source as the kernel): plan invariants on
random, skewed and multi-server routings, status codes, duplicate-route encoding and the route helpers.
Modelled on the reference's tests/ep/unit/test_tilexr_ep_plan_{algorithm,downstream,reference}.cpp."""
import numpy as np
import pytest
import torch

from tilexr_b200 import _C

PLAN_OK, NO_PAIR, SLOTS, SUPPLY, CONFIG, TPE, LAYOUT, OVERFLOW, INVARIANT = range(9)


def make_routing(R, S, K, E, seed, skew=None):
    g = np.random.default_rng(seed)
    topk = np.zeros((R, S, K), dtype=np.int32)
    for r in range(R):
        for s in range(S):
            if skew is None:
                topk[r, s] = g.choice(E, size=K, replace=False)
            else:
                p = np.full(E, (1.0 - skew) / E)
                p[: E // R] += skew / (E // R)      # rank 0's experts are hot
                topk[r, s] = g.choice(E, size=K, replace=False, p=p / p.sum())
    tpe = np.stack([np.bincount(topk[r].reshape(-1), minlength=E) for r in range(R)]).astype(np.int32)
    return topk, tpe


def plan_all(topk, tpe, gids, B, nvs, padding=1, limit=0):
    R = topk.shape[0]
    return [_C.moonep_plan_v2_reference(r, torch.from_numpy(topk[r]), torch.from_numpy(tpe), torch.tensor(gids, dtype=torch.int32),
                                        B, nvs, padding, limit) for r in range(R)]


def check_plan(plans, topk, R, S, K, E, B, nvs, padding, expect_balanced=True):
    L = E // R
    cap = S * K
    rows = [dict() for _ in range(R)]          # dst rank -> row -> (src, route)
    per_rank = np.zeros(R, dtype=np.int64)
    for src in range(R):
        p = plans[src]
        dst = p["dst"].numpy().reshape(S, K)
        for tok in range(S):
            seen = set()
            for k in range(K):
                enc = int(dst[tok, k])
                raw = enc if enc >= 0 else ~enc
                d, row = divmod(raw, nvs)
                assert 0 <= d < R
                assert (enc < 0) == (d in seen), "a route is a duplicate exactly when an earlier route of its token goes to the same rank"
                seen.add(d)
                assert row not in rows[d], "two routes share a row"
                rows[d][row] = (src, int(topk[src, tok, k]))
                per_rank[d] += 1
    if expect_balanced:
        assert (per_rank == cap).all(), per_rank
    # rows of an expert lie in that expert's group on the destination, as laid out by the destination's own plan
    for d in range(R):
        p = plans[d]
        cu = p["cu_seqlens"].numpy()
        slots = p["experts_to_copy"].numpy().tolist()
        assert slots == plans[0]["remote_experts"].numpy()[d].tolist()
        assert all(e < 0 or e // L != d for e in slots), "a slot never holds a home expert"
        assert (np.diff(np.concatenate([[0], cu])) >= 0).all() and cu[-1] <= nvs
        assert (np.diff(np.concatenate([[0], cu])) % padding == 0).all()
        for row, (_, e) in rows[d].items():
            group = E + slots.index(e) if e in slots else e
            if group == e:
                assert e // L == d, "an expert computed without a slot is a home expert"
            lo = 0 if group == 0 else cu[group - 1]
            assert lo <= row < cu[group], (d, e, row, lo, cu[group])
        assert p["remote_stats"].numpy()[0] == sum(1 for e in slots if e >= 0)
        held_elsewhere = sum(1 for q in range(R) for e in plans[0]["remote_experts"].numpy()[q] if e >= 0 and e // L == d)
        assert p["remote_stats"].numpy()[1] == held_elsewhere
        # owner-side bitmap
        targets = p["expert_targets"].numpy().astype(np.uint64)
        for le in range(L):
            holders = {q for q in range(R) if (d * L + le) in plans[0]["remote_experts"].numpy()[q].tolist()}
            bits = {q for q in range(R) if (int(targets[le, q // 64]) >> (q % 64)) & 1}
            assert holders == bits
    # every rank computed the same global tables
    for p in plans[1:]:
        assert torch.equal(p["remote_experts"], plans[0]["remote_experts"])
        assert p["status"][0] == plans[0]["status"][0]


@pytest.mark.parametrize("R,S,K,E,B", [(2, 16, 2, 8, 4), (4, 32, 4, 32, 8), (8, 64, 8, 64, 8), (8, 24, 3, 256, 32)])
def test_random_routing_is_balanced(R, S, K, E, B):
    topk, tpe = make_routing(R, S, K, E, seed=R * 100 + K)
    nvs = S * K + E + B
    plans = plan_all(topk, tpe, list(range(R)), B, nvs)
    assert all(p["code"] == PLAN_OK for p in plans), [p["status"].tolist() for p in plans]
    st = plans[0]["status"].numpy()
    assert st[3] == 0 and st[2] == 0, "one server: everything is balanced inside it"
    check_plan(plans, topk, R, S, K, E, B, nvs, 1)


def test_padding_and_layout_limit():
    R, S, K, E, B = 4, 32, 4, 32, 8
    topk, tpe = make_routing(R, S, K, E, seed=5)
    nvs = S * K + (E + B) * 16
    plans = plan_all(topk, tpe, [0, 1, 2, 3], B, nvs, padding=16)
    assert all(p["code"] == PLAN_OK for p in plans)
    check_plan(plans, topk, R, S, K, E, B, nvs, 16)
    tight = plan_all(topk, tpe, [0, 1, 2, 3], B, S * K, padding=16)       # padded groups cannot fit cap rows
    assert all(p["code"] == LAYOUT for p in tight)


def test_two_servers_move_across():
    R, S, K, E, B = 16, 16, 4, 64, 16
    topk, tpe = make_routing(R, S, K, E, seed=9, skew=0.6)
    gids = list(range(R))                       # ranks 0-7 and 8-15 are two servers
    nvs = R * S * K                             # room for the rows of a plan that stays unbalanced
    plans = plan_all(topk, tpe, gids, B, nvs)
    st = plans[0]["status"].numpy()
    assert st[0] in (PLAN_OK, NO_PAIR, SLOTS, SUPPLY)
    assert st[1] > 0, "the hot rank's server balances itself first"
    if st[0] == PLAN_OK:
        assert st[3] == 0
    check_plan(plans, topk, R, S, K, E, B, nvs, 1, expect_balanced=st[0] == PLAN_OK)
    # permuting the global ids changes servers and affinity: still a valid plan
    gids2 = [(7 * i + 3) % 64 for i in range(R)]
    plans2 = plan_all(topk, tpe, gids2, B, nvs)
    check_plan(plans2, topk, R, S, K, E, B, nvs, 1, expect_balanced=plans2[0]["status"][0] == PLAN_OK)


def test_slot_exhaustion_is_partial_and_consistent():
    R, S, K, E, B = 4, 64, 4, 64, 1
    topk, tpe = make_routing(R, S, K, E, seed=3, skew=0.9)
    nvs = 4 * S * K
    plans = plan_all(topk, tpe, list(range(R)), B, nvs)
    st = plans[0]["status"].numpy()
    assert st[0] == SLOTS and st[3] > 0, st
    check_plan(plans, topk, R, S, K, E, B, nvs, 1, expect_balanced=False)


def test_pair_limit_caps_every_pair():
    R, S, K, E, B = 4, 64, 4, 32, 8
    topk, tpe = make_routing(R, S, K, E, seed=4, skew=0.7)
    nvs = 2 * S * K
    limit = 24
    plans = plan_all(topk, tpe, list(range(R)), B, nvs, limit=limit)
    L = E // R
    for src in range(R):
        dst = plans[src]["dst"].numpy()
        moved = np.zeros(R, dtype=np.int64)
        for route, enc in enumerate(dst):
            raw = int(enc) if enc >= 0 else ~int(enc)
            d = raw // nvs
            if d != int(topk[src].reshape(-1)[route]) // L:
                moved[d] += 1
        assert (moved <= limit).all(), moved
    unlimited = plan_all(topk, tpe, list(range(R)), B, nvs)
    assert unlimited[0]["status"][0] == PLAN_OK


def test_rejects_bad_inputs():
    R, S, K, E, B = 2, 8, 2, 8, 2
    topk, tpe = make_routing(R, S, K, E, seed=1)
    nvs = S * K + E + B
    bad = tpe.copy()
    bad[0, 0] += 1
    bad[0, 1] -= 1 if bad[0, 1] > 0 else 0
    assert plan_all(topk, bad, [0, 1], B, nvs)[0]["code"] == TPE
    assert plan_all(topk, tpe, [3, 3], B, nvs)[0]["code"] == CONFIG          # duplicate global ids
    assert plan_all(topk, tpe, [0, 1], B, S * K - 1)[0]["code"] == CONFIG    # nvS below the capacity
    assert plan_all(topk, tpe, [0, 1], B, nvs, limit=S * K + 1)[0]["code"] == CONFIG


def test_route_helpers():
    R, s, k, nvs = 8, 100, 6, 1000
    gid = _C.moonep_global_token_id(3, 57, 4, R, s, k)
    assert gid == (3 * s + 57) * k + 4
    assert _C.moonep_decode_global_token_id(gid, R, s, k) == (3, 57, 4)
    assert _C.moonep_decode_dst(5 * nvs + 17, nvs, R) == (5 * nvs + 17, 5, 17, 1, 1)
    assert _C.moonep_decode_dst(~(5 * nvs + 17), nvs, R) == (5 * nvs + 17, 5, 17, 0, 1)
    with pytest.raises(RuntimeError):
        _C.moonep_global_token_id(R, 0, 0, R, s, k)
    # rows of two tokens on this rank: token (1, 7) has a primary and two duplicates, token (0, 2) a single row
    rec = torch.tensor([[1, 7, 3, 40, 0], [0, 2, 0, 11, 1], [1, 7, 0, 41, 1], [1, 7, 5, 39, 0]], dtype=torch.int32)
    d = _C.moonep_duplicate_metadata(rec, R, s, k, 64)
    assert d["code"] == PLAN_OK and d["dup_counts"].tolist() == [1, 2]
    assert d["dup_groups"][0].tolist() == [41, 0, 2] and d["dup_loffs"][:2].tolist() == [40, 39]
    assert d["dup_groups"][1].tolist() == [-1, -1, -1] and d["dup_loffs"][2] == -1
    two_primaries = rec.clone()
    two_primaries[0, 4] = 1
    assert _C.moonep_duplicate_metadata(two_primaries, R, s, k, 64)["code"] == INVARIANT


def test_cross_server_moves():
    """All experts of the first server are hot: its ranks cannot balance among themselves, the second server takes over."""
    R, S, K, E, B = 16, 32, 4, 64, 16
    g = np.random.default_rng(21)
    p = np.where(np.arange(E) < E // 2, 1.6, 0.4)
    topk = np.stack([np.stack([g.choice(E, size=K, replace=False, p=p / p.sum()) for _ in range(S)]) for _ in range(R)]).astype(np.int32)
    tpe = np.stack([np.bincount(topk[r].reshape(-1), minlength=E) for r in range(R)]).astype(np.int32)
    nvs = R * S * K
    plans = plan_all(topk, tpe, list(range(R)), B, nvs)
    st = plans[0]["status"].numpy()
    assert st[2] > 0, st                    # rounds across servers
    assert st[0] == PLAN_OK and st[3] == 0, st
    check_plan(plans, topk, R, S, K, E, B, nvs, 1)
    # receivers take from the closest senders: every foreign expert on a rank of the second server has its home in the first
    L = E // R
    remote = plans[0]["remote_experts"].numpy()
    assert all(e < 0 or e // L < 8 for d in range(8, 16) for e in remote[d])
