"""The balance planner on the CPU: invariants of the plan for random and skewed routings."""
import pytest
import torch


def _all_topk(r, s, k, e, seed, skew):
    g = torch.Generator().manual_seed(seed)
    if skew:
        p = torch.ones(e)
        p[: max(1, e // 8)] = 12.0          # a few hot experts on the first ranks
        return torch.stack([torch.multinomial(p, s * k, replacement=True, generator=g) for _ in range(r)]).to(torch.int32)
    return torch.randint(0, e, (r, s * k), generator=g, dtype=torch.int32)


@pytest.mark.parametrize("r,s,k,e,b,pad,skew", [
    (2, 2, 1, 2, 1, 1, False), (4, 64, 4, 32, 8, 1, False), (4, 64, 4, 32, 8, 16, True), (8, 128, 8, 64, 4, 8, True),
    (8, 32, 2, 16, 2, 128, True), (1, 16, 2, 4, 2, 4, False),
])
def test_reference_plan_invariants(r, s, k, e, b, pad, skew):
    import tilexr_b200 as txr

    topk = _all_topk(r, s, k, e, 7, skew)
    n, per = s * k, e // r
    plans = [txr._C.moonep_reference_plan(topk, rank, s, k, e, b, pad) for rank in range(r)]
    nvs = plans[0]["NvS"]
    assert nvs == n + (pad - 1) * 2 * per
    # every rank computes the same slot assignment
    for p in plans[1:]:
        assert torch.equal(p["experts_to_copy"], plans[0]["experts_to_copy"])
    taken = [set() for _ in range(r)]
    received = [0] * r
    for rank in range(r):
        dst = plans[rank]["dst"]
        assert (dst >= 0).all()
        for i, raw in enumerate(dst.tolist()):
            d, slot = divmod(raw, nvs)
            assert d < r and slot not in taken[d]
            taken[d].add(slot)
            received[d] += 1
            # the slot lies inside the group of the route's expert at that destination
            expert = int(topk[rank, i])
            cu = plans[d]["cu_seqlens"].tolist()
            etc = plans[d]["experts_to_copy"][d].tolist()
            group = e + etc.index(expert) if expert in etc else expert
            begin = 0 if group == 0 else cu[group - 1]
            assert begin <= slot < cu[group]
            if group < e and not (d * per <= expert < (d + 1) * per):
                pytest.fail("a remote expert without a prefetch slot received rows")
    # balanced: every rank receives exactly N rows unless slots ran out
    assert sum(received) == r * n
    if b == per:
        assert all(x == n for x in received)
    for rank in range(r):
        cu = plans[rank]["cu_seqlens"].tolist()
        assert all(x <= y for x, y in zip(cu, cu[1:])) and cu[-1] <= nvs
        assert all(c % pad == 0 for c in cu)
        zf = plans[rank]["zero_fill_ranges"]
        padded = sum(int(x) for x in zf[:, 1])
        assert padded == nvs - received[rank]


def test_capabilities():
    import tilexr_b200 as txr

    abi, native, stub = txr._C.moonep_capabilities()
    assert abi == 2 and native == 0b11111 and stub == 0
