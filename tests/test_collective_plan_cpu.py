"""How a collective call is cut into tiles, blocks and launches (pure host arithmetic, `TileXRCollectivePlan`): the
invariants the kernels rely on, for every operator over seven decades of message size.  Counterpart of the reference's
host tests of its block-dim tables (tests/collectives/unit)."""
import pytest
import torch

from tilexr_b200 import _C

OPS = {"all_reduce": 1, "reduce_scatter": 2, "all_gather": 3, "broadcast": 4, "all_to_all": 5}
FLAGS_PER_PAIR = 1024
ONE_SHOT, TWO_SHOT = 4, 5


@pytest.mark.parametrize("op", sorted(OPS))
@pytest.mark.parametrize("ranks", [2, 4, 8, 16])
def test_plan_invariants(op, ranks):
    half = 512 << 20
    max_grid = 296
    last_grid = 0
    for count in (8, 64, 4096, 1 << 16, 1 << 20, 1 << 24, 1 << 28, 1 << 31):
        d = _C.collective_plan(OPS[op], count, torch.bfloat16, ranks, half, max_grid)
        nbytes = count * 2
        assert d["grid"] == d["producers"] + d["reducers"] + d["consumers"] <= max_grid
        assert d["producers"] >= 1 and d["consumers"] >= 1
        assert d["tile_bytes"] % 16 == 0 and d["tile_bytes"] > 0
        assert 1 <= d["tiles_per_launch"] <= FLAGS_PER_PAIR            # one flag per tile and pair: a launch never wraps its ring
        assert d["launches"] >= 1 and d["launches"] * d["bytes_per_launch"] >= nbytes
        assert (d["launches"] - 1) * d["bytes_per_launch"] < nbytes      # no empty launch
        # what one launch stages per (source, destination) pair fits the share of the window half of that pair
        assert d["tiles_per_launch"] * d["tile_bytes"] <= half // ranks + d["tile_bytes"]
        if count >= 1 << 16:
            assert d["grid"] >= last_grid                                 # more bytes never get fewer blocks
        last_grid = d["grid"]
    small = _C.collective_plan(OPS[op], 64, torch.bfloat16, ranks, half, max_grid)
    large = _C.collective_plan(OPS[op], 1 << 26, torch.bfloat16, ranks, half, max_grid)
    assert small["grid"] < large["grid"] and small["launches"] == 1
    assert _C.collective_plan(OPS[op], 1 << 31, torch.bfloat16, ranks, half, max_grid)["launches"] > 1


def test_all_reduce_switches_algorithm_with_size():
    kinds = [_C.collective_plan(OPS["all_reduce"], c, torch.bfloat16, 8, 512 << 20, 296)["kind"] for c in (64, 4096, 1 << 16, 1 << 20, 1 << 26)]
    assert kinds[0] == ONE_SHOT and kinds[-1] == TWO_SHOT
    assert kinds == sorted(kinds)                                         # one switch, from one-shot to two-shot
    two = _C.collective_plan(OPS["all_reduce"], 1 << 26, torch.bfloat16, 8, 512 << 20, 296)
    assert two["reducers"] > 0
    one = _C.collective_plan(OPS["all_reduce"], 64, torch.bfloat16, 8, 512 << 20, 296)
    assert one["reducers"] == 0


def test_small_grid_limit_is_respected_and_bad_arguments_are_refused():
    d = _C.collective_plan(OPS["all_reduce"], 1 << 20, torch.bfloat16, 8, 512 << 20, 40)
    assert d["grid"] <= 40 and d["producers"] >= 1 and d["reducers"] >= 1 and d["consumers"] >= 1
    small_half = _C.collective_plan(OPS["all_gather"], 1 << 24, torch.bfloat16, 8, 8 << 20, 296)
    assert small_half["launches"] > 1                                     # a small window means more launches, not a wrapped ring
    assert small_half["tiles_per_launch"] * small_half["tile_bytes"] <= (8 << 20) // 8 + small_half["tile_bytes"]
    for bad_op in (0, 6, 7, 99):
        with pytest.raises(RuntimeError):
            _C.collective_plan(bad_op, 1024, torch.bfloat16, 8, 512 << 20, 296)
    with pytest.raises(RuntimeError):
        _C.collective_plan(OPS["all_gather"], 0, torch.bfloat16, 8, 512 << 20, 296)
