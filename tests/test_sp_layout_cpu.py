"""Index arithmetic of the sequence-parallel token layouts (no GPU: the mixin's pure tensor code)."""
import pytest
import torch

from causal_trainer_dev_b200.training.sp_engine import SequenceParallelAttention


def _rank(world: int, rank: int, layout: str) -> SequenceParallelAttention:
    sp = SequenceParallelAttention()
    sp.sp_world, sp.sp_rank, sp.sp_layout = world, rank, layout
    return sp


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_ranks_partition_the_row_and_the_gathered_slabs_reorder_to_the_sequence(world, layout):
    s = 256 * world
    tokens = torch.arange(s).view(1, s)
    slabs, seen = [], []
    for r in range(world):
        sp = _rank(world, r, layout)
        mine = sp.select_tokens(tokens)
        assert mine.shape == (1, s // world)
        ranges = sp.token_ranges(s)
        assert mine[0].tolist() == [t for lo, n in ranges for t in range(lo, lo + n)]
        assert all(lo % 128 == 0 and n % 128 == 0 for lo, n in ranges)        # whole query tiles
        seen += mine[0].tolist()
        slabs.append(mine[0])
    assert sorted(seen) == list(range(s))
    # what an all-gather over the ranks leaves: one slab per rank, in rank order
    gathered = torch.cat(slabs).view(s, 1).float().repeat(1, 3)
    sp = _rank(world, 0, layout)
    in_order = sp._to_sequence_order(gathered, s)
    assert in_order[:, 0].tolist() == list(range(s))
    if layout == "zigzag":
        back = torch.empty_like(gathered)
        sp._to_slab_order(in_order, back, s)
        assert torch.equal(back, gathered)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_zigzag_gives_every_rank_the_same_causal_work(world):
    s = 256 * world
    work = {}
    for layout in ("contiguous", "zigzag"):
        work[layout] = []
        for r in range(world):
            ranges = _rank(world, r, layout).token_ranges(s)
            work[layout].append(sum(t + 1 for lo, n in ranges for t in range(lo, lo + n)))   # keys a causal query sees
    assert max(work["zigzag"]) == min(work["zigzag"])
    mean = sum(work["contiguous"]) / world
    assert max(work["contiguous"]) / mean == pytest.approx((2 * world - 1) / world, rel=0.02)


def test_rows_that_do_not_divide_into_whole_tiles_fall_back_to_slices():
    sp = _rank(2, 1, "zigzag")
    assert sp.token_ranges(256) == [(128, 128)]            # 64-token chunks would split a query tile
    assert sp.token_ranges(512) == [(128, 128), (256, 128)]
    with pytest.raises(ValueError):
        sp.token_ranges(384 + 64)
