"""Attention metadata on the CPU: the per-token intervals the flash kernels mask with describe the
visibility rule exactly (runs are contiguous, so visible keys / seeing queries are intervals)."""
import pytest
import torch

from causal_trainer_dev_b200.models.decoder import canonicalize_segment_ids
from causal_trainer_dev_b200.ops import attention as A


def _case(seed: int, s: int, maskgit: bool):
    gen = torch.Generator().manual_seed(seed)
    b = 2
    mask = torch.ones((b, s), dtype=torch.int32)
    label = torch.zeros((b, s), dtype=torch.int32)
    end = torch.zeros((b, s), dtype=torch.int32)
    for row in range(b):
        p, doc = 0, 0
        while p < s:
            n = min(int(torch.randint(1, s // 3, (1,), generator=gen)), s - p)
            label[row, p:p + n] = doc % 2
            if doc % 5 == 4:
                mask[row, p:p + n] = 0
            elif maskgit and n > 6:
                lo, hi = p + n // 4, p + n // 2
                end[row, lo:hi] = hi - 1
                if n > 20:                      # a second image block in the same document
                    lo2, hi2 = p + (3 * n) // 4, p + n - 1
                    end[row, lo2:hi2] = hi2 - 1
            p += n
            doc += 1
    return mask, label, (end if maskgit else None)


@pytest.mark.parametrize("maskgit", [False, True])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_intervals_equal_the_visibility_rule(seed, maskgit):
    s = 256
    mask, label, end = _case(seed, s, maskgit)
    seg, pos, meta = A.attention_metadata(mask, label, end)
    assert torch.equal(seg, canonicalize_segment_ids(mask, label))
    vis = A.visibility_mask(seg, end)                      # [B,S,S]: query i sees key j
    idx = torch.arange(s)
    lim = meta.lim if meta.lim is not None else idx.expand_as(seg)
    for b in range(seg.shape[0]):
        for i in range(s):
            if seg[b, i] == 0:
                assert not vis[b, i].any() and not vis[b, :, i].any()
                continue
            keys = torch.nonzero(vis[b, i]).reshape(-1)
            assert keys.tolist() == list(range(int(meta.start[b, i]), int(lim[b, i]) + 1)), (b, i)
            queries = torch.nonzero(vis[b, :, i]).reshape(-1)
            assert queries.tolist() == list(range(int(meta.first_q[b, i]), int(meta.end[b, i]) + 1)), (b, i)
    # block ranges cover what their rows need
    nb = s // 128
    for b in range(seg.shape[0]):
        for blk in range(nb):
            rows = [i for i in range(blk * 128, blk * 128 + 128) if seg[b, i] != 0]
            if not rows:
                assert int(meta.kv_hi[b, blk]) <= int(meta.kv_lo[b, blk])
                continue
            assert int(meta.kv_lo[b, blk]) == min(int(meta.start[b, i]) for i in rows)
            assert int(meta.kv_hi[b, blk]) == max(int(lim[b, i]) for i in rows) + 1
            assert int(meta.q_lo[b, blk]) == min(int(meta.first_q[b, i]) for i in rows)
            assert int(meta.q_hi[b, blk]) == max(int(meta.end[b, i]) for i in rows) + 1
    # positions restart with every run
    assert bool(((pos == 0) == ((idx.expand_as(seg) == meta.start) | (seg == 0))).all())
