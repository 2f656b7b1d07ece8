"""The O(S^2) attention oracle that the CUDA kernels are tested against, checked on the CPU against
its own definition: per-query softmax over exactly the visible keys, nothing else."""
import math

import torch

from causal_trainer_dev_b200.ops import attention as A


def _inputs(b=2, s=48, hq=4, hkv=2, d=16, seed=0):
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(b, s, h, d, generator=g) for h in (hq, hkv, hkv))
    seg = torch.zeros(b, s, dtype=torch.int32)
    seg[0, :20], seg[0, 20:41] = 1, 2                      # two documents and a padded tail
    seg[1, 5:30], seg[1, 30:] = 1, 2                       # padding in front
    return q, k, v, seg


def _by_hand(q, k, v, seg, end=None):
    b, s, hq, d = q.shape
    group = hq // k.shape[2]
    out = torch.zeros_like(q)
    for bi in range(b):
        for i in range(s):
            if seg[bi, i] == 0:
                continue
            lim = i if end is None else max(i, int(end[bi, i]))
            keys = [j for j in range(s) if seg[bi, j] == seg[bi, i] and j <= lim]
            for h in range(hq):
                kh = h // group
                scores = torch.stack([q[bi, i, h] @ k[bi, j, kh] for j in keys]) / math.sqrt(d)
                p = torch.softmax(scores, dim=0)
                out[bi, i, h] = sum(p[n] * v[bi, j, kh] for n, j in enumerate(keys))
    return out


def test_matches_the_definition_written_out_per_query():
    q, k, v, seg = _inputs()
    torch.testing.assert_close(A.vanilla_attention(q, k, v, seg), _by_hand(q, k, v, seg), rtol=1e-5, atol=1e-5)


def test_bidirectional_blocks_see_their_own_later_tokens_and_nothing_past_them():
    q, k, v, seg = _inputs(seed=1)
    end = torch.arange(48, dtype=torch.int32).repeat(2, 1)
    end[0, 24:32] = 31                                     # an image block inside document 2 of row 0
    torch.testing.assert_close(A.vanilla_attention(q, k, v, seg, end), _by_hand(q, k, v, seg, end), rtol=1e-5, atol=1e-5)
    base = A.vanilla_attention(q, k, v, seg, end)
    k2, v2 = k.clone(), v.clone()
    k2[0, 32:41] += 3.0                                    # tokens after the block, same document
    v2[0, 32:41] -= 2.0
    moved = A.vanilla_attention(q, k2, v2, seg, end)
    assert torch.equal(moved[0, :32], base[0, :32])        # the block and everything before it do not see them
    assert not torch.equal(moved[0, 32:41], base[0, 32:41])
    mask = A.visibility_mask(seg, end)
    assert mask[0, 24, 31] and mask[0, 31, 24] and not mask[0, 24, 32] and not mask[0, 23, 24]


def test_documents_padding_and_key_value_groups():
    q, k, v, seg = _inputs(seed=2)
    base = A.vanilla_attention(q, k, v, seg)
    assert torch.equal(base[seg == 0], torch.zeros_like(base[seg == 0]))          # padding rows are zero
    k2, v2, q2 = k.clone(), v.clone(), q.clone()
    k2[0, :20] *= -1.0
    v2[0, :20] += 1.0
    q2[0, :20] += 0.5
    other = A.vanilla_attention(q2, k2, v2, seg)
    assert torch.equal(other[0, 20:], base[0, 20:]) and torch.equal(other[1], base[1])   # document 2 and row 1 untouched
    # grouped key/value heads equal the same heads written out once per query head
    wide_k, wide_v = k.repeat_interleave(2, dim=2), v.repeat_interleave(2, dim=2)
    torch.testing.assert_close(A.vanilla_attention(q, wide_k, wide_v, seg), base, rtol=1e-6, atol=1e-6)
    # a custom scale is applied to the scores
    torch.testing.assert_close(A.vanilla_attention(q * 2.0, k, v, seg, scale=0.5 / math.sqrt(16)), base, rtol=1e-5, atol=1e-5)


def test_oracle_is_differentiable_and_gradients_respect_the_documents():
    q, k, v, seg = _inputs(seed=3)
    q, k, v = (t.requires_grad_() for t in (q, k, v))
    out = A.vanilla_attention(q, k, v, seg)
    cot = torch.zeros_like(out)
    cot[0, 20:41] = 1.0                                    # cotangent in document 2 of row 0 only
    out.backward(cot)
    for grad in (q.grad, k.grad, v.grad):
        assert torch.equal(grad[0, :20], torch.zeros_like(grad[0, :20])) and torch.equal(grad[1], torch.zeros_like(grad[1]))
        assert grad[0, 20:41].abs().sum() > 0
