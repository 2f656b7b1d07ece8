"""MoBA routing and attention against an independent slow statement of the algorithm."""
import math

import pytest
import torch

from causal_trainer_dev_b200.models import moba as M
from causal_trainer_dev_b200.ops import attention as A


def slow_moba(q, k, v, seg, block, top_k, scale):
    """Per document: blocks from the document start; score completed earlier blocks by q . mean(K);
    keep top_k - 1 (stable), add the current block causally, one softmax over the union."""
    b, s, hq, d = q.shape
    g = hq // k.shape[2]
    out = torch.zeros_like(q, dtype=torch.float32)
    for bi in range(b):
        starts = {}
        for t in range(s):
            sg = int(seg[bi, t])
            if sg and sg not in starts:
                starts[sg] = t
        for t in range(s):
            sg = int(seg[bi, t])
            if not sg:
                continue
            st = starts[sg]
            cur = (t - st) // block
            for h in range(hq):
                kh = h // g
                scores = [float(q[bi, t, h].float() @ k[bi, st + c * block:st + (c + 1) * block, kh].float().mean(0))
                          for c in range(cur)]
                order = sorted(range(cur), key=lambda c: (-scores[c], c))[: top_k - 1]
                keys = [j for c in order for j in range(st + c * block, st + (c + 1) * block)]
                keys += list(range(st + cur * block, t + 1))
                keys = sorted(keys)
                logits = torch.stack([q[bi, t, h].float() @ k[bi, j, kh].float() for j in keys]) * scale
                p = torch.softmax(logits, 0)
                out[bi, t, h] = sum(p[n] * v[bi, j, kh].float() for n, j in enumerate(keys))
    return out


def _inputs(b=1, s=32, hq=2, hkv=1, d=8, seed=0):
    torch.manual_seed(seed)
    return torch.randn(b, s, hq, d), torch.randn(b, s, hkv, d), torch.randn(b, s, hkv, d)


def test_matches_slow_oracle_on_packed_documents():
    q, k, v = _inputs()
    seg = torch.tensor([[1] * 19 + [2] * 13])
    opts = M.AttentionOptions(method="moba", backend="reference", moba_block_size=4, moba_top_k=2)
    got = M.moba_attention(q, k, v, seg, opts, 1 / math.sqrt(8))
    assert torch.allclose(got.float(), slow_moba(q, k, v, seg, 4, 2, 1 / math.sqrt(8)), atol=1e-5)


def test_full_budget_is_exactly_dense():
    q, k, v = _inputs()
    seg = torch.tensor([[1] * 19 + [2] * 13])
    opts = M.AttentionOptions(method="moba", backend="reference", moba_block_size=8, moba_top_k=4)
    dense = A.vanilla_attention(q, k, v, seg, None, 0.3)
    assert torch.equal(M.moba_attention(q, k, v, seg, opts, 0.3), dense)


def test_future_tokens_and_other_documents_cannot_change_a_prefix():
    q, k, v = _inputs(s=32)
    seg = torch.tensor([[1] * 20 + [2] * 12])
    opts = M.AttentionOptions(method="moba", backend="reference", moba_block_size=4, moba_top_k=2)
    base = M.moba_attention(q, k, v, seg, opts, 0.35)
    q2, k2, v2 = q.clone(), k.clone(), v.clone()
    k2[:, 14:] += 1.0
    v2[:, 14:] -= 2.0
    q2[:, 14:] *= 3.0
    again = M.moba_attention(q2, k2, v2, seg, opts, 0.35)
    assert torch.equal(again[:, :14], base[:, :14])


def test_layer_selection_and_option_validation():
    o = M.AttentionOptions(method="moba", dense_prefix_layers=1, dense_suffix_layers=2, dense_after_step=5)
    assert [o.applies_to_layer(i, 6, 0) for i in range(6)] == [False, True, True, True, False, False]
    assert not o.applies_to_layer(2, 6, 5) and o.needs_dense_backend
    with pytest.raises(ValueError):
        M.AttentionOptions(method="dense", dense_prefix_layers=1)
    with pytest.raises(ValueError):
        o.validate_layers(2)


def test_decoder_uses_moba_on_the_selected_layers():
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.decoder import ForwardOptions, decoder_forward
    from causal_trainer_dev_b200.models.params import ModelParams

    cfg = preset("tiny", vocab_size=100)
    p = ModelParams.init_random(cfg, 0, torch.float32)
    ids = torch.randint(3, 100, (1, 32))
    mask = torch.ones(1, 32, dtype=torch.long)
    dense = decoder_forward(p, ids, mask)
    sparse = ForwardOptions(attention_options=M.AttentionOptions(method="moba", backend="reference", moba_block_size=4,
                                                                 moba_top_k=2))
    recovered = ForwardOptions(attention_options=M.AttentionOptions(method="moba", backend="reference", moba_block_size=4,
                                                                    moba_top_k=2, dense_after_step=3), optimizer_step=3)
    assert not torch.allclose(decoder_forward(p, ids, mask, options=sparse), dense, atol=1e-4)
    assert torch.allclose(decoder_forward(p, ids, mask, options=recovered), dense, atol=1e-6)
