"""tcgen05 flash attention (forward, dQ, dK/dV) against the O(S^2) fp32 oracle.

Tolerances are those of the reference's accelerator tests
(tests/kernels/test_efficient_attention_tpu.py:54-59); leakage checks are bit-exact.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def _segments(b, s, ndoc, pad_left=0, seed=0):
    gen = torch.Generator().manual_seed(seed)
    seg = torch.zeros(b, s, dtype=torch.int32)
    for i in range(b):
        cuts = sorted((torch.randperm(s - pad_left - 1, generator=gen)[: ndoc - 1] + 1 + pad_left).tolist())
        bounds = [pad_left] + cuts + [s]
        for j in range(len(bounds) - 1):
            seg[i, bounds[j]:bounds[j + 1]] = j + 1
    return seg.cuda()


def _run(b, s, hq, hkv, d, seg, end=None, seed=0):
    from causal_trainer_dev_b200.ops import attention as A

    torch.manual_seed(seed)
    q = torch.randn(b, s, hq, d, device="cuda").bfloat16()
    k = torch.randn(b, s, hkv, d, device="cuda").bfloat16()
    v = torch.randn(b, s, hkv, d, device="cuda").bfloat16()
    do = torch.randn(b, s, hq, d, device="cuda").bfloat16()
    meta = A.build_attention_meta(seg, end)
    o, lse = A.flash_attention_forward(q, k, v, meta)
    dq, dk, dv = A.flash_attention_backward(q, k, v, o, do, lse, meta)
    return (q, k, v, do), (o, lse, dq, dk, dv)


@pytest.mark.parametrize("d,hq,hkv", [(128, 4, 2), (64, 4, 2), (128, 4, 1)])
@pytest.mark.parametrize("layout", ["one", "packed", "padded", "maskgit"])
def test_matches_oracle(cuda_lib, d, hq, hkv, layout):
    from causal_trainer_dev_b200.ops import attention as A

    b, s = 2, 768
    seg = _segments(b, s, {"one": 1, "packed": 5, "padded": 3, "maskgit": 2}[layout],
                    pad_left=90 if layout in ("padded", "maskgit") else 0)
    end = None
    if layout == "maskgit":
        end = torch.arange(s, device="cuda", dtype=torch.int32).repeat(b, 1)
        for i in range(b):
            st, en = 120, 330
            if seg[i, st] == seg[i, en - 1]:
                end[i, st:en] = en - 1
    (q, k, v, do), (o, lse, dq, dk, dv) = _run(b, s, hq, hkv, d, seg, end)
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    ref = A.vanilla_attention(qf, kf, vf, seg, end)
    ref.backward(do.float())
    assert _rel(o, ref) < 0.04
    assert _rel(dq, qf.grad) < 0.10
    assert _rel(dk, kf.grad) < 0.12
    assert _rel(dv, vf.grad) < 0.10
    # padding rows: zero output, zero gradients
    pad = seg == 0
    if pad.any():
        assert torch.all(o[pad] == 0) and torch.all(dq[pad] == 0) and torch.all(dk[pad] == 0) and torch.all(dv[pad] == 0)
        assert torch.all(lse.permute(0, 2, 1)[pad] == 0)
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_matches_oracle_at_the_training_shape(cuda_lib):
    """32 query / 8 key-value heads, 4096 tokens packed from six documents (the benchmark's layer
    shape), forward and all three gradients against the fp32 PyTorch attention."""
    from causal_trainer_dev_b200.ops import attention as A

    b, s, hq, hkv, d = 1, 4096, 32, 8, 128
    seg = _segments(b, s, 6)
    (q, k, v, do), (o, lse, dq, dk, dv) = _run(b, s, hq, hkv, d, seg, seed=11)
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    ref = A.vanilla_attention(qf, kf, vf, seg, None)
    ref.backward(do.float())
    assert _rel(o, ref) < 0.04
    assert _rel(dq, qf.grad) < 0.10
    assert _rel(dk, kf.grad) < 0.12
    assert _rel(dv, vf.grad) < 0.10
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_gradients_vanish_outside_the_document_of_the_cotangent(cuda_lib):
    """A cotangent that is non-zero in one document only: dQ, dK and dV are exactly zero everywhere
    else (reference: tests/kernels/test_efficient_attention_tpu.py:353-424)."""
    from causal_trainer_dev_b200.ops import attention as A

    b, s, hq, hkv, d = 1, 1536, 8, 2, 128
    seg = torch.ones(b, s, dtype=torch.int32, device="cuda")
    seg[:, 500:1100] = 2
    seg[:, 1100:] = 3
    torch.manual_seed(4)
    q = torch.randn(b, s, hq, d, device="cuda").bfloat16()
    k = torch.randn(b, s, hkv, d, device="cuda").bfloat16()
    v = torch.randn(b, s, hkv, d, device="cuda").bfloat16()
    do = torch.zeros(b, s, hq, d, device="cuda").bfloat16()
    do[:, 500:1100] = torch.randn(b, 600, hq, d, device="cuda").bfloat16()
    meta = A.build_attention_meta(seg)
    o, lse = A.flash_attention_forward(q, k, v, meta)
    dq, dk, dv = A.flash_attention_backward(q, k, v, o, do, lse, meta)
    inside = torch.zeros(s, dtype=torch.bool, device="cuda")
    inside[500:1100] = True
    for g in (dq, dk, dv):
        assert torch.all(g[:, ~inside] == 0)
        assert float(g[:, inside].float().abs().sum()) > 0
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_no_leakage_between_documents(cuda_lib):
    """Perturbing document 1 changes nothing, bit for bit, in document 2."""
    from causal_trainer_dev_b200.ops import attention as A

    b, s, hq, hkv, d = 1, 512, 4, 2, 128
    seg = torch.ones(b, s, dtype=torch.int32, device="cuda")
    seg[:, 200:] = 2
    (q, k, v, do), base = _run(b, s, hq, hkv, d, seg)
    q2, k2, v2 = q.clone(), k.clone(), v.clone()
    q2[:, :200] += 1
    k2[:, :200] -= 1
    v2[:, :200] *= 2
    meta = A.build_attention_meta(seg)
    o2, lse2 = A.flash_attention_forward(q2, k2, v2, meta)
    dq2, dk2, dv2 = A.flash_attention_backward(q2, k2, v2, o2, do, lse2, meta)
    o, lse, dq, dk, dv = base
    for a, c in ((o, o2), (dq, dq2), (dk, dk2), (dv, dv2)):
        assert torch.equal(a[:, 200:], c[:, 200:])


def test_deterministic(cuda_lib):
    seg = _segments(2, 512, 3)
    _, first = _run(2, 512, 4, 2, 128, seg, seed=5)
    _, second = _run(2, 512, 4, 2, 128, seg, seed=5)
    for a, c in zip(first, second):
        assert torch.equal(a, c)


def test_query_range_matches_slices_of_the_full_pass(cuda_lib):
    """Sequence parallelism: a rank that holds queries [q_off, q_off + Sq) and all keys gets the
    same O / LSE / dQ rows as the full pass, and the ranks' partial dK / dV add up to the full ones."""
    from causal_trainer_dev_b200.ops import attention as A

    torch.manual_seed(7)
    b, s, hq, hkv, d, parts = 2, 1024, 4, 2, 128, 4
    seg = torch.ones(b, s, dtype=torch.int32, device="cuda")
    seg[0, 300:] = 2
    seg[0, 900:] = 0
    seg[1, 517:] = 2
    meta = A.build_attention_meta(seg)
    q = (torch.randn(b, s, hq, d, device="cuda") * 0.7).bfloat16()
    k = (torch.randn(b, s, hkv, d, device="cuda") * 0.7).bfloat16()
    v = torch.randn(b, s, hkv, d, device="cuda").bfloat16()
    do = torch.randn(b, s, hq, d, device="cuda").bfloat16()
    o, lse = A.flash_attention_forward(q, k, v, meta)
    dq, dk, dv = A.flash_attention_backward(q, k, v, o, do, lse, meta)
    sq = s // parts
    dk_sum = torch.zeros_like(dk, dtype=torch.float32)
    dv_sum = torch.zeros_like(dv, dtype=torch.float32)
    for r in range(parts):
        sl = slice(r * sq, (r + 1) * sq)
        q_r, do_r = q[:, sl].contiguous(), do[:, sl].contiguous()
        o_r, lse_r = A.flash_attention_forward(q_r, k, v, meta, q_offset=r * sq)
        assert torch.equal(o_r, o[:, sl]) and torch.equal(lse_r, lse[:, :, sl])
        dq_r, dk_r, dv_r = A.flash_attention_backward(q_r, k, v, o_r, do_r, lse_r, meta, q_offset=r * sq)
        assert torch.equal(dq_r, dq[:, sl])
        dk_sum += dk_r.float()
        dv_sum += dv_r.float()
    assert (dk_sum - dk.float()).abs().max() <= 0.02 * dk.float().abs().max()
    assert (dv_sum - dv.float()).abs().max() <= 0.02 * dv.float().abs().max()
    assert cuda_lib.device_status() == (0, 0, 0, 0)


@pytest.mark.parametrize("s", [128, 1152, 4096, 33024])
@pytest.mark.parametrize("maskgit", [False, True])
def test_metadata_kernel_matches_pytorch_formulation(cuda_lib, s, maskgit):
    """Canonical segments, restart positions, visibility limits and block summaries from the one-launch kernel."""
    from causal_trainer_dev_b200.models.decoder import canonicalize_segment_ids, make_position_ids
    from causal_trainer_dev_b200.ops import attention as A

    gen = torch.Generator().manual_seed(s + int(maskgit))
    b = 3
    mask = torch.ones((b, s), dtype=torch.int32)
    label = torch.zeros((b, s), dtype=torch.int32)
    end = torch.zeros((b, s), dtype=torch.int32)
    for row in range(b):
        p, doc = 0, 0
        while p < s:
            n = int(torch.randint(1, max(2, s // 3), (1,), generator=gen))
            n = min(n, s - p)
            label[row, p:p + n] = doc % 3            # labels repeat: a reused label after another run is a new segment
            if doc % 4 == 3 and row != 1:
                mask[row, p:p + n] = 0               # a hole of padding in the middle
            elif maskgit and n > 8:                  # an image block in the middle of the document
                lo = p + n // 4
                hi = p + n // 2
                end[row, lo:hi] = hi - 1
            p += n
            doc += 1
    mask[0, s - s // 5:] = 0                         # trailing padding
    dev = torch.device("cuda")
    mask_d, label_d = mask.to(dev), label.to(dev)
    end_d = end.to(dev) if maskgit else None
    seg, pos, meta = A.attention_metadata(mask_d, label_d, end_d)
    want_seg = canonicalize_segment_ids(mask_d, label_d)
    assert torch.equal(seg, want_seg)
    assert torch.equal(pos, make_position_ids(mask_d, want_seg, canonical=True))
    want = A.build_attention_meta_reference(want_seg, end_d)
    if maskgit:
        assert torch.equal(meta.lim, want.lim)
    else:
        assert meta.lim is None and want.lim is None
    for name in ("kv_lo", "kv_hi", "q_lo", "q_hi"):
        assert torch.equal(getattr(meta, name), getattr(want, name)), name
    live = want_seg != 0                 # per-token intervals are only defined on real tokens
    for name in ("start", "end", "first_q"):
        assert torch.equal(getattr(meta, name)[live], getattr(want, name)[live]), name
    # canonical ids in, the same ids out
    again = A.build_attention_meta(seg, end_d)
    assert torch.equal(again.seg, seg) and torch.equal(again.kv_lo, want.kv_lo) and torch.equal(again.q_hi, want.q_hi)
