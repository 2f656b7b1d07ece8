"""MoBA on the sm_100a kernels: pooling + routing against the PyTorch router, and the block-sparse
flash forward / backward against an fp32 masked-softmax oracle that uses the kernel's own selection."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _segments(b, s, lengths, device):
    seg = torch.zeros((b, s), dtype=torch.int32, device=device)
    for row, lens in enumerate(lengths):
        pos = 0
        for i, n in enumerate(lens):
            seg[row, pos:pos + n] = i + 1
            pos += n
    return seg


def _mask_from_selection(sel, seg, doc_start, block):
    b, hq, s, _ = sel.shape
    idx = torch.arange(s, device=sel.device)
    same = (seg[:, :, None] == seg[:, None, :]) & (seg[:, :, None] != 0)                   # [B,Sq,Sk]
    kb = ((idx[None, None, :] - doc_start[:, :, None].long()) // block).clamp(0, 31)        # block of key j in i's frame
    bits = (sel[..., 0].long()[:, :, :, None] >> kb[:, None]) & 1                           # [B,Hq,Sq,Sk]
    causal = idx[None, :] <= idx[:, None]
    return bits.bool() & same[:, None] & causal[None, None]


@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 128), (2, 2, 64)])
def test_moba_sparse_flash_matches_masked_oracle(cuda_lib, hq, hkv, d):
    from causal_trainer_dev_b200.models import moba as M
    from causal_trainer_dev_b200.ops import moba as ops
    from causal_trainer_dev_b200.ops.attention import build_attention_meta

    torch.manual_seed(0)
    dev = torch.device("cuda")
    b, s, block, top_k = 2, 2048, 256, 3
    seg = _segments(b, s, [[1100, 700, 200], [2048]], dev)
    q = (torch.randn((b, s, hq, d), device=dev) * 0.8).bfloat16().requires_grad_(True)
    k = (torch.randn((b, s, hkv, d), device=dev) * 0.8).bfloat16().requires_grad_(True)
    v = torch.randn((b, s, hkv, d), device=dev).bfloat16().requires_grad_(True)
    meta = build_attention_meta(seg, None)
    scale = 1.0 / math.sqrt(d)
    routing = ops.build_routing(q.detach(), k.detach(), meta, block, top_k)
    assert 0.0 < routing.visited_fraction < 0.9
    # ---- router against the PyTorch oracle (near ties may flip a choice)
    current, previous, starts = M.moba_selected_blocks(q.detach(), k.detach(), seg, block, top_k)
    want = torch.zeros((b, s, hq), dtype=torch.long, device=dev)
    want |= torch.where(seg[:, :, None] != 0, 1 << current[:, :, None], torch.zeros_like(want))
    for r in range(previous.shape[-1]):
        pr = previous[..., r]
        want |= torch.where((pr >= 0) & (seg[:, :, None] != 0), 1 << pr.clamp(min=0), torch.zeros_like(want))
    got = routing.sel[..., 0].long().permute(0, 2, 1)
    assert (got != want).float().mean() < 5e-3
    assert torch.equal(routing.doc_start.long()[seg != 0], starts.long()[seg != 0])
    # every row keeps its own block and at most top_k blocks
    pop = sum(((got >> i) & 1) for i in range(32))
    assert int(pop.max()) <= top_k and bool(((pop >= 1) | (seg[:, :, None] == 0)).all())
    # ---- attention against the masked oracle with the kernel's selection
    out = ops.moba_flash_attention(q, k, v, seg, block, top_k, scale, meta)
    mask = _mask_from_selection(routing.sel, seg, routing.doc_start, block)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = M._masked_attention(qf, kf, vf, mask, scale)
    assert (out.float() - ref).abs().max() < 3e-2
    grad = torch.randn_like(out)
    out.backward(grad)
    ref.backward(grad.float())
    for name, a, r in (("dq", q.grad, qf.grad), ("dk", k.grad, kf.grad), ("dv", v.grad, vf.grad)):
        err = (a.float() - r).norm() / r.norm()
        assert err < 2e-2, (name, float(err))


def test_moba_with_full_budget_equals_dense(cuda_lib):
    from causal_trainer_dev_b200.ops import moba as ops
    from causal_trainer_dev_b200.ops.attention import build_attention_meta, flash_attention_forward

    torch.manual_seed(1)
    dev = torch.device("cuda")
    b, s, h, d, block = 1, 1024, 2, 128, 128
    seg = _segments(b, s, [[600, 424]], dev)
    q, k, v = ((torch.randn((b, s, h, d), device=dev) * 0.7).bfloat16() for _ in range(3))
    meta = build_attention_meta(seg, None)
    routing = ops.build_routing(q, k, meta, block, top_k=8)      # 8 * 128 >= every document: nothing is dropped
    sparse, lse_s = ops.moba_forward(q, k, v, meta, routing)
    dense, lse_d = flash_attention_forward(q, k, v, meta)
    assert (sparse.float() - dense.float()).abs().max() < 1e-2
    assert (lse_s - lse_d).abs().max() < 1e-3


@pytest.mark.parametrize("s,lengths", [(2048, [[1100, 700, 200], [2048]]), (1152, [[600, 500], [1000]])])
def test_work_list_kernels_match_pytorch_builder(cuda_lib, s, lengths):
    """The touch bitmap + list compaction kernels give the lists of the scatter / cumsum / nonzero builder."""
    from causal_trainer_dev_b200.ops import moba as ops
    from causal_trainer_dev_b200.ops.attention import build_attention_meta

    torch.manual_seed(3)
    dev = torch.device("cuda")
    b, hq, hkv, d, block, top_k = 2, 4, 2, 128, 128, 3
    seg = _segments(b, s, lengths, dev)
    q = (torch.randn((b, s, hq, d), device=dev) * 0.8).bfloat16()
    k = (torch.randn((b, s, hkv, d), device=dev) * 0.8).bfloat16()
    meta = build_attention_meta(seg, None)
    got = ops.build_routing(q, k, meta, block, top_k)
    want = ops.build_routing_reference(q, k, meta, block, top_k, sel=got.sel)
    assert torch.equal(got.allsel, want.allsel)
    for name in ("fwd", "dq", "dkv"):
        g, w = getattr(got, name), getattr(want, name)
        assert torch.equal(g.lengths().cpu(), w.lengths().cpu()), name
        n = g.lengths().numel()
        for item in {0, 1, n // 3, n // 2, n - 2, n - 1}:
            assert g.item(item) == w.item(item), (name, item)
    assert abs(got.visited_fraction - want.visited_fraction) < 1e-9


# ------------------------------------------------------------------------------- grouped MoBA
def _grouped(q, k, v, seg, block, top_k, scale, grad=None):
    from causal_trainer_dev_b200.ops import moba as ops
    from causal_trainer_dev_b200.ops.attention import build_attention_meta

    meta = build_attention_meta(seg, None)
    groups = ops.build_groups(q, k, meta, block, top_k)
    out, lse = ops.moba_grouped_forward(q, k, v, meta, groups, scale)
    grads = None
    if grad is not None:
        grads = ops.moba_grouped_backward(q, k, v, out, grad, lse, meta, groups, scale)
    return out, lse, grads, groups, meta


@pytest.mark.parametrize("hq,hkv,d,block", [(4, 2, 128, 256), (2, 2, 64, 128), (8, 2, 128, 384)])
def test_grouped_moba_matches_masked_oracle(cuda_lib, hq, hkv, d, block):
    """Own-block pass + dense pass per group + LSE merge against one fp32 masked softmax over the
    union, with the kernel's own selection; document starts that are not multiples of 128."""
    from causal_trainer_dev_b200.models import moba as M

    torch.manual_seed(0)
    dev = torch.device("cuda")
    b, s, top_k = 2, 2048, 3
    seg = _segments(b, s, [[1100, 700, 200], [2048]], dev)
    q = (torch.randn((b, s, hq, d), device=dev) * 0.8).bfloat16()
    k = (torch.randn((b, s, hkv, d), device=dev) * 0.8).bfloat16()
    v = torch.randn((b, s, hkv, d), device=dev).bfloat16()
    scale = 1.0 / math.sqrt(d)
    grad = torch.randn((b, s, hq, d), device=dev).bfloat16()
    out, lse, (dq, dk, dv), groups, meta = _grouped(q, k, v, seg, block, top_k, scale, grad)
    mask = _mask_from_selection(groups.sel, seg, meta.start, block)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    ref = M._masked_attention(qf, kf, vf, mask, scale)
    assert (out.float() - ref).abs().max() < 3e-2
    ref.backward(grad.float())
    for name, a, r in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
        err = (a.float() - r).norm() / r.norm()
        assert err < 2e-2, (name, float(err))
    # log-sum-exp of the union
    scores = torch.einsum("bqhd,bkhd->bhqk", qf.detach(), kf.detach().repeat_interleave(hq // hkv, dim=2)) * scale
    ref_lse = torch.logsumexp(scores.masked_fill(~mask, float("-inf")), dim=-1)
    live = (seg != 0)[:, None, :].expand_as(lse)
    assert (lse[live] - ref_lse[live]).abs().max() < 2e-2


def test_grouped_moba_work_follows_the_routing_budget_and_the_grouping_is_a_permutation(cuda_lib):
    """Counts the work: every (row, pick) pair occupies exactly one gathered row, the padding is
    below 256 rows per group, and the history tiles visited equal rows/128 * block/128 -- a
    function of top_k, not of the sequence length."""
    from causal_trainer_dev_b200.ops import moba as ops
    from causal_trainer_dev_b200.ops.attention import build_attention_meta

    torch.manual_seed(4)
    dev = torch.device("cuda")
    b, s, hq, hkv, d, block, top_k = 1, 4096, 4, 2, 128, 256, 3
    seg = _segments(b, s, [[4096]], dev)
    q = (torch.randn((b, s, hq, d), device=dev)).bfloat16()
    k = (torch.randn((b, s, hkv, d), device=dev)).bfloat16()
    meta = build_attention_meta(seg, None)
    groups = ops.build_groups(q, k, meta, block, top_k)
    summary = groups.work_summary()
    sel = groups.sel[..., 0].long()
    idx = torch.arange(s, device=dev)
    cur = (idx // block)[None, None, :]
    picks = sum(((sel >> c) & 1) * (c < cur) for c in range(s // block))             # earlier blocks picked per row
    assert int(picks.max()) == top_k - 1 and summary["real_rows"] == int(picks.sum())
    assert summary["gathered_rows"] - summary["real_rows"] < 256 * summary["groups"]
    assert summary["groups"] <= hkv * (s // block - 1)
    rows = summary["gathered_rows"]
    used = groups.row_of[:rows]
    real = used[used >= 0]
    # (token, head) pairs appear once per pick, and pos_of is the inverse of row_of
    pos = groups.pos_of.reshape(-1, top_k - 1)
    flat_rows = torch.arange(b * hq * s, device=dev)
    i_of, h_of = flat_rows % s, (flat_rows // s) % hq
    ids = (i_of * hq + h_of)[:, None].expand_as(pos)
    assert torch.equal(groups.row_of[pos[pos >= 0].long()].long(), ids[pos >= 0])
    assert real.numel() == int((pos >= 0).sum())
    # dense causal attention would visit s/128 * (s/128 + 1) / 2 tiles per head; the grouped history pass
    dense_tiles = hq * (s // 128) * (s // 128 + 1) // 2
    assert summary["history_tiles"] <= (hq * s * (top_k - 1) // 128 + 2 * summary["groups"]) * (block // 128)
    assert summary["history_tiles"] + hq * (s // 128) * (block // 128 + 1) // 2 < 0.5 * dense_tiles


def test_grouped_moba_with_full_budget_equals_dense_and_is_deterministic(cuda_lib):
    from causal_trainer_dev_b200.ops.attention import build_attention_meta, flash_attention_backward, flash_attention_forward

    torch.manual_seed(1)
    dev = torch.device("cuda")
    b, s, h, d, block = 1, 1024, 2, 128, 128
    seg = _segments(b, s, [[600, 424]], dev)
    q, k, v = ((torch.randn((b, s, h, d), device=dev) * 0.7).bfloat16() for _ in range(3))
    grad = torch.randn((b, s, h, d), device=dev).bfloat16()
    scale = 1.0 / math.sqrt(d)
    out, lse, (dq, dk, dv), _, meta = _grouped(q, k, v, seg, block, 8, scale, grad)      # 8 * 128 >= every document
    dense, lse_d = flash_attention_forward(q, k, v, meta, scale)
    assert (out.float() - dense.float()).abs().max() < 2e-2 and (lse - lse_d).abs().max() < 2e-3
    dq_d, dk_d, dv_d = flash_attention_backward(q, k, v, dense, grad, lse_d, meta, scale)
    for a, r in ((dq, dq_d), (dk, dk_d), (dv, dv_d)):
        assert (a.float() - r.float()).norm() / r.float().norm() < 2e-2
    again = _grouped(q, k, v, seg, block, 8, scale, grad)
    assert torch.equal(out, again[0]) and all(torch.equal(x, y) for x, y in zip((dq, dk, dv), again[2]))


def test_grouped_moba_does_not_leak_between_documents(cuda_lib):
    """Changing one document changes nothing, bit for bit, in the outputs and gradients of another."""
    torch.manual_seed(2)
    dev = torch.device("cuda")
    b, s, hq, hkv, d, block, top_k = 1, 2048, 4, 2, 128, 128, 3
    seg = _segments(b, s, [[900, 1148]], dev)
    q = (torch.randn((b, s, hq, d), device=dev) * 0.8).bfloat16()
    k = (torch.randn((b, s, hkv, d), device=dev) * 0.8).bfloat16()
    v = torch.randn((b, s, hkv, d), device=dev).bfloat16()
    grad = torch.randn((b, s, hq, d), device=dev).bfloat16()
    scale = 1.0 / math.sqrt(d)
    out_a, _, grads_a, _, _ = _grouped(q, k, v, seg, block, top_k, scale, grad)
    q2, k2, v2, g2 = q.clone(), k.clone(), v.clone(), grad.clone()
    for t in (q2, k2, v2, g2):
        t[:, 900:] = torch.randn_like(t[:, 900:])
    out_b, _, grads_b, _, _ = _grouped(q2, k2, v2, seg, block, top_k, scale, g2)
    assert torch.equal(out_a[:, :900], out_b[:, :900])
    for x, y in zip(grads_a, grads_b):
        assert torch.equal(x[:, :900], y[:, :900])
    # and the cotangent of one document reaches no other document
    g3 = torch.zeros_like(grad)
    g3[:, 900:] = grad[:, 900:]
    _, _, (dq, dk, dv), _, _ = _grouped(q, k, v, seg, block, top_k, scale, g3)
    assert not dq[:, :900].any() and not dk[:, :900].any() and not dv[:, :900].any()
