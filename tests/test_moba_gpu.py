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
