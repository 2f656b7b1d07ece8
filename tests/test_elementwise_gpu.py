"""Memory-bound sm_100a kernels against their PyTorch reference statements."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("d", [256, 1536, 4096])
def test_rmsnorm_forward_backward(cuda_lib, d):
    from causal_trainer_dev_b200.ops import elementwise as E

    torch.manual_seed(0)
    rows = 777
    x = torch.randn(rows, d, device="cuda").bfloat16()
    res = torch.randn(rows, d, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    y, rstd, h = E.rmsnorm_forward(x, w, 1e-6, residual=res)
    h_ref = (x + res)
    assert torch.equal(h, h_ref)
    assert _rel(y, E.rmsnorm_reference(h_ref, w, 1e-6)) < 4e-3
    y2, _, h2 = E.rmsnorm_forward(x, w, 1e-6)
    assert h2 is x and _rel(y2, E.rmsnorm_reference(x, w, 1e-6)) < 4e-3
    # backward against autograd of the fp32 formula
    xf = h_ref.float().requires_grad_()
    wf = w.float().requires_grad_()
    dy = torch.randn(rows, d, device="cuda").bfloat16()
    dres = torch.randn(rows, d, device="cuda").bfloat16()
    out = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wf
    out.backward(dy.float())
    dx, dw = E.rmsnorm_backward(dy, h, w, rstd, dres=dres)
    assert _rel(dx, xf.grad + dres.float()) < 6e-3
    assert _rel(dw, wf.grad) < 6e-3
    dw2 = dw.clone()
    E.rmsnorm_backward(dy, h, w, rstd, dw_out=dw2, dw_accumulate=True)
    assert _rel(dw2, 2 * wf.grad) < 6e-3


@pytest.mark.parametrize("style", ["gpt-j", "gpt-neox"])
@pytest.mark.parametrize("rot", [128, 64])
def test_rope_inplace_and_inverse(cuda_lib, style, rot):
    from causal_trainer_dev_b200.ops import elementwise as E

    torch.manual_seed(1)
    t, hq, hkv, d = 300, 4, 2, 128
    width = (hq + 2 * hkv) * d
    qkv = torch.randn(t, width, device="cuda").bfloat16()
    pos = torch.randint(0, 100000, (t,), device="cuda", dtype=torch.int32)
    inv = E.inverse_frequencies(rot, 500000.0, device="cuda")
    cos, sin = E.rope_table(pos, inv)
    cr, sr = E.rope_table_reference(pos, inv, torch.bfloat16)
    assert (cos - cr).abs().max() < 1e-2 and (sin - sr).abs().max() < 1e-2
    ref = qkv.clone()
    q_ref = E.rope_reference(ref[:, : hq * d].view(t, hq, d), cos, sin, rot, style)
    k_ref = E.rope_reference(ref[:, hq * d:(hq + hkv) * d].view(t, hkv, d), cos, sin, rot, style)
    work = qkv.clone()
    E.rope_inplace(work, cos, sin, hq + hkv, d, rot, style)
    assert _rel(work[:, : hq * d], q_ref.reshape(t, -1)) < 4e-3
    assert _rel(work[:, hq * d:(hq + hkv) * d], k_ref.reshape(t, -1)) < 4e-3
    assert torch.equal(work[:, (hq + hkv) * d:], qkv[:, (hq + hkv) * d:])  # V untouched
    E.rope_inplace(work, cos, sin, hq + hkv, d, rot, style, inverse=True)
    assert _rel(work, qkv) < 8e-3


def test_swiglu(cuda_lib):
    from causal_trainer_dev_b200.ops import elementwise as E

    torch.manual_seed(2)
    t, f = 513, 688
    gu = torch.randn(t, 2 * f, device="cuda").bfloat16()
    h = E.swiglu_forward(gu)
    assert _rel(h, E.swiglu_reference(gu)) < 4e-3
    guf = gu.float().requires_grad_()
    ref = torch.nn.functional.silu(guf[:, :f]) * guf[:, f:]
    dh = torch.randn(t, f, device="cuda").bfloat16()
    ref.backward(dh.float())
    assert _rel(E.swiglu_backward(gu, dh), guf.grad) < 6e-3


def test_embedding_delta_sumsq_adamw(cuda_lib):
    from causal_trainer_dev_b200.ops import elementwise as E

    torch.manual_seed(3)
    table = torch.randn(1000, 256, device="cuda").bfloat16()
    ids = torch.randint(0, 1000, (4, 64), device="cuda")
    assert torch.equal(E.embedding_gather(ids, table), table[ids.reshape(-1)])
    o = torch.randn(2, 128, 4, 64, device="cuda").bfloat16()
    do = torch.randn(2, 128, 4, 64, device="cuda").bfloat16()
    ref = (o.float() * do.float()).sum(-1).permute(0, 2, 1)
    assert torch.allclose(E.attention_delta(o, do), ref, atol=1e-3, rtol=1e-3)
    x = torch.randn(100003, device="cuda").bfloat16()
    assert torch.allclose(E.sum_of_squares(x), x.float().pow(2).sum(), rtol=1e-4)
    n = 70001
    p = torch.randn(n, device="cuda").bfloat16()
    g = (0.01 * torch.randn(n, device="cuda")).bfloat16()
    m = (0.01 * torch.randn(n, device="cuda")).bfloat16()
    v = (1e-4 * torch.rand(n, device="cuda")).bfloat16()
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    kw = dict(lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, decay=0.1, step=3)
    E.adamw_reference(pr, g, mr, vr, clip=0.5, **kw)
    clip = torch.tensor(0.5, device="cuda")
    E.adamw_update(p, g, m, v, clip=clip, **kw)
    # fp32 arithmetic may contract differently (FMA); the stored bf16 state agrees to one ulp
    assert _rel(m, mr) < 4e-3 and _rel(v, vr) < 4e-3
    assert (p.float() - pr.float()).abs().max() <= 2 ** -7 * pr.float().abs().max()
    assert _rel(p, pr) < 1e-3


@pytest.mark.parametrize("grad_dtype", [torch.bfloat16, torch.float32])
def test_adamw_over_an_arena_of_regions_in_one_launch(cuda_lib, grad_dtype):
    """Decay, no-decay and frozen regions with boundaries both on and off the 8-element grid,
    against the fp32 PyTorch statement applied region by region."""
    from causal_trainer_dev_b200.ops import elementwise as E

    torch.manual_seed(5)
    n = 8 * 9000
    bounds = [0, 4096, 4099, 20000, 20008, 50001, n]
    modes = [0, 1, -1, 0, 1, -1]
    p = torch.randn(n, device="cuda").bfloat16()
    g = (0.01 * torch.randn(n, device="cuda")).to(grad_dtype)
    m = (0.01 * torch.randn(n, device="cuda")).bfloat16()
    v = (1e-4 * torch.rand(n, device="cuda")).bfloat16()
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    kw = dict(lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, step=2)
    for lo, hi, mode in zip(bounds[:-1], bounds[1:], modes):
        if mode >= 0:
            gr = g[lo:hi].bfloat16() if grad_dtype == torch.float32 else g[lo:hi]
            E.adamw_reference(pr[lo:hi], gr, mr[lo:hi], vr[lo:hi], clip=0.25, decay=0.1 if mode else 0.0, **kw)
    E.adamw_regions(p, g, m, v, torch.tensor(bounds, device="cuda"), torch.tensor(modes, dtype=torch.int32, device="cuda"),
                    decay=0.1, clip=torch.tensor(0.25, device="cuda"), round_bf16=grad_dtype == torch.float32, **kw)
    assert _rel(m, mr) < 4e-3 and _rel(v, vr) < 4e-3 and _rel(p, pr) < 1e-3
    for lo, hi, mode in zip(bounds[:-1], bounds[1:], modes):
        if mode < 0:   # frozen: bit-identical parameter and moments
            assert torch.equal(p[lo:hi], pr[lo:hi]) and torch.equal(m[lo:hi], mr[lo:hi]) and torch.equal(v[lo:hi], vr[lo:hi])


def test_active_row_compaction_is_stable_and_round_trips(cuda_lib):
    from causal_trainer_dev_b200.ops import elementwise as E

    torch.manual_seed(8)
    rows, d = 5000, 256
    w = (torch.rand(rows, device="cuda") > 0.6).float() * torch.rand(rows, device="cuda")
    w[0] = 0.7                                           # row 0 is active AND the padding target
    idx, total, n = E.active_rows(w)
    want = torch.nonzero(w != 0).reshape(-1)
    assert n == want.numel() == int(total) and idx.numel() == -(-n // 128) * 128
    assert torch.equal(idx[:n].long(), want) and not idx[n:].any()
    src = torch.randn(rows, d, device="cuda").bfloat16()
    packed = E.gather_rows(src, idx)
    assert torch.equal(packed[:n], src[want]) and torch.equal(packed[n:], src[:1].expand(idx.numel() - n, d))
    back = E.scatter_rows(packed, idx, total, rows)
    expect = torch.zeros_like(src)
    expect[want] = src[want]
    assert torch.equal(back, expect)                     # padding slots did not overwrite row 0
    none, _, n0 = E.active_rows(torch.zeros(300, device="cuda"))
    assert n0 == 0 and none.numel() == 0
