"""tcgen05 GEMM family against an fp32 PyTorch matmul of the same operands."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("a_mn", [False, True])
@pytest.mark.parametrize("b_mn", [False, True])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (200, 328, 136), (1000, 520, 72)])
def test_layouts(cuda_lib, a_mn, b_mn, shape):
    from causal_trainer_dev_b200.ops import gemm as G

    m, n, k = shape
    torch.manual_seed(1)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    out = G.gemm(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, a_mn=a_mn, b_mn=b_mn)
    assert _rel(out, ref) < 4e-3
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_fp32_out_accumulate_bias_alpha(cuda_lib):
    from causal_trainer_dev_b200.ops import gemm as G

    torch.manual_seed(2)
    a = torch.randn(384, 192, device="cuda").bfloat16()
    b = torch.randn(520, 192, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    out = G.gemm(a, b, out_dtype=torch.float32)
    assert _rel(out, ref) < 1e-5
    acc = torch.randn(384, 520, device="cuda")
    expect = acc + 0.5 * ref
    G.gemm(a, b, out=acc, accumulate=True, alpha=0.5)
    assert _rel(acc, expect) < 1e-5
    bias = torch.randn(520, device="cuda").bfloat16()
    out = G.gemm(a, b, bias=bias)
    assert _rel(out, ref + bias.float()) < 4e-3
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_linear_triplet_matches_autograd(cuda_lib):
    from causal_trainer_dev_b200.ops import gemm as G

    torch.manual_seed(3)
    x = torch.randn(640, 256, device="cuda").bfloat16()
    w = torch.randn(384, 256, device="cuda").bfloat16()
    dy = torch.randn(640, 384, device="cuda").bfloat16()
    assert _rel(G.linear_forward(x, w), x.float() @ w.float().t()) < 4e-3
    assert _rel(G.linear_dgrad(dy, w), dy.float() @ w.float()) < 4e-3
    assert _rel(G.linear_wgrad(dy, x), dy.float().t() @ x.float()) < 4e-3


def test_lora_merge_matches_fp32_reference(cuda_lib):
    from causal_trainer_dev_b200.ops.gemm import lora_merge

    torch.manual_seed(5)
    for out_f, in_f, r in ((512, 384, 16), (256, 1024, 12)):
        w = (torch.randn(out_f, in_f, device="cuda") * 0.05).bfloat16()
        a = (torch.randn(in_f, r, device="cuda") * 0.1).bfloat16()
        b = (torch.randn(r, out_f, device="cuda") * 0.1).bfloat16()
        ref = (w.float() + (a.float() @ b.float()).t()).bfloat16()
        got = lora_merge(w, a, b)
        assert (got.float() - ref.float()).abs().max() <= 2 * ref.float().abs().max() * 2 ** -8


@pytest.mark.parametrize("shape", [(512, 512, 8192), (4096, 1024, 16384), (640, 328, 4104)])
def test_split_k_weight_gradient_shapes(cuda_lib, shape):
    """Few output tiles and a long K (dy^T x): the K slices reduce-add into one output."""
    from causal_trainer_dev_b200.ops import gemm as G

    m, n, k = shape
    torch.manual_seed(5)
    before = cuda_lib.lib().ctb_gemm_set_split_k(1)
    try:
        _check_split_k(G, m, n, k)
    finally:
        cuda_lib.lib().ctb_gemm_set_split_k(before)
    assert cuda_lib.device_status() == (0, 0, 0, 0)


@pytest.mark.parametrize("shape", [(4096, 14336, 2048), (4096, 14336, 8192), (4000, 14400, 4104), (4096, 28672, 4096)])
def test_tail_split_of_a_mostly_empty_last_wave(cuda_lib, shape):
    """fp32 weight-gradient shapes whose tiles leave a small last wave: those tiles are cut into
    K slices that reduce-add into C (first write and accumulation), the others stay whole."""
    from causal_trainer_dev_b200.ops import gemm as G

    m, n, k = shape
    torch.manual_seed(6)
    dy = (torch.randn(k, m, device="cuda") * 0.5).bfloat16()
    x = (torch.randn(k, n, device="cuda") * 0.5).bfloat16()
    ref = dy.float().t() @ x.float()
    before = cuda_lib.lib().ctb_gemm_set_tail_split(1)
    try:
        out = torch.full((m, n), 7.0, device="cuda")               # overwritten, not accumulated
        G.gemm(dy, x, a_mn=True, b_mn=True, out=out)
        assert _rel(out, ref) < 1e-4
        # every 256 x 256 block on its own: a tile that was skipped or added twice does not hide in the norm
        blocks = (out - ref).abs().unfold(0, 128, 128).unfold(1, 128, 128).amax(dim=(-1, -2))
        assert float(blocks.max()) < 0.05 * float(ref.abs().max())
        G.gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=True)
        assert _rel(out, 2 * ref) < 1e-4
        view = torch.full((m + 64, n + 64), 3.0, device="cuda")    # a strided destination keeps its frame
        G.gemm(dy, x, a_mn=True, b_mn=True, out=view[:m, :n])
        assert _rel(view[:m, :n], ref) < 1e-4
        assert bool((view[m:, :] == 3.0).all()) and bool((view[:, n:] == 3.0).all())
    finally:
        cuda_lib.lib().ctb_gemm_set_tail_split(before)
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def _check_split_k(G, m, n, k):
    dy = (torch.randn(k, m, device="cuda") * 0.5).bfloat16()       # [tokens, out]
    x = (torch.randn(k, n, device="cuda") * 0.5).bfloat16()        # [tokens, in]
    ref = dy.float().t() @ x.float()
    out32 = torch.full((m, n), 7.0, device="cuda")                 # overwritten, not accumulated
    G.gemm(dy, x, a_mn=True, b_mn=True, out=out32)
    assert _rel(out32, ref) < 1e-4
    G.gemm(dy, x, a_mn=True, b_mn=True, out=out32, accumulate=True)
    assert _rel(out32, 2 * ref) < 1e-4
    out16 = torch.full((m, n), 7.0, device="cuda").bfloat16()
    G.gemm(dy, x, a_mn=True, b_mn=True, out=out16)
    assert _rel(out16, ref) < 8e-3
    # K-major operands take the same path
    out = G.gemm(dy.t().contiguous(), x.t().contiguous(), out_dtype=torch.float32)
    assert _rel(out, ref) < 1e-4


@pytest.mark.parametrize("shape", [(4864, 4864, 512), (5000, 4936, 520)])
def test_two_cta_pair_kernel_matches_reference(cuda_lib, shape):
    """tcgen05.mma.cta_group::2 on clusters of two CTAs: all operand layouts, bf16 / fp32 out, accumulate."""
    from causal_trainer_dev_b200.ops import gemm as G

    m, n, k = shape
    torch.manual_seed(7)
    a = torch.randn(m, k, device="cuda").bfloat16()
    b = torch.randn(n, k, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    before = cuda_lib.lib().ctb_gemm_set_pair(1)
    try:
        for a_mn in (False, True):
            for b_mn in (False, True):
                out = G.gemm(a.t().contiguous() if a_mn else a, b.t().contiguous() if b_mn else b, a_mn=a_mn, b_mn=b_mn)
                assert _rel(out, ref) < 4e-3, (a_mn, b_mn)
        acc = torch.randn(m, n, device="cuda")
        expect = acc + 0.5 * ref
        G.gemm(a, b, out=acc, accumulate=True, alpha=0.5)
        assert _rel(acc, expect) < 1e-5
    finally:
        cuda_lib.lib().ctb_gemm_set_pair(before)
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_low_rank_shapes_and_bf16_accumulation_into_a_column_slice(cuda_lib):
    """The adapter products of LoRA: K or N as small as 16, results added into a slice of a wider
    bf16 matrix (reduce-add epilogue) and into fp32 gradient buffers."""
    from causal_trainer_dev_b200.ops import gemm as G

    torch.manual_seed(11)
    t, d_in, d_out, r = 1000, 512, 768, 16
    x = (torch.randn(t, d_in, device="cuda") * 0.5).bfloat16()
    a = (torch.randn(d_in, r, device="cuda") * 0.1).bfloat16()
    b = (torch.randn(r, d_out, device="cuda") * 0.1).bfloat16()
    y = torch.randn(t, 2 * d_out, device="cuda").bfloat16()
    want = y.float().clone()
    low = G.gemm(x, a, b_mn=True)                                         # x @ a
    assert _rel(low, x.float() @ a.float()) < 4e-3
    want[:, d_out:] += low.float() @ b.float()
    G.gemm(low, b, b_mn=True, out=y[:, d_out:], accumulate=True)          # y[:, slice] += low @ b
    assert _rel(y, want) < 6e-3 and torch.equal(y[:, :d_out].float(), want[:, :d_out])
    dy = torch.randn(t, 2 * d_out, device="cuda").bfloat16()
    dys = dy[:, d_out:]
    dt = G.gemm(dys, b)                                                   # dy @ b^T
    assert _rel(dt, dys.float() @ b.float().t()) < 4e-3
    gb = torch.zeros(r, d_out, device="cuda")
    G.gemm(low, dys, a_mn=True, b_mn=True, out=gb)                        # low^T @ dy
    assert _rel(gb, low.float().t() @ dys.float()) < 1e-3
    ga = torch.ones(d_in, r, device="cuda")
    G.gemm(x, dt, a_mn=True, b_mn=True, out=ga, accumulate=True)          # += x^T @ dt
    assert _rel(ga, 1 + x.float().t() @ dt.float()) < 1e-3
    dx = torch.randn(t, d_in, device="cuda").bfloat16()
    want_dx = dx.float() + dt.float() @ a.float().t()
    G.gemm(dt, a, out=dx, accumulate=True)                                # dx += dt @ a^T
    assert _rel(dx, want_dx) < 6e-3
    assert cuda_lib.device_status() == (0, 0, 0, 0)
