"""Out-of-bounds writes and unsynchronised accumulation, looked for without a sanitizer.

Outputs of the kernels are placed between guard bands filled with a pattern; after the launch the
bands must be untouched.  Shapes are ragged on purpose (rows and columns that are not multiples of
the tile sizes, documents that start off the 128-token grid).  Index kernels that read row numbers
from device memory are given a bad index: they must record it in the status word and skip the row.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BAND = 4096          # elements of guard band on each side


class Guarded:
    """A tensor of ``shape`` carved out of a larger buffer whose margins hold a canary pattern."""

    def __init__(self, shape, dtype=torch.bfloat16, row_stride=None):
        numel = math.prod(shape) if row_stride is None else shape[0] * row_stride
        self.buf = torch.empty(numel + 2 * BAND, dtype=dtype, device="cuda")
        self.pattern = 1.25 if dtype.is_floating_point else 77
        self.buf.fill_(self.pattern)
        inner = self.buf[BAND:BAND + numel]
        if row_stride is None:
            self.view = inner.view(shape)
        else:                                     # rows with slack between them: the slack is guarded too
            self.view = inner.view(shape[0], row_stride)[:, :math.prod(shape[1:])].view(shape)
        self.numel, self.shape, self.row_stride = numel, shape, row_stride

    def intact(self) -> bool:
        ok = bool((self.buf[:BAND] == self.pattern).all() and (self.buf[BAND + self.numel:] == self.pattern).all())
        if self.row_stride is not None:
            width = math.prod(self.shape[1:])
            slack = self.buf[BAND:BAND + self.numel].view(self.shape[0], self.row_stride)[:, width:]
            ok = ok and bool((slack == self.pattern).all())
        return ok


def test_gemm_outputs_stay_inside_their_rows(cuda_lib):
    from causal_trainer_dev_b200.ops import gemm as G

    torch.manual_seed(0)
    for m, n, k in ((1000, 520, 264), (130, 8, 4104), (257, 1288, 72)):
        a = torch.randn(m, k, device="cuda").bfloat16()
        b = torch.randn(n, k, device="cuda").bfloat16()
        out = Guarded((m, n), row_stride=n + 24)           # ldc > N: columns beyond N belong to someone else
        G.gemm(a, b, out=out.view)
        ref = a.float() @ b.float().t()
        assert out.intact(), (m, n, k)
        assert ((out.view.float() - ref).norm() / ref.norm()) < 6e-3
        acc = Guarded((m, n), dtype=torch.float32, row_stride=n + 12)
        acc.view.zero_()
        G.gemm(a, b, out=acc.view, accumulate=True)
        assert acc.intact() and ((acc.view - ref).norm() / ref.norm()) < 1e-3


def test_attention_outputs_stay_inside_their_tensors(cuda_lib):
    from causal_trainer_dev_b200.ops.attention import build_attention_meta, flash_attention_backward, flash_attention_forward

    torch.manual_seed(1)
    b, s, hq, hkv, d = 2, 640, 4, 2, 128
    seg = torch.zeros(b, s, dtype=torch.int32, device="cuda")
    seg[0, :333] = 1
    seg[0, 333:601] = 2                                       # documents off the 128-token grid, padded tail
    seg[1, 7:640] = 1
    q = torch.randn(b, s, hq, d, device="cuda").bfloat16()
    k = torch.randn(b, s, hkv, d, device="cuda").bfloat16()
    v = torch.randn(b, s, hkv, d, device="cuda").bfloat16()
    meta = build_attention_meta(seg, None)
    o = Guarded((b, s, hq, d))
    out, lse = flash_attention_forward(q, k, v, meta, out=o.view)
    assert o.intact()
    dq, dk, dv = Guarded((b, s, hq, d)), Guarded((b, s, hkv, d)), Guarded((b, s, hkv, d))
    do = torch.randn_like(out)
    flash_attention_backward(q, k, v, out, do, lse, meta, dq=dq.view, dk=dk.view, dv=dv.view)
    assert dq.intact() and dk.intact() and dv.intact()
    again = Guarded((b, s, hkv, d))
    flash_attention_backward(q, k, v, out, do, lse, meta, dq=dq.view, dk=again.view, dv=dv.view)
    assert torch.equal(again.view, dk.view)                   # run twice, bit-compare: no unordered accumulation


def test_norm_embedding_and_optimizer_kernels_stay_in_bounds(cuda_lib):
    from causal_trainer_dev_b200.ops import elementwise as E

    torch.manual_seed(2)
    rows, d = 777, 1544
    x = torch.randn(rows, d, device="cuda").bfloat16()
    w = torch.ones(d, device="cuda").bfloat16()
    y, rstd, _ = E.rmsnorm_forward(x, w, 1e-6)
    dx = Guarded((rows, d))
    dw = Guarded((d,), dtype=torch.float32)
    E.rmsnorm_backward(y, x, w, rstd, dw_out=dw.view, dx_out=dx.view)
    assert dx.intact() and dw.intact()
    n = 8 * 1237
    p, m, v = Guarded((n,)), Guarded((n,)), Guarded((n,))
    for t in (p, m, v):
        t.view.copy_(torch.rand(n, device="cuda"))
    g = torch.randn(n, device="cuda").bfloat16()
    E.adamw_regions(p.view, g, m.view, v.view, torch.tensor([0, 1000, n], device="cuda"),
                    torch.tensor([0, 1], dtype=torch.int32, device="cuda"), lr=1e-3, b1=0.9, b2=0.999, eps=1e-8,
                    decay=0.1, step=1)
    assert p.intact() and m.intact() and v.intact()


def test_row_kernels_report_a_bad_index_and_skip_it(cuda_lib):
    from causal_trainer_dev_b200.ops import elementwise as E

    cuda_lib.device_status(raise_on_error=False)
    rows, d = 300, 64
    src = torch.randn(rows, d, device="cuda").bfloat16()
    idx = torch.tensor([5, 299, 300, -1, 17], dtype=torch.int32, device="cuda")      # two of them out of range
    out = E.gather_rows(src, idx)
    failure = cuda_lib.poll_device_status()
    assert failure is not None and "row gather" in str(failure)
    assert torch.equal(out[[0, 1, 4]], src[[5, 299, 17]]) and not out[[2, 3]].any()
    dst = Guarded((rows, d))
    dst.view.zero_()
    total = torch.tensor([5], dtype=torch.int32, device="cuda")
    code = cuda_lib.lib().ctb_scatter_rows(cuda_lib.ptr(out), cuda_lib.ptr(idx), cuda_lib.ptr(total), cuda_lib.ptr(dst.view),
                                           E._l(d), rows, E._l(5), d, cuda_lib.stream_ptr())
    cuda_lib.check(code, "ctb_scatter_rows")
    failure = cuda_lib.poll_device_status()
    assert failure is not None and "row scatter" in str(failure) and dst.intact()
    assert torch.equal(dst.view[[5, 299, 17]], src[[5, 299, 17]])
    assert cuda_lib.poll_device_status() is None
