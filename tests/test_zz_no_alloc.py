"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some programs that load this library keep the whole GPU for their own memory pool, or sit on
a path where cudaMalloc's device-wide synchronisation is not acceptable; they cannot hand a
kernel a freshly allocated scratch buffer.  ``ctb_rmsnorm_bwd_noalloc`` serves them: its
scratch is a fixed array inside the library.  This test calls it twice in a row (second call:
other sizes, so leftovers of the first call sit in the shared array) and checks both results
against the regular entry point, which takes caller-allocated scratch.

The file name sorts last on purpose: under ``-x`` every other test has run before this one.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def _oracle(dy, x, w, rstd, dres, start, accumulate):
    """fp32 PyTorch statement of the same op."""
    xh = x.float() * rstd[:, None]
    gx = dy.float() * w.float()
    dx = rstd[:, None] * (gx - xh * (gx * xh).mean(-1, keepdim=True))
    if dres is not None:
        dx = dx + dres.float()
    dw = (dy.float() * xh).sum(0)
    return dx, (start.float() + dw if accumulate else dw)


def _both(lib, rows, d, seed, dres_given, accumulate, dw_kind="f32"):
    torch.manual_seed(seed)
    dy = torch.randn(rows, d, device="cuda").bfloat16()
    x = torch.randn(rows, d, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    dres = torch.randn(rows, d, device="cuda").bfloat16() if dres_given else None
    start = torch.randn(d, device="cuda")
    if dw_kind == "bf16":
        start = start.bfloat16()
    f32 = int(dw_kind == "f32")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())  # noqa: E731

    # regular entry point: scratch allocated by the caller
    parts = lib.ctb_rmsnorm_bwd_parts(rows)
    scratch = torch.empty(parts * d, dtype=torch.float32, device="cuda")
    dx_ref, dw_ref = torch.empty_like(x), (None if dw_kind == "none" else start.clone())
    assert lib.ctb_rmsnorm_bwd(ptr(dy), ptr(x), ptr(w), ptr(rstd), ptr(dres), ptr(dx_ref), ptr(scratch), ptr(dw_ref), f32,
                               int(accumulate), rows, d, stream) == 0
    # allocation-free entry point: nothing but inputs and outputs
    dx, dw = torch.empty_like(x), (None if dw_kind == "none" else start.clone())
    code = lib.ctb_rmsnorm_bwd_noalloc(ptr(dy), ptr(x), ptr(w), ptr(rstd), ptr(dres), ptr(dx), ptr(dw), f32,
                                       int(accumulate), rows, d, stream)
    assert code == 0, lib.ctb_noalloc_last_error().decode()
    torch.cuda.synchronize()
    return (dx, dw), (dx_ref, dw_ref), _oracle(dy, x, w, rstd, dres, start, accumulate)


def test_matches_regular_entry_point_on_two_calls_in_a_row(cuda_lib):
    lib = cuda_lib.lib()
    lib.ctb_noalloc_last_error.restype = ctypes.c_char_p
    for rows, d, seed, dres_given, accumulate in ((1500, 4096, 0, True, False), (333, 1536, 1, False, True)):
        (dx, dw), (dx_ref, dw_ref), (dx_o, dw_o) = _both(lib, rows, d, seed, dres_given, accumulate)
        assert _rel(dx, dx_ref) < 6e-3 and _rel(dw, dw_ref) < 6e-3
        assert _rel(dx, dx_o) < 6e-3 and _rel(dw, dw_o) < 6e-3          # and against plain fp32 PyTorch
        assert torch.isfinite(dw).all()


def test_bf16_weight_gradient_and_no_weight_gradient(cuda_lib):
    lib = cuda_lib.lib()
    lib.ctb_noalloc_last_error.restype = ctypes.c_char_p
    (dx, dw), (dx_ref, dw_ref), (dx_o, dw_o) = _both(lib, 700, 2048, 2, True, True, dw_kind="bf16")
    assert dw.dtype == torch.bfloat16 and _rel(dx, dx_o) < 6e-3
    assert _rel(dw, dw_ref) < 1e-2 and _rel(dw, dw_o) < 1e-2
    (dx, dw), (dx_ref, _), (dx_o, _) = _both(lib, 257, 1024, 3, False, False, dw_kind="none")
    assert dw is None and _rel(dx, dx_ref) < 6e-3 and _rel(dx, dx_o) < 6e-3


def test_a_pointer_into_the_middle_of_a_vector_is_refused(cuda_lib):
    """Nothing is launched: the refusal comes from the host-side argument check."""
    lib = cuda_lib.lib()
    lib.ctb_noalloc_last_error.restype = ctypes.c_char_p
    rows, d = 4, 64
    buf = torch.zeros(rows * d + 8, device="cuda", dtype=torch.bfloat16)
    good = ctypes.c_void_p(buf.data_ptr())
    odd = ctypes.c_void_p(buf.data_ptr() + 2)           # one bf16 element in: not on a 16-byte boundary
    rstd = torch.ones(rows, device="cuda")
    r = ctypes.c_void_p(rstd.data_ptr())
    for args in ((odd, good, good, r, None, good), (good, good, good, r, odd, good), (good, good, good, r, None, odd)):
        code = lib.ctb_rmsnorm_bwd_noalloc(*args, None, 1, 0, rows, d, None)
        assert code != 0 and b"16-byte aligned" in lib.ctb_noalloc_last_error()


def test_sizes_beyond_the_static_scratch_are_refused(cuda_lib):
    lib = cuda_lib.lib()
    lib.ctb_noalloc_last_error.restype = ctypes.c_char_p
    t = torch.zeros(8, device="cuda")
    p = ctypes.c_void_p(t.data_ptr())
    code = lib.ctb_rmsnorm_bwd_noalloc(p, p, p, p, None, p, p, 1, 0, 4, 16384, None)
    assert code != 0 and b"8192" in lib.ctb_noalloc_last_error()
