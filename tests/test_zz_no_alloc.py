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


def _both(lib, rows, d, seed, dres_given, accumulate):
    torch.manual_seed(seed)
    dy = torch.randn(rows, d, device="cuda").bfloat16()
    x = torch.randn(rows, d, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6)
    dres = torch.randn(rows, d, device="cuda").bfloat16() if dres_given else None
    start = torch.randn(d, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())  # noqa: E731

    # regular entry point: scratch allocated by the caller
    parts = lib.ctb_rmsnorm_bwd_parts(rows)
    scratch = torch.empty(parts * d, dtype=torch.float32, device="cuda")
    dx_ref, dw_ref = torch.empty_like(x), start.clone()
    assert lib.ctb_rmsnorm_bwd(ptr(dy), ptr(x), ptr(w), ptr(rstd), ptr(dres), ptr(dx_ref), ptr(scratch), ptr(dw_ref), 1,
                               int(accumulate), rows, d, stream) == 0
    # allocation-free entry point: nothing but inputs and outputs
    dx, dw = torch.empty_like(x), start.clone()
    code = lib.ctb_rmsnorm_bwd_noalloc(ptr(dy), ptr(x), ptr(w), ptr(rstd), ptr(dres), ptr(dx), ptr(dw), 1,
                                       int(accumulate), rows, d, stream)
    assert code == 0, lib.ctb_noalloc_last_error().decode()
    torch.cuda.synchronize()
    return (dx, dw), (dx_ref, dw_ref)


def test_matches_regular_entry_point_on_two_calls_in_a_row(cuda_lib):
    lib = cuda_lib.lib()
    lib.ctb_noalloc_last_error.restype = ctypes.c_char_p
    for rows, d, seed, dres_given, accumulate in ((1500, 4096, 0, True, False), (333, 1536, 1, False, True)):
        (dx, dw), (dx_ref, dw_ref) = _both(lib, rows, d, seed, dres_given, accumulate)
        assert _rel(dx, dx_ref) < 6e-3 and _rel(dw, dw_ref) < 6e-3
        assert torch.isfinite(dw).all()


def test_sizes_beyond_the_static_scratch_are_refused(cuda_lib):
    lib = cuda_lib.lib()
    lib.ctb_noalloc_last_error.restype = ctypes.c_char_p
    t = torch.zeros(8, device="cuda")
    p = ctypes.c_void_p(t.data_ptr())
    code = lib.ctb_rmsnorm_bwd_noalloc(p, p, p, p, None, p, p, 1, 0, 4, 16384, None)
    assert code != 0 and b"8192" in lib.ctb_noalloc_last_error()
