"""Python face of the tcgen05 GEMM family (``csrc/gemm.cu``).

``gemm(a, b)`` computes ``C[M,N] = alpha * A @ B^T (+ bias)`` for bf16 operands with
fp32 accumulation.  ``a_mn`` / ``b_mn`` say that the tensor passed holds the transpose
(``[K,M]`` / ``[K,N]`` row-major), which is how dgrad and wgrad read weights and
activations in place, without a transpose pass.

Reference counterpart: ``linear`` (src/causal_trainer/modeling/architecture.py:186-202),
whose three matmuls per projection XLA derives from one ``dot_general``.
"""
from __future__ import annotations

import ctypes

import torch

from . import lib as _lib


class FlagSource:
    """A gathered buffer that an all-gather pull is filling, with its per-chunk flags."""

    def __init__(self, buffer: torch.Tensor, flags: torch.Tensor, chunk_elems: int):
        self.start = buffer.data_ptr()
        self.end = self.start + buffer.numel() * buffer.element_size()
        self.flags = flags
        self.chunk_elems = chunk_elems
        self.epoch = 0
        self.spin_budget = 0
        self.complete = None        # torch.cuda.Event recorded after the pull; once it has fired
                                    # the buffer is plain memory and GEMMs skip the flags
        self.own_start = 0          # element range of the buffer that this rank owns (arrives first)
        self.own_stop = 0


_FLAG_SOURCES: list[FlagSource] = []


def register_flag_source(src: FlagSource) -> None:
    """GEMMs whose B operand lies inside ``src`` acquire its flags tile by tile."""
    _FLAG_SOURCES.append(src)


def unregister_flag_source(src: FlagSource) -> None:
    if src in _FLAG_SOURCES:
        _FLAG_SOURCES.remove(src)


def flag_source_of(t: torch.Tensor) -> tuple[FlagSource, int] | None:
    p = t.data_ptr()
    for src in _FLAG_SOURCES:
        if src.start <= p < src.end and src.epoch > 0:
            if src.complete is not None and src.complete.query():
                return None
            return src, (p - src.start) // t.element_size()
    return None


def _flag_args(hit):
    """(flags, chunk, base, epoch) of one operand for the C entry points (nulls when unflagged)."""
    if hit is None:
        return None, ctypes.c_long(0), ctypes.c_long(0), ctypes.c_uint(0)
    src, base = hit
    return _lib.ptr(src.flags), ctypes.c_long(src.chunk_elems), ctypes.c_long(base), ctypes.c_uint(src.epoch)


def _rotations(hit, hit_a, a, b, a_mn, b_mn, m, n) -> tuple[int, int]:
    """Tile-walk rotations that start a GEMM on the part of a gathered operand this rank owns.

    The pull delivers the rest in increasing (wrapping) rank order, which is the order the
    rotated walk needs it.
    """
    n_rotate = m_rotate = 0
    if hit is not None and not b_mn:
        src, base = hit
        if src.own_stop > src.own_start:
            first_own_row = max(0, -(-(src.own_start - base) // b.stride(0)))
            if first_own_row < n:
                n_rotate = -(-first_own_row // 256)
    if hit_a is not None and not a_mn:
        src, base = hit_a
        if src.own_stop > src.own_start:
            first_own_row = max(0, -(-(src.own_start - base) // a.stride(0)))
            if first_own_row < m:
                m_rotate = -(-first_own_row // 128)
    return n_rotate, m_rotate


def _check_operand(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1 or not t.is_cuda:
        raise ValueError(f"{name} must be a 2-D bf16 CUDA tensor with unit inner stride")


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype = torch.bfloat16,
    accumulate: bool = False,
    alpha: float = 1.0,
    bias: torch.Tensor | None = None,
    max_ctas: int = 0,
) -> torch.Tensor:
    _check_operand(a, "a")
    _check_operand(b, "b")
    m, k = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    n, kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if k != kb:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an existing `out`")
        out = torch.empty((m, n), dtype=out_dtype, device=a.device)
    if out.shape != (m, n) or out.stride(1) != 1 or out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("out must be [M,N] bf16/fp32 with unit inner stride")
    if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != n):
        raise ValueError("bias must be bf16 of length N")
    hit = flag_source_of(b) if _FLAG_SOURCES else None
    hit_a = flag_source_of(a) if _FLAG_SOURCES else None
    if hit is not None or hit_a is not None:
        n_rotate, m_rotate = _rotations(hit, hit_a, a, b, a_mn, b_mn, m, n)
        bf = _flag_args(hit)
        af = _flag_args(hit_a)
        budget = max(hit[0].spin_budget if hit else 0, hit_a[0].spin_budget if hit_a else 0)
        code = _lib.lib().ctb_gemm_flagged(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), m, n, k,
            ctypes.c_long(a.stride(0)), ctypes.c_long(b.stride(0)), ctypes.c_long(out.stride(0)),
            int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), ctypes.c_float(alpha),
            _lib.ptr(bias), *bf, 0, n_rotate, *af, m_rotate, ctypes.c_longlong(budget), max_ctas, _lib.stream_ptr(),
        )
        _lib.check(code, "ctb_gemm_flagged")
        return out
    code = _lib.lib().ctb_gemm(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), m, n, k,
        ctypes.c_long(a.stride(0)), ctypes.c_long(b.stride(0)), ctypes.c_long(out.stride(0)),
        int(a_mn), int(b_mn), int(out.dtype == torch.float32), int(accumulate), ctypes.c_float(alpha),
        _lib.ptr(bias), max_ctas, _lib.stream_ptr(),
    )
    _lib.check(code, "ctb_gemm")
    return out


def gemm_push(a: torch.Tensor, b: torch.Tensor, push, *, b_mn: bool = False, row_offset: int = 0,
              tiles_per_dest: int | None = None, alpha: float = 1.0, max_ctas: int = 0) -> None:
    """``A @ B^T`` whose bf16 partial-sum tiles go straight into the receive buffers of the ranks
    that own the rows (reduce-scatter by push, see ``GemmPush`` in ``csrc/gemm.h``).

    ``push`` describes the destination: ``dest_table``/``flag_table`` (int64 device tensors, one
    address per rank), ``world``, ``counters`` (int32 tensor), ``rows_per_rank``, ``src_rank``,
    ``ld``, ``epoch`` and ``spin_budget``.
    """
    _check_operand(a, "a")
    _check_operand(b, "b")
    m, k = a.shape
    n, kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    if k != kb:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    hit = flag_source_of(b) if _FLAG_SOURCES else None
    n_rotate, _ = _rotations(hit, None, a, b, False, b_mn, m, n)
    # every rank starts on the rows of its right-hand neighbour and finishes on its own, so the
    # receivers' inbound links are used evenly and nobody waits for a straggling last slab
    num_m = -(-m // 128)
    first = ((push.src_rank + 1) % push.world) * push.rows_per_rank - row_offset
    m_rotate = (first // 128) % num_m if 0 <= first < m else 0
    if tiles_per_dest is None:
        tiles_per_dest = (push.rows_per_rank // 128) * (-(-n // 256))
    code = _lib.lib().ctb_gemm_push(
        _lib.ptr(a), _lib.ptr(b), m, n, k, ctypes.c_long(a.stride(0)), ctypes.c_long(b.stride(0)), 0, int(b_mn),
        ctypes.c_float(alpha), _lib.ptr(push.dest_table), _lib.ptr(push.flag_table), _lib.ptr(push.counters),
        push.rows_per_rank, row_offset, push.src_rank, tiles_per_dest, ctypes.c_long(push.ld),
        ctypes.c_uint(push.epoch), *_flag_args(hit), 0, n_rotate, m_rotate, ctypes.c_longlong(push.spin_budget),
        max_ctas, _lib.stream_ptr(),
    )
    _lib.check(code, "ctb_gemm_push")


def linear_forward(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``y[T,out] = x[T,in] @ w[out,in]^T (+ bias)``."""
    return gemm(x, w, bias=bias)


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``dx[T,in] = dy[T,out] @ w[out,in]`` reading ``w`` in place."""
    return gemm(dy, w, b_mn=True)


def linear_wgrad(
    dy: torch.Tensor, x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False,
    out_dtype: torch.dtype = torch.bfloat16,
) -> torch.Tensor:
    """``dw[out,in] (+)= dy[T,out]^T @ x[T,in]`` reading both in place."""
    return gemm(dy, x, a_mn=True, b_mn=True, out=out, accumulate=accumulate, out_dtype=out_dtype)


def lora_merge(w: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Merged projection weight ``W + (A @ B)^T`` for export (no alpha: the reference's convention,
    src/causal_trainer/modeling/lora.py:279-295).

    ``w`` is ``[out, in]``, ``a`` ``[in, r]``, ``b`` ``[r, out]`` (bf16, CUDA).  The rank-r update
    runs on the tcgen05 GEMM with fp32 accumulation straight into an fp32 copy of ``w`` (TMA
    reduce-add epilogue); the result is rounded once to ``w``'s dtype.
    """
    out_f, in_f = w.shape
    r = a.shape[1]
    if a.shape[0] != in_f or b.shape != (r, out_f):
        raise ValueError("adapter shapes do not match the projection")
    pad = (-r) % 8                    # leading dimensions must be multiples of 16 bytes
    bt = b.t().contiguous().to(torch.bfloat16)            # [out, r]  K-major A operand
    at = a.contiguous().to(torch.bfloat16)                # [in, r]   K-major B operand
    if pad:
        bt = torch.nn.functional.pad(bt, (0, pad))
        at = torch.nn.functional.pad(at, (0, pad))
    acc = w.float()
    gemm(bt, at, out=acc, accumulate=True)
    return acc.to(w.dtype)
