"""Python face of ``csrc/elementwise.cu`` plus PyTorch reference versions of the same ops.

Every op has two entry points: ``<op>`` runs the sm_100a kernel on bf16 CUDA tensors and
``<op>_reference`` is the plain PyTorch statement of the same math, used on CPU and as the
oracle in GPU tests.  Semantics follow the reference trainer:

* RMSNorm: fp32 mean square, normalised value cast to the compute dtype *before* the scale
  (src/causal_trainer/modeling/architecture.py:155-162);
* RoPE: fp32 angles from arbitrary integer positions, table cast to the compute dtype once
  per step, only the first ``rotary_dim`` channels rotated, two pairings
  (src/causal_trainer/modeling/rotary.py:53-60, 132-204);
* SwiGLU: ``silu(gate) * up`` (architecture.py:205-229);
* AdamW: moments in the parameter dtype, update cast to the parameter dtype before the add
  (src/causal_trainer/training/steps.py:173-186, optimizer.py:53-75).
"""
from __future__ import annotations

import ctypes

import torch

from . import lib as _lib

_f = ctypes.c_float
_l = ctypes.c_long


# ------------------------------------------------------------------------------ RMSNorm
def rmsnorm_reference(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    normed = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)
    return (normed * w.to(x.dtype)).to(x.dtype)


def rmsnorm_forward(x, w, eps, residual=None, out=None):
    """Returns (y, rstd, h) where h = x + residual (or x itself); ``out`` receives y when given."""
    rows, d = x.shape
    y = torch.empty_like(x) if out is None else out
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    h = torch.empty_like(x) if residual is not None else x
    code = _lib.lib().ctb_rmsnorm_fwd(
        _lib.ptr(x), _lib.ptr(residual), _lib.ptr(w), _lib.ptr(y), _lib.ptr(h if residual is not None else None),
        _lib.ptr(rstd), rows, d, _f(eps), _lib.stream_ptr(),
    )
    _lib.check(code, "ctb_rmsnorm_fwd")
    return y, rstd, h


_norm_scratch: dict[tuple[int, int], torch.Tensor] = {}


def rmsnorm_backward(dy, x, w, rstd, dres=None, dw_out=None, dw_accumulate=False, dx_out=None):
    """Returns (dx, dw).  ``dx`` includes ``dres`` when given (the residual branch gradient)."""
    rows, d = x.shape
    L = _lib.lib()
    parts = L.ctb_rmsnorm_bwd_parts(rows)
    key = (x.device.index or 0, parts * d)
    scratch = _norm_scratch.get(key)
    if scratch is None:
        scratch = torch.empty(parts * d, dtype=torch.float32, device=x.device)
        _norm_scratch[key] = scratch
    dx = torch.empty_like(x) if dx_out is None else dx_out
    if dw_out is None:
        dw_out = torch.empty(d, dtype=torch.float32, device=x.device)
        dw_accumulate = False
    code = L.ctb_rmsnorm_bwd(
        _lib.ptr(dy), _lib.ptr(x), _lib.ptr(w), _lib.ptr(rstd), _lib.ptr(dres), _lib.ptr(dx), _lib.ptr(scratch),
        _lib.ptr(dw_out), int(dw_out.dtype == torch.float32), int(dw_accumulate), rows, d, _lib.stream_ptr(),
    )
    _lib.check(code, "ctb_rmsnorm_bwd")
    return dx, dw_out


# ------------------------------------------------------------------------------ RoPE
def inverse_frequencies(rotary_dim: int, theta: float, device=None) -> torch.Tensor:
    channels = torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=device)
    return 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32, device=device), channels / rotary_dim)


def rope_table_reference(position_ids: torch.Tensor, inv_freq: torch.Tensor, dtype: torch.dtype):
    """cos/sin [T, rot/2] rounded to the compute dtype, kept in fp32 storage."""
    ang = position_ids.reshape(-1, 1).float() * inv_freq[None, :].float()
    return torch.cos(ang).to(dtype).float(), torch.sin(ang).to(dtype).float()


def rope_table(position_ids: torch.Tensor, inv_freq: torch.Tensor):
    pos = position_ids.reshape(-1).to(torch.int32).contiguous()
    t, half = pos.numel(), inv_freq.numel()
    cos = torch.empty((t, half), dtype=torch.float32, device=pos.device)
    sin = torch.empty_like(cos)
    code = _lib.lib().ctb_rope_table(_lib.ptr(pos), _lib.ptr(inv_freq), _lib.ptr(cos), _lib.ptr(sin), t, half,
                                     _lib.stream_ptr())
    _lib.check(code, "ctb_rope_table")
    return cos, sin


def rope_reference(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int, style: str,
                   inverse: bool = False) -> torch.Tensor:
    """x [T,H,D]; cos/sin [T, rot/2].  Returns a rotated copy."""
    xf = x.float()
    rot, rest = xf[..., :rotary_dim], xf[..., rotary_dim:]
    c, s = cos[:, None, :], sin[:, None, :] * (-1.0 if inverse else 1.0)
    if style == "gpt-j":
        a, b = rot[..., 0::2], rot[..., 1::2]
        out = torch.stack((a * c - b * s, b * c + a * s), dim=-1).reshape(rot.shape)
    else:
        a, b = rot[..., : rotary_dim // 2], rot[..., rotary_dim // 2:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return torch.cat((out, rest), dim=-1).to(x.dtype)


def rope_inplace(x2d: torch.Tensor, cos, sin, heads: int, head_dim: int, rotary_dim: int, style: str,
                 inverse: bool = False, col_offset: int = 0) -> None:
    """Rotates ``heads`` heads starting at column ``col_offset`` of the packed rows in place."""
    t = x2d.shape[0]
    base = x2d[:, col_offset:]
    code = _lib.lib().ctb_rope(
        _lib.ptr(base), _lib.ptr(cos), _lib.ptr(sin), _l(x2d.stride(0)), t, heads, head_dim, rotary_dim,
        0 if style == "gpt-j" else 1, int(inverse), _lib.stream_ptr(),
    )
    _lib.check(code, "ctb_rope")


# ------------------------------------------------------------------------------ SwiGLU
def swiglu_reference(gu: torch.Tensor) -> torch.Tensor:
    f = gu.shape[-1] // 2
    g, u = gu[..., :f], gu[..., f:]
    return (torch.nn.functional.silu(g.float()).to(gu.dtype) * u).to(gu.dtype)


def swiglu_forward(gu: torch.Tensor) -> torch.Tensor:
    t, f2 = gu.shape
    h = torch.empty((t, f2 // 2), dtype=gu.dtype, device=gu.device)
    _lib.check(_lib.lib().ctb_swiglu_fwd(_lib.ptr(gu), _lib.ptr(h), _l(t), f2 // 2, _lib.stream_ptr()), "ctb_swiglu_fwd")
    return h


def swiglu_backward(gu: torch.Tensor, dh: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    t, f2 = gu.shape
    dgu = torch.empty_like(gu) if out is None else out
    _lib.check(_lib.lib().ctb_swiglu_bwd(_lib.ptr(gu), _lib.ptr(dh), _lib.ptr(dgu), _l(t), f2 // 2, _lib.stream_ptr()),
               "ctb_swiglu_bwd")
    return dgu


# ------------------------------------------------------------------------------ embedding / delta
def embedding_gather(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    flat = ids.reshape(-1).to(torch.int32).contiguous()
    out = torch.empty((flat.numel(), table.shape[1]), dtype=table.dtype, device=table.device)
    code = _lib.lib().ctb_embedding_gather(_lib.ptr(flat), _lib.ptr(table), _lib.ptr(out), _l(flat.numel()),
                                           table.shape[1], table.shape[0], _lib.stream_ptr())
    _lib.check(code, "ctb_embedding_gather")
    return out


def embedding_backward(ids: torch.Tensor, dout: torch.Tensor, grad: torch.Tensor, pad_id: int, vocab_lo: int = 0) -> None:
    """``grad[id - vocab_lo] += sum of dout rows whose token is id`` (deterministic; pad row skipped).

    ``grad`` is the ``[rows, d]`` gradient table of the embedding rows ``[vocab_lo, vocab_lo + rows)``
    (bf16 or fp32); tokens outside that range belong to another vocabulary shard and are ignored.
    """
    flat = ids.reshape(-1).to(torch.int32)
    order = torch.sort(flat, stable=True)
    sorted_ids = order.values.contiguous()
    perm = order.indices.to(torch.int32).contiguous()
    change = torch.ones_like(sorted_ids, dtype=torch.bool)
    change[1:] = sorted_ids[1:] != sorted_ids[:-1]
    starts = torch.nonzero(change).reshape(-1).to(torch.int32).contiguous()
    code = _lib.lib().ctb_embedding_backward(_lib.ptr(sorted_ids), _lib.ptr(perm), _lib.ptr(starts), starts.numel(),
                                             _l(flat.numel()), _lib.ptr(dout), _lib.ptr(grad),
                                             int(grad.dtype == torch.float32), dout.shape[1], vocab_lo, grad.shape[0],
                                             pad_id, _lib.stream_ptr())
    _lib.check(code, "ctb_embedding_backward")


def attention_delta(o: torch.Tensor, dout: torch.Tensor) -> torch.Tensor:
    """delta[b,h,s] = sum_d O*dO for [B,S,H,D] views."""
    b, s, h, d = o.shape
    delta = torch.empty((b, h, s), dtype=torch.float32, device=o.device)
    code = _lib.lib().ctb_attn_delta(_lib.ptr(o), _lib.ptr(dout), _lib.ptr(delta), b, s, h, d, _l(o.stride(1)),
                                     _l(dout.stride(1)), _lib.stream_ptr())
    _lib.check(code, "ctb_attn_delta")
    return delta


def attention_backward_stats(o: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``(-lse * log2(e), -sum_d O*dO)``, both [B,H,S] fp32: the per-query statistics in the form the
    flash backward kernels consume (packed fma / add, no negation in their inner loops)."""
    b, s, h, d = o.shape
    neg_lse2 = torch.empty((b, h, s), dtype=torch.float32, device=o.device)
    neg_delta = torch.empty_like(neg_lse2)
    code = _lib.lib().ctb_attn_bwd_stats(_lib.ptr(o), _lib.ptr(dout), _lib.ptr(lse), _lib.ptr(neg_lse2),
                                         _lib.ptr(neg_delta), b, s, h, d, _l(o.stride(1)), _l(dout.stride(1)),
                                         _lib.stream_ptr())
    _lib.check(code, "ctb_attn_bwd_stats")
    return neg_lse2, neg_delta


# ------------------------------------------------------------------------------ optimizer pieces
def sum_of_squares(x: torch.Tensor, round_bf16: bool = False) -> torch.Tensor:
    """fp32 scalar tensor on the device (no host sync).

    ``round_bf16`` squares the bf16 rounding of fp32 elements: the norm of gradients cast to
    the parameter dtype, without writing the cast anywhere."""
    L = _lib.lib()
    parts = L.ctb_sumsq_parts()
    partial = torch.empty(parts, dtype=torch.float32, device=x.device)
    flat = x.reshape(-1)
    _lib.check(L.ctb_sumsq(_lib.ptr(flat), _l(flat.numel()), int(x.dtype == torch.float32), int(round_bf16),
                           _lib.ptr(partial),
                           _lib.stream_ptr()), "ctb_sumsq")
    return partial.sum()


def adamw_reference(p, g, m, v, *, lr, b1, b2, eps, decay, step, clip=1.0, gscale=1.0):
    """In-place reference update (fp32 arithmetic, parameter-dtype state)."""
    gf = g.float() * (clip * gscale)
    mf = b1 * m.float() + (1 - b1) * gf
    vf = b2 * v.float() + (1 - b2) * gf * gf
    upd = -lr * ((mf / (1 - b1 ** step)) / (torch.sqrt(vf / (1 - b2 ** step)) + eps) + decay * p.float())
    m.copy_(mf.to(m.dtype))
    v.copy_(vf.to(v.dtype))
    p.copy_((p.float() + upd.to(p.dtype).float()).to(p.dtype))


def adamw_update(p, g, m, v, *, lr, b1, b2, eps, decay, step, clip: torch.Tensor | None = None, gscale=1.0,
                 round_bf16: bool = False) -> None:
    n = p.numel()
    code = _lib.lib().ctb_adamw(
        _lib.ptr(p), _lib.ptr(g), int(g.dtype == torch.float32), _lib.ptr(m), _lib.ptr(v), _l(n), _f(lr), _f(b1),
        _f(b2), _f(eps), _f(decay), _f(1 - b1 ** step), _f(1 - b2 ** step), _lib.ptr(clip), _f(gscale),
        int(round_bf16), _lib.stream_ptr(),
    )
    _lib.check(code, "ctb_adamw")


def adamw_regions(p, g, m, v, bounds: torch.Tensor, modes: torch.Tensor, *, lr, b1, b2, eps, decay, step,
                  clip: torch.Tensor | None = None, gscale=1.0, round_bf16: bool = False) -> None:
    """AdamW over a flat bf16 arena in ONE launch (16-byte accesses).  ``bounds`` (int64, device,
    ``[R + 1]``) cuts the arena into regions and ``modes`` (int32, device, ``[R]``) says what each
    gets: 1 weight decay, 0 no decay, -1 frozen (skipped, moments untouched).  Same arithmetic as
    :func:`adamw_update` (src/causal_trainer/training/optimizer.py:42-75)."""
    code = _lib.lib().ctb_adamw_regions(
        _lib.ptr(p), _lib.ptr(g), int(g.dtype == torch.float32), _lib.ptr(m), _lib.ptr(v), _l(p.numel()),
        _lib.ptr(bounds), _lib.ptr(modes), int(modes.numel()), _f(lr), _f(b1), _f(b2), _f(eps), _f(decay),
        _f(1 - b1 ** step), _f(1 - b2 ** step), _lib.ptr(clip), _f(gscale), int(round_bf16), _lib.stream_ptr())
    _lib.check(code, "ctb_adamw_regions")


# ------------------------------------------------------------------------------ active-row compaction
def active_rows(weights: torch.Tensor, tile: int = 128) -> tuple[torch.Tensor, torch.Tensor, int]:
    """Rows with a non-zero weight, in row order: ``(idx, total, n)`` where ``idx`` (int32) holds the
    active rows followed by zeros up to a whole number of ``tile`` rows, ``total`` is the device
    count and ``n`` the same count on the host (one read back: the shapes that follow depend on
    it).  Stable compaction by block scan (src/causal_trainer/kernels/cut_cross_entropy.py:673-694)."""
    w = weights.reshape(-1).to(torch.float32).contiguous()
    rows = w.numel()
    dev = w.device
    idx = torch.zeros(rows + tile, dtype=torch.int32, device=dev)
    counts = torch.empty(-(-rows // 1024), dtype=torch.int32, device=dev)
    total = torch.empty(1, dtype=torch.int32, device=dev)
    code = _lib.lib().ctb_active_rows(_lib.ptr(w), rows, _lib.ptr(counts), _lib.ptr(idx), _lib.ptr(total),
                                      _lib.stream_ptr())
    _lib.check(code, "ctb_active_rows")
    n = int(total.item())
    padded = -(-n // tile) * tile
    return idx[:padded], total, n


def gather_rows(src: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """``src[idx]`` for a 2-D bf16 matrix with unit inner stride."""
    out = torch.empty((idx.numel(), src.shape[1]), dtype=src.dtype, device=src.device)
    code = _lib.lib().ctb_gather_rows(_lib.ptr(src), _l(src.stride(0)), src.shape[0], _lib.ptr(idx), _lib.ptr(out),
                                      _l(idx.numel()), src.shape[1], _lib.stream_ptr())
    _lib.check(code, "ctb_gather_rows")
    return out


def scatter_rows(src: torch.Tensor, idx: torch.Tensor, total: torch.Tensor, rows: int) -> torch.Tensor:
    """``out[idx[j]] = src[j]`` for the first ``total`` entries of ``idx``; every other row of the
    ``[rows, d]`` result is zero."""
    out = torch.zeros((rows, src.shape[1]), dtype=src.dtype, device=src.device)
    code = _lib.lib().ctb_scatter_rows(_lib.ptr(src), _lib.ptr(idx), _lib.ptr(total), _lib.ptr(out), _l(out.stride(0)),
                                       rows, _l(idx.numel()), src.shape[1], _lib.stream_ptr())
    _lib.check(code, "ctb_scatter_rows")
    return out
