"""Segment-masked flash attention: visibility metadata, the sm_100a kernels and the oracle.

Visibility rule (shared by every backend):

    key j is visible to query i  <=>  seg[j] == seg[i] != 0  and  j <= max(i, attention_end[i])

``seg`` holds canonical run ids (0 = padding) and ``attention_end`` is the optional
inclusive end index that gives MaskGIT image blocks block-local bidirectional attention.
Rows that see no key produce a zero output and zero gradients.

Reference counterparts: ``vanilla_attention`` (src/causal_trainer/modeling/attention.py:100-148),
``efficient_attention`` and its block summaries
(src/causal_trainer/kernels/efficient_attention.py:313-412, 1890-1960).
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from . import lib as _lib

BLOCK = 128


@dataclass
class AttentionMeta:
    """Per-step visibility metadata, built once and reused by every layer."""

    seg: torch.Tensor            # [B,S] int32 canonical segment ids
    lim: torch.Tensor | None     # [B,S] int32 inclusive last visible key (None: plain causal)
    kv_lo: torch.Tensor          # [B,S/128] int32
    kv_hi: torch.Tensor          # [B,S/128] int32
    q_lo: torch.Tensor           # [B,S/128] int32 first query that sees the key block
    q_hi: torch.Tensor           # [B,S/128] int32 one past the last such query
    attention_end: torch.Tensor | None = None  # kept for the oracle backend
    start: torch.Tensor | None = None        # [B,S] int32 first token of the token's run
    end: torch.Tensor | None = None          # [B,S] int32 last token of the token's run
    first_q: torch.Tensor | None = None      # [B,S] int32 first query that sees the token as a key

    @property
    def batch(self) -> int:
        return self.seg.shape[0]

    @property
    def seq(self) -> int:
        return self.seg.shape[1]


def attention_metadata(attention_mask: torch.Tensor, segment_ids: torch.Tensor | None = None,
                       attention_end: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor, AttentionMeta]:
    """Canonical segment ids, restart positions and the block summaries of one micro-batch.

    On a GPU this is one launch of ``ctb_attention_meta`` (``csrc/attention_meta.cu``); elsewhere
    the PyTorch formulation (also the kernel's test oracle).  Returns ``(seg, pos, meta)``.
    """
    if not attention_mask.is_cuda:
        from ..models.decoder import canonicalize_segment_ids, make_position_ids
        seg = canonicalize_segment_ids(attention_mask, segment_ids)
        return seg, make_position_ids(attention_mask, seg, canonical=True), build_attention_meta_reference(seg, attention_end)
    bsz, s = attention_mask.shape
    if s % BLOCK:
        raise ValueError(f"sequence length {s} must be a multiple of {BLOCK}")
    dev = attention_mask.device
    i32 = lambda t: None if t is None else t.to(torch.int32).contiguous()  # noqa: E731
    mask, label, end = i32(attention_mask), i32(segment_ids), i32(attention_end)
    seg = torch.empty((bsz, s), dtype=torch.int32, device=dev)
    pos = torch.empty_like(seg)
    lim = torch.empty_like(seg)
    rows = torch.empty((4, bsz, s), dtype=torch.int32, device=dev)
    s128 = torch.empty((4, bsz, s // BLOCK), dtype=torch.int32, device=dev)
    code = _lib.lib().ctb_attention_meta(_lib.ptr(mask), _lib.ptr(label), _lib.ptr(end), bsz, s, _lib.ptr(seg),
                                         _lib.ptr(pos), _lib.ptr(lim), _lib.ptr(rows), _lib.ptr(s128),
                                         _lib.stream_ptr())
    _lib.check(code, "ctb_attention_meta")
    meta = AttentionMeta(seg, lim if attention_end is not None else None, s128[0], s128[1], s128[2], s128[3],
                         attention_end, rows[0], rows[1], rows[2])
    return seg, pos, meta


def build_attention_meta(segment_ids: torch.Tensor, attention_end: torch.Tensor | None = None) -> AttentionMeta:
    """Block summaries from canonical segment ids (contiguous runs numbered 1.., 0 for padding) and
    MaskGIT ends; ``S`` must be a multiple of 128."""
    if segment_ids.is_cuda:
        return attention_metadata(segment_ids != 0, segment_ids, attention_end)[2]
    return build_attention_meta_reference(segment_ids, attention_end)


def build_attention_meta_reference(segment_ids: torch.Tensor, attention_end: torch.Tensor | None = None) -> AttentionMeta:
    """PyTorch formulation of :func:`build_attention_meta` (CPU path and test oracle)."""
    seg = segment_ids.to(torch.int32).contiguous()
    bsz, s = seg.shape
    if s % BLOCK:
        raise ValueError(f"sequence length {s} must be a multiple of {BLOCK}")
    dev = seg.device
    idx = torch.arange(s, device=dev, dtype=torch.int32).expand(bsz, s)
    valid = seg != 0
    big = torch.iinfo(torch.int32).max
    prev = torch.cat([torch.zeros_like(seg[:, :1]), seg[:, :-1]], dim=1)
    nxt = torch.cat([seg[:, 1:], torch.zeros_like(seg[:, :1])], dim=1)
    starts = valid & (seg != prev)
    ends = valid & (seg != nxt)
    seg_start = torch.cummax(torch.where(starts, idx, torch.zeros_like(idx)), dim=1).values
    rev_end = torch.where(ends, idx, torch.full_like(idx, big)).flip(1)
    seg_end = torch.cummin(rev_end, dim=1).values.flip(1)  # inclusive last index of the run
    if attention_end is None:
        lim = None
        lim_full = idx
    else:
        lim_full = torch.maximum(idx, attention_end.to(torch.int32))
        lim_full = torch.minimum(lim_full, torch.where(valid, seg_end, idx)).contiguous()
        lim = lim_full
    nb = s // BLOCK

    def blk(x):
        return x.reshape(bsz, nb, BLOCK)

    kv_lo = blk(torch.where(valid, seg_start, torch.full_like(idx, big))).amin(-1)
    kv_hi = blk(torch.where(valid, lim_full + 1, torch.zeros_like(idx))).amax(-1)
    kv_lo = torch.where(kv_hi > 0, kv_lo, torch.zeros_like(kv_lo))
    # first query that sees key j: suffix-min over p >= j of min{i : lim[i] == p}
    if attention_end is None:
        first_q = idx
    else:
        m = torch.full((bsz, s), big, device=dev, dtype=torch.int32)
        m = m.scatter_reduce(1, lim_full.long(), torch.where(valid, idx, torch.full_like(idx, big)), "amin")
        first_q = torch.cummin(m.flip(1), dim=1).values.flip(1)
        first_q = torch.minimum(first_q, idx)
    q_lo = blk(torch.where(valid, first_q, torch.full_like(idx, big))).amin(-1)
    q_hi = blk(torch.where(valid, seg_end + 1, torch.zeros_like(idx))).amax(-1)
    q_lo = torch.where(q_hi > 0, q_lo, torch.zeros_like(q_lo))
    i32 = lambda t: t.to(torch.int32).contiguous()  # noqa: E731
    return AttentionMeta(
        seg, lim, i32(kv_lo), i32(kv_hi), i32(q_lo), i32(q_hi), attention_end,
        i32(seg_start), i32(seg_end), i32(first_q),
    )


def visibility_mask(segment_ids: torch.Tensor, attention_end: torch.Tensor | None = None) -> torch.Tensor:
    """Dense [B,S,S] boolean mask of the visibility rule (oracle only)."""
    seg = segment_ids
    s = seg.shape[1]
    idx = torch.arange(s, device=seg.device)
    lim = idx.expand_as(seg) if attention_end is None else torch.maximum(idx.expand_as(seg), attention_end.long())
    same = (seg[:, :, None] == seg[:, None, :]) & (seg[:, :, None] != 0)
    return same & (idx[None, None, :] <= lim[:, :, None])


def vanilla_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, segment_ids: torch.Tensor,
    attention_end: torch.Tensor | None = None, scale: float | None = None,
) -> torch.Tensor:
    """O(S^2) fp32-softmax oracle with GQA.  q [B,S,Hq,D]; k, v [B,S,Hkv,D]."""
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    g = hq // hkv
    qf = q.float().view(b, s, hkv, g, d)
    scores = torch.einsum("bqhgd,bkhd->bhgqk", qf, k.float()) * scale
    mask = visibility_mask(segment_ids, attention_end)[:, None, None]
    scores = scores.masked_fill(~mask, torch.finfo(torch.float32).min)
    probs = torch.softmax(scores, dim=-1)
    probs = torch.where(mask.any(-1, keepdim=True), probs, torch.zeros_like(probs))
    probs = probs * mask
    out = torch.einsum("bhgqk,bkhd->bqhgd", probs, v.float())
    return out.reshape(b, s, hq, d).to(q.dtype)


def _row_stride(t: torch.Tensor) -> int:
    # [B,S,H,D] view: D contiguous, heads D apart, batches S rows apart.
    b, s, h, d = t.shape
    if t.stride(3) != 1 or t.stride(2) != d or (b > 1 and t.stride(0) != t.stride(1) * s):
        raise ValueError("attention operands must be [B,S,H,D] views with contiguous heads")
    return t.stride(1)


def flash_attention_forward(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, meta: AttentionMeta, scale: float | None = None,
    out: torch.Tensor | None = None, spin_budget: int = 0, q_offset: int = 0,
    kv_flags: tuple[torch.Tensor, int, int, int] | None = None,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Runs the tcgen05 forward kernel; returns (O [B,Sq,Hq,D] bf16, LSE [B,Hq,Sq] fp32).

    Under sequence parallelism ``q`` holds only the queries ``[q_offset, q_offset + Sq)`` of every
    row while ``k`` / ``v`` (and ``meta``) cover the whole sequence.  ``kv_flags = (flags, chunk
    elements, elements per gathered row, epoch)`` says that ``k`` / ``v`` are the two halves of a
    buffer an all-gather pull is still filling: the kernel's producer warp acquires the chunk flags
    of every key tile before loading it.
    """
    b, sq, hq, d = q.shape
    s = k.shape[1]
    hkv = k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    if out is None:
        out = torch.empty((b, sq, hq, d), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
    common = (_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(meta.seg), _lib.ptr(meta.lim),
              _lib.ptr(meta.start), _lib.ptr(meta.kv_lo), _lib.ptr(meta.kv_hi),
              b, s, sq, q_offset, hq, hkv, d, ctypes.c_long(_row_stride(q)), ctypes.c_long(_row_stride(k)),
              ctypes.c_long(_row_stride(v)), ctypes.c_long(_row_stride(out)), ctypes.c_float(scale))
    if kv_flags is None:
        code = _lib.lib().ctb_attn_fwd_range(*common, ctypes.c_longlong(spin_budget), _lib.stream_ptr())
        _lib.check(code, "ctb_attn_fwd_range")
    else:
        flags, chunk, row_elems, epoch = kv_flags
        code = _lib.lib().ctb_attn_fwd_gathered(*common, _lib.ptr(flags), ctypes.c_long(chunk), ctypes.c_long(row_elems),
                                                ctypes.c_uint(epoch), ctypes.c_longlong(spin_budget), _lib.stream_ptr())
        _lib.check(code, "ctb_attn_fwd_gathered")
    return out, lse


def flash_attention_backward(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor, dout: torch.Tensor, lse: torch.Tensor,
    meta: AttentionMeta, scale: float | None = None, spin_budget: int = 0,
    dq: torch.Tensor | None = None, dk: torch.Tensor | None = None, dv: torch.Tensor | None = None,
    q_offset: int = 0, stats: tuple[torch.Tensor, torch.Tensor] | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """dQ (query-tile-owned kernel) and dK/dV (key-tile-owned kernel, group reduced in TMEM).

    With a query range (``q_offset``, ``Sq < S``) dK / dV are this rank's partial sums over its
    queries, for all ``S`` keys.
    """
    b, sq, hq, d = q.shape
    s = k.shape[1]
    hkv = k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    from .elementwise import attention_backward_stats

    _row_stride(out), _row_stride(dout)
    # [B,Hq,Sq] fp32; a caller that splits one softmax over several passes hands in the shared ones
    neg_lse2, neg_delta = attention_backward_stats(out, dout, lse) if stats is None else stats
    dq = torch.empty((b, sq, hq, d), dtype=torch.bfloat16, device=q.device) if dq is None else dq
    dk = torch.empty((b, s, hkv, d), dtype=torch.bfloat16, device=q.device) if dk is None else dk
    dv = torch.empty((b, s, hkv, d), dtype=torch.bfloat16, device=q.device) if dv is None else dv
    L = _lib.lib()
    for mode in (0, 1):
        code = L.ctb_attn_bwd_range(
            mode, _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(dout), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
            _lib.ptr(neg_lse2), _lib.ptr(neg_delta), _lib.ptr(meta.seg), _lib.ptr(meta.lim), _lib.ptr(meta.kv_lo),
            _lib.ptr(meta.kv_hi), _lib.ptr(meta.q_lo), _lib.ptr(meta.q_hi), _lib.ptr(meta.start), _lib.ptr(meta.end), _lib.ptr(meta.first_q),
            b, s, sq, q_offset, hq, hkv, d,
            ctypes.c_long(_row_stride(q)), ctypes.c_long(_row_stride(k)), ctypes.c_long(_row_stride(v)),
            ctypes.c_long(_row_stride(dout)), ctypes.c_long(_row_stride(dq)), ctypes.c_long(_row_stride(dk)),
            ctypes.c_long(_row_stride(dv)), ctypes.c_float(scale), ctypes.c_longlong(spin_budget), _lib.stream_ptr(),
        )
        _lib.check(code, "ctb_attn_bwd_range")
    return dq, dk, dv


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta, scale):
        out, lse = flash_attention_forward(q, k, v, meta, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta = meta
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dout = dout if dout.stride(3) == 1 and dout.stride(2) == dout.shape[3] else dout.contiguous()
        dq, dk, dv = flash_attention_backward(q, k, v, out, dout, lse, ctx.meta, ctx.scale)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, meta: AttentionMeta, scale: float | None = None) -> torch.Tensor:
    """Differentiable segment-masked flash attention on the sm_100a kernels."""
    return _FlashAttention.apply(q, k, v, meta, scale)
