"""MoBA block-sparse attention on the sm_100a kernels.

Pipeline of one layer (all on the GPU):

1. ``ctb_moba_pool``   mean key of every complete document-relative block (fp32);
2. ``ctb_moba_route``  per (token, query head): ``q . mean(K_block)`` over the completed blocks
   before the query's own, top-(k-1) with ties to the earlier block, as a selection bit mask;
3. ``ctb_moba_touch`` / ``ctb_moba_lists``  work lists: for every CTA of the flash kernels the key
   tiles (forward), the 64-key blocks (dQ) and the (64-query block, head) pairs (dK/dV) that at
   least one of its rows selected, at a fixed stride with a count per CTA (no host round trip);
4. the tcgen05 flash kernels of ``csrc/attention_fwd.cu`` / ``attention_bwd.cu`` walk those
   lists and test the selection bits per row, so one softmax covers the union of the query's own
   block (causal) and its selected blocks, and unselected key tiles are never loaded.

The routing carries no gradient.  Semantics follow the reference's MoBA graph
(src/causal_trainer/modeling/approximate_attention.py:29-127) whose Pallas path groups queries by
selected block and merges per-rank partial softmaxes
(src/causal_trainer/kernels/grouped_moba.py:25-57,75-164,177-272, moba_current_block.py:34-127);
here the per-row bit mask makes the merge unnecessary.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from . import lib as _lib
from .attention import AttentionMeta, _row_stride
from .elementwise import attention_backward_stats


@dataclass
class WorkList:
    """Per-CTA work list: CSR (``off`` [items+1], ``entries``) or strided (``count`` [items],
    ``entries`` [items, stride])."""

    entries: torch.Tensor
    off: torch.Tensor | None = None
    count: torch.Tensor | None = None
    stride: int = 0

    def lengths(self) -> torch.Tensor:
        return self.count if self.count is not None else (self.off[1:] - self.off[:-1])

    def item(self, i: int) -> list[int]:
        if self.count is not None:
            return self.entries.view(-1, self.stride)[i, :int(self.count[i])].tolist()
        return self.entries[int(self.off[i]):int(self.off[i + 1])].tolist()


@dataclass
class MobaRouting:
    """Selection masks and CTA work lists of one layer."""

    sel: torch.Tensor          # [B,Hq,S,W] int32 bit masks of selected document-relative blocks
    allsel: torch.Tensor       # [B,Hq,S/64,W] int32: AND of sel over each 64-query block (padding counts as all)
    doc_start: torch.Tensor    # [B,S] int32
    block: int
    words: int
    fwd: WorkList
    dq: WorkList
    dkv: WorkList

    @property
    def visited_fraction(self) -> float:
        """Key tiles visited by the forward kernel / tiles a dense causal kernel visits (reads back)."""
        b, hq, s, _ = self.sel.shape
        nqp, nb128 = (s + 255) // 256, s // 128
        dense = sum(min(nb128, 2 * (p + 1)) for p in range(nqp)) * b * hq
        return float(self.fwd.lengths().sum()) / max(1, dense)


def document_starts(seg: torch.Tensor) -> torch.Tensor:
    """First token index of every token's document (canonical run ids; 0 for padding)."""
    b, s = seg.shape
    idx = torch.arange(s, device=seg.device, dtype=torch.int32).expand(b, s)
    prev = torch.cat([torch.zeros_like(seg[:, :1]), seg[:, :-1]], dim=1)
    first = (seg != 0) & (seg != prev)
    return torch.cummax(torch.where(first, idx, torch.zeros_like(idx)), dim=1).values.to(torch.int32)


def route(q: torch.Tensor, k: torch.Tensor, seg: torch.Tensor, doc_start: torch.Tensor, block: int,
          top_k: int, with_pool_start: bool = False):
    """Selection bit masks ``[B,Hq,S,W]`` (int32) from the pooling and routing kernels (and, on
    request, ``pool_start [B,S/128]``: the first token of the complete block that starts in each tile)."""
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    words = max(1, -(-(-(-s // block)) // 32))
    L = _lib.lib()
    pooled = torch.empty((b, s // 128, hkv, d), dtype=torch.float32, device=q.device)
    pool_start = torch.empty((b, s // 128), dtype=torch.int32, device=q.device)
    code = L.ctb_moba_pool(_lib.ptr(k), ctypes.c_long(_row_stride(k)), _lib.ptr(seg), _lib.ptr(doc_start), b, s, hkv,
                           d, block, _lib.ptr(pooled), _lib.ptr(pool_start), _lib.stream_ptr())
    _lib.check(code, "ctb_moba_pool")
    sel = torch.empty((b, hq, s, words), dtype=torch.int32, device=q.device)
    code = L.ctb_moba_route(_lib.ptr(q), ctypes.c_long(_row_stride(q)), _lib.ptr(pooled), _lib.ptr(pool_start),
                            _lib.ptr(seg), _lib.ptr(doc_start), b, s, hq, hkv, d, block, top_k, words, _lib.ptr(sel),
                            _lib.stream_ptr())
    _lib.check(code, "ctb_moba_route")
    return (sel, pool_start) if with_pool_start else sel


def _touched_blocks(sel: torch.Tensor, seg: torch.Tensor, doc_start: torch.Tensor, block: int) -> torch.Tensor:
    """``[B,Hq,S/64,S/64]`` bool: some row of the 64-query block selected keys inside the 64-key block."""
    b, hq, s, words = sel.shape
    nb = s // 64
    dev = sel.device
    idx = torch.arange(s, device=dev, dtype=torch.int64)
    row = ((torch.arange(b, device=dev)[:, None, None] * hq + torch.arange(hq, device=dev)[None, :, None]) * nb
           + (idx // 64)[None, None, :]) * (nb + 1)                                   # [B,Hq,S]
    diff = torch.zeros(b * hq * nb * (nb + 1), dtype=torch.int32, device=dev)
    live = (seg != 0)[:, None, :]
    start = doc_start.to(torch.int64)
    for c in range(min(-(-s // block), 32 * words)):
        bit = ((sel[..., c >> 5] >> (c & 31)) & 1).bool() & live                       # [B,Hq,S]
        lo = start + c * block                                                         # [B,S]
        hi = torch.minimum(lo + block - 1, idx[None, :])
        ok = bit & (lo <= idx[None, :])[:, None, :]
        w = ok.to(torch.int32).reshape(-1)
        diff.scatter_add_(0, (row + (lo // 64).clamp(max=nb)[:, None, :]).reshape(-1), w)
        diff.scatter_add_(0, (row + (hi // 64 + 1).clamp(max=nb)[:, None, :]).reshape(-1), -w)
    return diff.view(b, hq, nb, nb + 1).cumsum(-1)[..., :nb] > 0


def _block_and(sel: torch.Tensor, seg: torch.Tensor) -> torch.Tensor:
    """Bitwise AND of the selection masks over each block of 64 queries (padding rows count as all ones)."""
    b, hq, s, words = sel.shape
    eff = torch.where((seg != 0)[:, None, :, None], sel, torch.full_like(sel, -1)).view(b, hq, s // 64, 64, words)
    n = 64
    while n > 1:                      # log-step reduction: no bitwise-AND reduce in PyTorch
        n //= 2
        eff = eff[:, :, :, :n] & eff[:, :, :, n:2 * n]
    return eff[:, :, :, 0].contiguous()


def _csr(table: torch.Tensor, values: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Offsets and entries of a ``[items, candidates]`` bool table (entry = candidate index or ``values``)."""
    counts = table.sum(-1, dtype=torch.int32)
    off = torch.zeros(table.shape[0] + 1, dtype=torch.int32, device=table.device)
    off[1:] = torch.cumsum(counts, 0)
    hit = torch.nonzero(table)
    entries = hit[:, 1] if values is None else values[hit[:, 1]]
    if entries.numel() == 0:
        entries = torch.zeros(1, dtype=torch.int32, device=table.device)
    return off, entries.to(torch.int32).contiguous()


def build_routing_reference(q: torch.Tensor, k: torch.Tensor, meta: AttentionMeta, block: int, top_k: int,
                            sel: torch.Tensor | None = None) -> MobaRouting:
    """Work lists from PyTorch ops (scatter / cumsum / nonzero); the oracle of :func:`build_routing`."""
    b, s, hq, _ = q.shape
    hkv = k.shape[2]
    g = hq // hkv
    seg = meta.seg
    doc_start = document_starts(seg)
    if sel is None:
        sel = route(q, k, seg, doc_start, block, top_k)
    touch = _touched_blocks(sel, seg, doc_start, block)                                # [B,Hq,nq64,nk64]
    allsel = _block_and(sel, seg)
    nb64, nb128 = s // 64, s // 128
    nqp = (s + 255) // 256
    # forward: (query pair descending, batch, head) x 128-key tiles
    t = touch.view(b, hq, nb64, nb128, 2).any(-1)
    if nb64 % 4:
        t = torch.cat([t, torch.zeros((b, hq, 4 - nb64 % 4, nb128), dtype=torch.bool, device=t.device)], dim=2)
    t = t.view(b, hq, nqp, 4, nb128).any(3)
    fwd_off, fwd_list = _csr(t.permute(2, 0, 1, 3).flip(0).reshape(-1, nb128))
    # dQ: (query tile descending, batch, head) x 64-key blocks
    t = touch.view(b, hq, nb128, 2, nb64).any(3)
    dq_off, dq_list = _csr(t.permute(2, 0, 1, 3).flip(0).reshape(-1, nb64))
    # dK/dV: (key tile ascending, batch, kv head) x (head in group, 64-query block)
    t = touch.view(b, hkv, g, nb64, nb128, 2).any(-1).permute(4, 0, 1, 2, 3).reshape(-1, g * nb64)
    packed = (torch.arange(g, device=t.device)[:, None] * (1 << 24) + torch.arange(nb64, device=t.device)[None, :])
    dkv_off, dkv_list = _csr(t, packed.reshape(-1))
    return MobaRouting(sel, allsel, doc_start, block, sel.shape[-1], WorkList(fwd_list, off=fwd_off),
                       WorkList(dq_list, off=dq_off), WorkList(dkv_list, off=dkv_off))


def build_routing(q: torch.Tensor, k: torch.Tensor, meta: AttentionMeta, block: int, top_k: int) -> MobaRouting:
    """Routing and work lists entirely on the GPU, no host round trip: pool, route, a touch bitmap per
    64-query block, then one warp per flash-kernel CTA compacts its candidates (``csrc/moba.cu``)."""
    b, s, hq, _ = q.shape
    hkv = k.shape[2]
    g = hq // hkv
    seg = meta.seg
    dev = q.device
    # the run start of every token is part of the step's attention metadata (one launch per micro-batch)
    doc_start = meta.start.contiguous() if meta.start is not None else document_starts(seg)
    sel = route(q, k, seg, doc_start, block, top_k)
    words = sel.shape[-1]
    nb64, nb128, nqp = s // 64, s // 128, (s + 255) // 256
    tw = -(-nb64 // 32)
    L = _lib.lib()
    touch = torch.empty((b, hq, nb64, tw), dtype=torch.int32, device=dev)
    allsel = torch.empty((b, hq, nb64, words), dtype=torch.int32, device=dev)
    code = L.ctb_moba_touch(_lib.ptr(sel), _lib.ptr(seg), _lib.ptr(doc_start), b, s, hq, block, words, tw,
                            _lib.ptr(touch), _lib.ptr(allsel), _lib.stream_ptr())
    _lib.check(code, "ctb_moba_touch")
    lists = []
    for mode, items, stride in ((0, b * hq * nqp, nb128), (1, b * hq * nb128, nb64), (2, b * hkv * nb128, g * nb64)):
        entries = torch.empty((items, stride), dtype=torch.int32, device=dev)
        count = torch.empty(items, dtype=torch.int32, device=dev)
        code = L.ctb_moba_lists(mode, _lib.ptr(touch), b, s, hq, hkv, tw, items, stride, _lib.ptr(entries),
                                _lib.ptr(count), _lib.stream_ptr())
        _lib.check(code, "ctb_moba_lists")
        lists.append(WorkList(entries, count=count, stride=stride))
    return MobaRouting(sel, allsel, doc_start, block, words, *lists)


def moba_forward(q, k, v, meta: AttentionMeta, routing: MobaRouting, scale: float | None = None,
                 spin_budget: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """Block-sparse forward; returns (O [B,S,Hq,D] bf16, LSE [B,Hq,S] fp32)."""
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out = torch.empty((b, s, hq, d), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((b, hq, s), dtype=torch.float32, device=q.device)
    r = routing
    code = _lib.lib().ctb_attn_fwd_sparse(
        _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(out), _lib.ptr(lse), _lib.ptr(meta.seg), _lib.ptr(meta.lim),
        _lib.ptr(meta.start), _lib.ptr(meta.kv_lo), _lib.ptr(meta.kv_hi),
        _lib.ptr(r.fwd.off), _lib.ptr(r.fwd.count), r.fwd.stride, _lib.ptr(r.fwd.entries), _lib.ptr(r.sel),
        _lib.ptr(r.doc_start), r.block, r.words,
        b, s, hq, hkv, d, ctypes.c_long(_row_stride(q)), ctypes.c_long(_row_stride(k)), ctypes.c_long(_row_stride(v)),
        ctypes.c_long(_row_stride(out)), ctypes.c_float(scale), ctypes.c_longlong(spin_budget), _lib.stream_ptr())
    _lib.check(code, "ctb_attn_fwd_sparse")
    return out, lse


def moba_backward(q, k, v, out, dout, lse, meta: AttentionMeta, routing: MobaRouting, scale: float | None = None,
                  spin_budget: int = 0, dq=None, dk=None, dv=None):
    """dQ and dK/dV of the block-sparse attention (same kernels as the dense backward, list-driven)."""
    b, s, hq, d = q.shape
    hkv = k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    neg_lse2, neg_delta = attention_backward_stats(out, dout, lse)
    dq = torch.empty((b, s, hq, d), dtype=torch.bfloat16, device=q.device) if dq is None else dq
    dk = torch.empty((b, s, hkv, d), dtype=torch.bfloat16, device=q.device) if dk is None else dk
    dv = torch.empty((b, s, hkv, d), dtype=torch.bfloat16, device=q.device) if dv is None else dv
    r = routing
    L = _lib.lib()
    for mode, wl in ((0, r.dkv), (1, r.dq)):
        code = L.ctb_attn_bwd_sparse(
            mode, _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(dout), _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv),
            _lib.ptr(neg_lse2), _lib.ptr(neg_delta), _lib.ptr(meta.seg), _lib.ptr(meta.lim), _lib.ptr(meta.kv_lo),
            _lib.ptr(meta.kv_hi), _lib.ptr(meta.q_lo), _lib.ptr(meta.q_hi), _lib.ptr(meta.start), _lib.ptr(meta.end), _lib.ptr(meta.first_q),
            _lib.ptr(wl.off), _lib.ptr(wl.count), wl.stride, _lib.ptr(wl.entries), _lib.ptr(r.sel), _lib.ptr(r.allsel),
            _lib.ptr(r.doc_start), r.block, r.words,
            b, s, hq, hkv, d,
            ctypes.c_long(_row_stride(q)), ctypes.c_long(_row_stride(k)), ctypes.c_long(_row_stride(v)),
            ctypes.c_long(_row_stride(dout)), ctypes.c_long(_row_stride(dq)), ctypes.c_long(_row_stride(dk)),
            ctypes.c_long(_row_stride(dv)), ctypes.c_float(scale), ctypes.c_longlong(spin_budget), _lib.stream_ptr())
        _lib.check(code, "ctb_attn_bwd_sparse")
    return dq, dk, dv


# ----------------------------------------------------------------------------------------- query grouping
@dataclass
class MobaGroups:
    """Routing of one layer in grouped form: the (token, head) rows that selected a key block sit
    next to each other in a gathered row space (``csrc/moba.cu``), so the history part of MoBA is
    dense attention per group and its cost follows ``top_k * block``, whatever the routing."""

    sel: torch.Tensor          # [B,Hq,S,W] selection bit masks
    block: int
    picks: int                 # top_k - 1
    rows_cap: int              # capacity of the gathered row space (multiple of 256)
    slot_cap: int              # most non-empty groups there can be
    fwd_desc: torch.Tensor     # [rows_cap/256, 4] int32
    dq_desc: torch.Tensor      # [rows_cap/128, 4]
    dkv_desc: torch.Tensor     # [slot_cap * block/128, 4]
    row_of: torch.Tensor       # [rows_cap] (token * Hq + head), -1 = padding
    pos_of: torch.Tensor       # [B,Hq,S,picks] gathered position of each pick, -1 = none
    totals: torch.Tensor       # [2] rows in use, non-empty groups
    own_meta: AttentionMeta    # visibility of the own-block pass: every (document, block) is a run

    def work_summary(self) -> dict:
        """Reads back how much attention work the grouped pass does (tests, profiles)."""
        rows, slots = (int(x) for x in self.totals.tolist())
        real = int((self.row_of[:rows] >= 0).sum()) if rows else 0
        return {"gathered_rows": rows, "real_rows": real, "groups": slots,
                "history_tiles": rows // 128 * (self.block // 128)}


def own_block_meta(meta: AttentionMeta, block: int) -> AttentionMeta:
    """Metadata under which the dense kernels compute exactly the own-block part of MoBA: causal
    attention inside each (document, block) run.  Cached on ``meta`` (one launch per micro-batch)."""
    cache = meta.__dict__.setdefault("_own_block_meta", {})
    if block not in cache:
        seg = meta.seg
        s = seg.shape[1]
        idx = torch.arange(s, device=seg.device, dtype=torch.int32)[None, :]
        nblk = -(-s // block)
        runs = torch.where(seg != 0, seg * (nblk + 1) + (idx - meta.start) // block + 1, torch.zeros_like(seg))
        from .attention import attention_metadata

        cache[block] = attention_metadata((seg != 0).to(torch.int32), runs)[2]
    return cache[block]


def build_groups(q: torch.Tensor, k: torch.Tensor, meta: AttentionMeta, block: int, top_k: int) -> MobaGroups:
    """Pool, route, then a stable counting sort of the routed rows by selected block (no host round
    trip: capacities depend on shapes only, the kernels skip what is not in use)."""
    b, s, hq, _ = q.shape
    hkv = k.shape[2]
    if block % 128:
        raise ValueError("grouped MoBA needs moba_block_size to be a multiple of 128")
    picks = top_k - 1
    if picks < 1:
        raise ValueError("grouped MoBA needs top_k >= 2 (top_k = 1 is the own block alone)")
    dev = q.device
    seg, doc_start = meta.seg, meta.start.contiguous()
    sel, pool_start = route(q, k, seg, doc_start, block, top_k, with_pool_start=True)
    words = sel.shape[-1]
    gsize, nt128 = hq // hkv, s // 128
    groups = b * hkv * nt128
    slot_cap = b * hkv * (-(-s // block))
    rows_cap = -(-(b * hq * s * picks) // 256) * 256 + 256 * slot_cap
    i32 = lambda *shape: torch.empty(shape, dtype=torch.int32, device=dev)  # noqa: E731
    rank, cnt, row0, hoff = i32(b, hq, s, picks), i32(groups, gsize), i32(groups), i32(groups, gsize)
    ginfo, greal, totals = i32(slot_cap, 4), i32(slot_cap), i32(2)
    fwd_desc, dq_desc, dkv_desc = i32(rows_cap // 256, 4), i32(rows_cap // 128, 4), i32(slot_cap * (block // 128), 4)
    row_of, pos_of = i32(rows_cap), i32(b, hq, s, picks)
    code = _lib.lib().ctb_moba_group(
        _lib.ptr(sel), _lib.ptr(seg), _lib.ptr(doc_start), _lib.ptr(pool_start), b, s, hq, hkv, block, words, picks,
        rows_cap, slot_cap, _lib.ptr(rank), _lib.ptr(cnt), _lib.ptr(row0), _lib.ptr(hoff), _lib.ptr(ginfo),
        _lib.ptr(greal), _lib.ptr(totals), _lib.ptr(fwd_desc), _lib.ptr(dq_desc), _lib.ptr(dkv_desc), _lib.ptr(row_of),
        _lib.ptr(pos_of), _lib.stream_ptr())
    _lib.check(code, "ctb_moba_group")
    return MobaGroups(sel, block, picks, rows_cap, slot_cap, fwd_desc, dq_desc, dkv_desc, row_of, pos_of, totals,
                      own_block_meta(meta, block))


def _gather(groups: MobaGroups, src: torch.Tensor | None, stats: tuple[torch.Tensor, torch.Tensor] | None, s: int,
            hq: int, d: int):
    dev = groups.row_of.device
    dst = torch.empty((groups.rows_cap, d), dtype=torch.bfloat16, device=dev) if src is not None else None
    out_a = out_b = None
    if stats is not None:
        out_a = torch.empty(groups.rows_cap, dtype=torch.float32, device=dev)
        out_b = torch.empty(groups.rows_cap, dtype=torch.float32, device=dev)
    code = _lib.lib().ctb_moba_gather(
        _lib.ptr(groups.row_of), _lib.ptr(groups.totals), _lib.ptr(src),
        ctypes.c_long(_row_stride(src) if src is not None else 0), s, hq, d, _lib.ptr(dst),
        _lib.ptr(stats[0] if stats else None), _lib.ptr(stats[1] if stats else None), _lib.ptr(out_a), _lib.ptr(out_b),
        groups.rows_cap, _lib.stream_ptr())
    _lib.check(code, "ctb_moba_gather")
    return dst, out_a, out_b


def moba_grouped_forward(q, k, v, meta: AttentionMeta, groups: MobaGroups, scale: float | None = None,
                         spin_budget: int = 0) -> tuple[torch.Tensor, torch.Tensor]:
    """MoBA forward as own-block causal pass + dense history pass per group + log-sum-exp merge
    (src/causal_trainer/kernels/grouped_moba.py:75-164, 418-423; moba_current_block.py:34-127).
    Returns (O [B,S,Hq,D] bf16, LSE [B,Hq,S] fp32) of the single softmax over the union."""
    from .attention import flash_attention_forward

    b, s, hq, d = q.shape
    hkv = k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    out, lse = flash_attention_forward(q, k, v, groups.own_meta, scale, spin_budget=spin_budget)
    qg, _, _ = _gather(groups, q, None, s, hq, d)
    og = torch.empty_like(qg)
    lse_g = torch.empty(groups.rows_cap, dtype=torch.float32, device=q.device)
    L = _lib.lib()
    code = L.ctb_attn_fwd_grouped(_lib.ptr(qg), _lib.ptr(k), _lib.ptr(v), _lib.ptr(og), _lib.ptr(lse_g),
                                  _lib.ptr(groups.fwd_desc), groups.rows_cap, groups.block, b, s, hkv, d,
                                  ctypes.c_long(_row_stride(k)), ctypes.c_long(_row_stride(v)), ctypes.c_float(scale),
                                  ctypes.c_longlong(spin_budget), _lib.stream_ptr())
    _lib.check(code, "ctb_attn_fwd_grouped")
    code = L.ctb_moba_merge_fwd(_lib.ptr(out), ctypes.c_long(_row_stride(out)), _lib.ptr(lse), _lib.ptr(og),
                                _lib.ptr(lse_g), _lib.ptr(groups.pos_of), b, s, hq, d, groups.picks, _lib.stream_ptr())
    _lib.check(code, "ctb_moba_merge_fwd")
    return out, lse


def moba_grouped_backward(q, k, v, out, dout, lse, meta: AttentionMeta, groups: MobaGroups, scale: float | None = None,
                          spin_budget: int = 0, dq=None, dk=None, dv=None):
    """Backward of :func:`moba_grouped_forward`.  Every pass uses the statistics of the merged
    softmax (total LSE, ``delta = sum O dO``), so the partial gradients simply add: own-block dQ / dK
    / dV from the dense kernels, history dQ per gathered row (scattered back and added), history
    dK / dV per key block over its group's rows (grouped_moba.py:177-272)."""
    from .attention import flash_attention_backward

    b, s, hq, d = q.shape
    hkv = k.shape[2]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    stats = attention_backward_stats(out, dout, lse)
    dq, dk, dv = flash_attention_backward(q, k, v, out, dout, lse, groups.own_meta, scale, spin_budget=spin_budget,
                                          dq=dq, dk=dk, dv=dv, stats=stats)
    qg, _, _ = _gather(groups, q, None, s, hq, d)
    dog, lse_g, delta_g = _gather(groups, dout, stats, s, hq, d)
    dqg = torch.empty_like(qg)
    dkh = torch.zeros((b, s, hkv, d), dtype=torch.bfloat16, device=q.device)
    dvh = torch.zeros_like(dkh)
    L = _lib.lib()
    for mode, desc in ((0, groups.dkv_desc), (1, groups.dq_desc)):
        code = L.ctb_attn_bwd_grouped(
            mode, _lib.ptr(qg), _lib.ptr(k), _lib.ptr(v), _lib.ptr(dog), _lib.ptr(dqg), _lib.ptr(dkh), _lib.ptr(dvh),
            _lib.ptr(lse_g), _lib.ptr(delta_g), _lib.ptr(desc), desc.shape[0], groups.rows_cap, groups.block, b, s, hkv,
            d, ctypes.c_long(_row_stride(k)), ctypes.c_long(_row_stride(v)), ctypes.c_long(_row_stride(dkh)),
            ctypes.c_long(_row_stride(dvh)), ctypes.c_float(scale), ctypes.c_longlong(spin_budget), _lib.stream_ptr())
        _lib.check(code, "ctb_attn_bwd_grouped")
    code = L.ctb_moba_merge_dq(_lib.ptr(dq), ctypes.c_long(_row_stride(dq)), _lib.ptr(dqg), _lib.ptr(groups.pos_of), b, s,
                               hq, d, groups.picks, _lib.stream_ptr())
    _lib.check(code, "ctb_moba_merge_dq")
    dk.add_(dkh)
    dv.add_(dvh)
    return dq, dk, dv


class _MobaFlash(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, meta, block, top_k, scale):
        routing = build_routing(q, k, meta, block, top_k)
        out, lse = moba_forward(q, k, v, meta, routing, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.meta, ctx.routing, ctx.scale = meta, routing, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = moba_backward(q, k, v, out, dout.contiguous(), lse, ctx.meta, ctx.routing, ctx.scale)
        return dq, dk, dv, None, None, None, None


def moba_flash_attention(q, k, v, segments, block: int, top_k: int, scale: float, meta: AttentionMeta | None = None):
    """Differentiable MoBA attention for ``[B,S,H,D]`` bf16 CUDA tensors (``S`` a multiple of 128)."""
    if block < 128:
        raise ValueError("the sm_100a MoBA kernels need moba_block_size >= 128")
    if meta is None:
        from .attention import build_attention_meta

        meta = build_attention_meta(segments.to(torch.int32), None)
    return _MobaFlash.apply(q, k, v, meta, block, top_k, scale)
