"""Sequence-parallel engine: every rank of the ``sp`` group computes a contiguous slice of the
tokens of each row; attention sees the whole row through all-gathered keys and values.

This is the reference's sequence (context) parallelism: Q, O and the log-sum-exp are sharded over
``sp`` while K / V are replicated over it, and the partial dK / dV of the ranks are summed
(src/causal_trainer/kernels/efficient_attention.py:296-310, 1713-1774; src/causal_trainer/
modeling/attention.py:182-198).  Everything that is per token -- embedding, norms, projections,
MLP, the loss -- runs on the local slice unchanged; only attention communicates:

* forward: the layer's K / V slices are all-gathered over ``sp`` by a pull kernel over NVLink peer
  memory that publishes one flag per chunk (``parallel.tp.TpContext``, the same machinery as the
  tensor-parallel activation gather); the flash kernel runs the local query range against all keys
  and its producer warp acquires the flags of each key tile before loading it, so the transfer
  overlaps the attention over the keys that are already there (all-gather -> attention).  That
  in-kernel wait is used when the forward grid leaves SMs free for the pull kernel's CTAs; larger
  grids wait for the gather on the stream instead (``_flags_are_safe``);
* backward: K / V are gathered again (nothing of size ``S`` is kept between the passes), the dQ
  kernel runs on the local queries and the dK/dV kernel on all keys, writing this rank's partial
  sums into a symmetric buffer; every rank then sums its own key slice from all peers' partials with
  peer loads, in rank order, in fp32 (attention -> reduce-scatter).
* ``fused=False`` is the NCCL variant of the same schedule (all-gather, reduce-scatter calls).

Which tokens a rank computes is a layout choice (``token_ranges``): a contiguous slice per rank, as
in the reference, or zig-zag chunks (``r`` and ``2 sp - 1 - r`` of ``2 sp``) that give every rank
the same causal work; the per-token code never looks at token positions other than through the
rotary table, so only the attention below and the order of the gathered K / V slabs know about it.

Rows of a micro-batch are processed one at a time through the gather (a gathered buffer is one
``[S, 2 * kv_width]`` row), so the buffers do not grow with the batch.

Parameters are not replicated over ``sp``: the sp ranks are further FSDP ranks (each sees
different tokens), so gradients are reduced and optimizer state is sharded over them as well.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..ops import attention as attn_ops
from ..parallel.tp import PULL_CTAS, TpContext
from .engine import EngineOptions, LayerwiseEngine


class SequenceParallelAttention:
    """Mixin: the token slice, its rotary positions and the attention of a rank of an ``sp`` group.
    Combined with :class:`LayerwiseEngine` it is sequence parallelism alone, with
    ``TpLayerwiseEngine`` sequence x tensor parallelism (heads over tp, tokens over sp; dK / dV
    summed over sp here and, for shared key/value heads, over tp by that engine -- the reference's
    ``psum`` over ``("tp", "sp")``, src/causal_trainer/kernels/efficient_attention.py:296-310)."""

    def _init_sp(self, sp_group, fused: bool, layout: str = "contiguous") -> None:
        if layout not in ("contiguous", "zigzag"):
            raise ValueError(f"sp layout must be 'contiguous' or 'zigzag', got {layout!r}")
        self.sp_group = sp_group
        self.sp_world = dist.get_world_size(sp_group)
        self.sp_rank = dist.get_rank(sp_group)
        self.sp_fused = fused
        self.sp_layout = layout
        self._kv_ctx: dict[tuple[int, int], TpContext] = {}
        if self.options.attention_options is not None and self.options.attention_options.method == "moba":
            raise ValueError("MoBA and sequence parallelism (sp > 1) cannot be combined: shard long rows over tp instead")

    # ------------------------------------------------------------------ token slice
    def _local_seq(self, s: int) -> int:
        return s // self.sp_world

    def token_ranges(self, s: int) -> list[tuple[int, int]]:
        """``(first token, count)`` of the pieces of a row this rank computes, in local order.

        ``contiguous``: one slice per rank.  ``zigzag``: the row is cut into ``2 * sp`` chunks and
        rank ``r`` takes chunks ``r`` and ``2 * sp - 1 - r``; under a causal mask every rank then
        has the same number of visible (query, key) pairs, where contiguous slices give the last
        rank ``(2 sp - 1) / sp`` times the mean.  Needs chunks of whole 128-row query tiles; rows
        that do not divide fall back to contiguous slices."""
        w, r = self.sp_world, self.sp_rank
        if s % (w * 128):
            raise ValueError(f"sequence length {s} must be a multiple of 128 * sp ({128 * w})")
        if self._zigzag(s):
            c = s // (2 * w)
            return [(r * c, c), ((2 * w - 1 - r) * c, c)]
        n = s // w
        return [(r * n, n)]

    def _zigzag(self, s: int) -> bool:
        return self.sp_layout == "zigzag" and self.sp_world > 1 and s % (256 * self.sp_world) == 0

    def select_tokens(self, t: torch.Tensor) -> torch.Tensor:
        parts = [t[:, lo:lo + n] for lo, n in self.token_ranges(t.shape[1])]
        return (parts[0] if len(parts) == 1 else torch.cat(parts, dim=1)).contiguous()

    def _to_sequence_order(self, slabs: torch.Tensor, s: int) -> torch.Tensor:
        """``[S, width]`` rows as the gather leaves them (one slab per rank, each in that rank's
        local order) -> rows in sequence order."""
        if not self._zigzag(s):
            return slabs
        w = self.sp_world
        f = slabs.view(w, 2, s // (2 * w), -1)
        return torch.cat([f[:, 0], f[:, 1].flip(0)], dim=0).reshape(s, -1)

    def _to_slab_order(self, rows: torch.Tensor, out: torch.Tensor, s: int) -> None:
        """Inverse of :meth:`_to_sequence_order`, written into ``out`` (a ring slot)."""
        w = self.sp_world
        c = s // (2 * w)
        q, o = rows.view(2 * w, c, -1), out.view(w, 2, c, -1)
        o[:, 0].copy_(q[:w])
        o[:, 1].copy_(q[w:].flip(0))

    def _context(self, batch):
        ctx = super()._context(batch)            # metadata of the whole rows; rotary table of all positions
        s = ctx["seq"]
        n = s // self.sp_world
        b = ctx["batch"]
        # the rotary table is [B*S, ...]: keep this rank's positions of every row
        ctx["cos"] = self.select_tokens(ctx["cos"].view(b, s, -1)).reshape(b * n, -1)
        ctx["sin"] = self.select_tokens(ctx["sin"].view(b, s, -1)).reshape(b * n, -1)
        ctx.update(seq=n, seq_full=s, q_ranges=self.token_ranges(s))
        return ctx

    def _uses_moba(self, li: int, seq: int, longest: int | None = None) -> bool:
        return False

    # ------------------------------------------------------------------ K / V of one row over sp
    def _gather_ctx(self, s: int, width: int, device) -> TpContext:
        """Symmetric ring buffers and flags for ``[S, width]`` rows sharded over the sp group."""
        key = (s, width)
        if key not in self._kv_ctx:
            self._kv_ctx[key] = TpContext(self.sp_group, device, s, width, fused=self.sp_fused)
        return self._kv_ctx[key]

    @staticmethod
    def _row_meta(meta: attn_ops.AttentionMeta, b: int) -> attn_ops.AttentionMeta:
        """The metadata of batch row ``b`` alone (every field is ``[B, ...]``)."""
        pick = lambda t: None if t is None else t[b:b + 1]     # noqa: E731
        return attn_ops.AttentionMeta(pick(meta.seg), pick(meta.lim), pick(meta.kv_lo), pick(meta.kv_hi), pick(meta.q_lo),
                                      pick(meta.q_hi), pick(meta.attention_end), pick(meta.start), pick(meta.end),
                                      pick(meta.first_q))

    def _gather_row(self, kv: TpContext, k: torch.Tensor, v: torch.Tensor, b: int):
        """Starts the all-gather of row ``b``'s keys and values; returns the slot (``slot.full`` is
        ``[S, 2 kvw]``: keys | values, one slab of local rows per rank)."""
        _, n, hkv, d = k.shape
        kvw = hkv * d
        g = kv.next_slot()
        g.mine[:, :kvw].copy_(k[b].reshape(n, kvw))
        g.mine[:, kvw:].copy_(v[b].reshape(n, kvw))
        kv.all_gather(g)
        return g

    @staticmethod
    def _keys_values(rows: torch.Tensor, hkv: int, d: int):
        s, kvw = rows.shape[0], hkv * d
        return rows[:, :kvw].view(1, s, hkv, d), rows[:, kvw:].view(1, s, hkv, d)

    # ------------------------------------------------------------------ attention
    def _flags_are_safe(self, heads: int, queries: int, device) -> bool:
        """Whether the forward kernel may wait for the gather's chunk flags itself.

        A kernel that waits for another launch on the same GPU is only safe when both are certain to
        be resident together.  A forward CTA takes a whole SM (its registers), so that holds when
        the grid leaves enough SMs free for every pull CTA (four fit on one SM); a larger grid could
        fill the GPU with waiting CTAs before the pull kernel is scheduled, and the bounded waits
        would then expire.  Large grids therefore take the stream-level dependency: their attention
        runs for many times the half millisecond the gather takes, so little overlap is lost."""
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        ctas = heads * ((queries + 255) // 256)                  # the forward grid of one row
        return ctas <= sms - (PULL_CTAS + 3) // 4

    def _attention_forward(self, q, k, v, ctx, li):
        b, n, hkv, d = k.shape
        s = ctx["seq_full"]
        kv = self._gather_ctx(s, 2 * hkv * d, k.device)
        zig = self._zigzag(s)
        o = torch.empty((b, n, q.shape[2], d), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((b, q.shape[2], n), dtype=torch.float32, device=q.device)
        for row in range(b):
            g = self._gather_row(kv, k, v, row)
            # the kernel can follow the gather's flags only over a buffer that is in sequence order
            flags = kv.gathered_flags(g) if not zig and self._flags_are_safe(q.shape[2], n, q.device) else None
            if flags is None:
                kv.wait_gathered(g)
            k_full, v_full = self._keys_values(self._to_sequence_order(g.full, s), hkv, d)
            meta = self._row_meta(ctx["meta"], row)
            at = 0
            for lo, cnt in ctx["q_ranges"]:
                _, lse_part = attn_ops.flash_attention_forward(
                    q[row:row + 1, at:at + cnt], k_full, v_full, meta, q_offset=lo, out=o[row:row + 1, at:at + cnt],
                    kv_flags=flags)
                lse[row:row + 1, :, at:at + cnt].copy_(lse_part)
                at += cnt
                self._count(2)
            self._count(3)
        return o, lse, {"sp": True}

    def _attention_backward(self, q, k, v, o, do, lse, aux, ctx, dq, dk, dv) -> None:
        b, n, hkv, d = k.shape
        s = ctx["seq_full"]
        kvw = hkv * d
        kv = self._gather_ctx(s, 2 * kvw, k.device)
        zig = self._zigzag(s)
        ranges = ctx["q_ranges"]
        for row in range(b):
            g = self._gather_row(kv, k, v, row)
            kv.wait_gathered(g)                                  # the backward kernels read plain memory
            k_full, v_full = self._keys_values(self._to_sequence_order(g.full, s), hkv, d)
            part = kv.next_slot()                                # this rank's partial dK | dV for all S keys
            # partial sums in sequence order: the slot itself when that is also its slab order
            total = torch.empty_like(part.full) if zig else part.full
            extra = torch.empty_like(part.full) if len(ranges) > 1 else None
            meta = self._row_meta(ctx["meta"], row)
            at = 0
            for i, (lo, cnt) in enumerate(ranges):
                into = total if i == 0 else extra
                dk_full, dv_full = self._keys_values(into, hkv, d)
                attn_ops.flash_attention_backward(
                    q[row:row + 1, at:at + cnt], k_full, v_full, o[row:row + 1, at:at + cnt], do[row:row + 1, at:at + cnt],
                    lse[row:row + 1, :, at:at + cnt].contiguous(), meta, dq=dq[row:row + 1, at:at + cnt], dk=dk_full,
                    dv=dv_full, q_offset=lo)
                if i:
                    total.add_(extra)
                at += cnt
                self._count(4)
            if zig:
                self._to_slab_order(total, part.full, s)
            mine = kv.reduce_scatter_rows(part)                  # [n, 2 kvw]: the key rows this rank projected
            dk[row].copy_(mine[:, :kvw].view(n, hkv, d))
            dv[row].copy_(mine[:, kvw:].view(n, hkv, d))
            self._count(5)


class SpLayerwiseEngine(SequenceParallelAttention, LayerwiseEngine):
    """Sequence parallelism on the plain layer schedule (every rank holds all heads)."""

    def __init__(self, cfg: ModelConfig, sp_group, provider, options: EngineOptions | None = None, fused: bool = True,
                 layout: str = "contiguous"):
        LayerwiseEngine.__init__(self, cfg, provider, options)
        self._init_sp(sp_group, fused, layout)


def sp_tp_engine(full_cfg: ModelConfig, tp_group, sp_group, provider, options: EngineOptions | None = None,
                 fused: bool = True, layout: str = "contiguous"):
    """Sequence x tensor parallelism: the tensor-parallel schedule on this rank's token slice, its
    attention seeing the whole row through the sp gather."""
    from .tp_engine import TpLayerwiseEngine

    class SpTpLayerwiseEngine(SequenceParallelAttention, TpLayerwiseEngine):
        def __init__(self):
            TpLayerwiseEngine.__init__(self, full_cfg, tp_group, provider, options, fused=fused)
            self._init_sp(sp_group, fused, layout)

    return SpTpLayerwiseEngine()
