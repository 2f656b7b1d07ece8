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

    def _init_sp(self, sp_group, fused: bool) -> None:
        self.sp_group = sp_group
        self.sp_world = dist.get_world_size(sp_group)
        self.sp_rank = dist.get_rank(sp_group)
        self.sp_fused = fused
        self._kv_ctx: dict[tuple[int, int], TpContext] = {}
        if self.options.attention_options is not None and self.options.attention_options.method == "moba":
            raise ValueError("MoBA and sequence parallelism (sp > 1) cannot be combined: shard long rows over tp instead")

    # ------------------------------------------------------------------ token slice
    def _local_seq(self, s: int) -> int:
        return s // self.sp_world

    def select_tokens(self, t: torch.Tensor) -> torch.Tensor:
        s = t.shape[1]
        if s % (self.sp_world * 128):
            raise ValueError(f"sequence length {s} must be a multiple of 128 * sp ({128 * self.sp_world})")
        n = s // self.sp_world
        return t[:, self.sp_rank * n:(self.sp_rank + 1) * n].contiguous()

    def _context(self, batch):
        ctx = super()._context(batch)            # metadata of the whole rows; rotary table of all positions
        s = ctx["seq"]
        n = s // self.sp_world
        lo = self.sp_rank * n
        b = ctx["batch"]
        # the rotary table is [B*S, ...]: keep this rank's positions of every row
        ctx["cos"] = ctx["cos"].view(b, s, -1)[:, lo:lo + n].reshape(b * n, -1).contiguous()
        ctx["sin"] = ctx["sin"].view(b, s, -1)[:, lo:lo + n].reshape(b * n, -1).contiguous()
        ctx.update(seq=n, seq_full=s, q_off=lo)
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
        """Starts the all-gather of row ``b``'s keys and values; returns ``(slot, K [1,S,Hkv,D], V)``."""
        _, n, hkv, d = k.shape
        kvw = hkv * d
        g = kv.next_slot()
        g.mine[:, :kvw].copy_(k[b].reshape(n, kvw))
        g.mine[:, kvw:].copy_(v[b].reshape(n, kvw))
        full = kv.all_gather(g)                                  # [S, 2 kvw]: keys | values of every token
        s = full.shape[0]
        return g, full[:, :kvw].view(1, s, hkv, d), full[:, kvw:].view(1, s, hkv, d)

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
        o = torch.empty((b, n, q.shape[2], d), dtype=torch.bfloat16, device=q.device)
        lse = torch.empty((b, q.shape[2], n), dtype=torch.float32, device=q.device)
        for row in range(b):
            g, k_full, v_full = self._gather_row(kv, k, v, row)
            flags = kv.gathered_flags(g) if self._flags_are_safe(q.shape[2], n, q.device) else None
            if flags is None:
                kv.wait_gathered(g)
            o_row, lse_row = attn_ops.flash_attention_forward(
                q[row:row + 1], k_full, v_full, self._row_meta(ctx["meta"], row), q_offset=ctx["q_off"],
                out=o[row:row + 1], kv_flags=flags)
            lse[row:row + 1].copy_(lse_row)
            self._count(5)
        return o, lse, {"sp": True}

    def _attention_backward(self, q, k, v, o, do, lse, aux, ctx, dq, dk, dv) -> None:
        b, n, hkv, d = k.shape
        s = ctx["seq_full"]
        kvw = hkv * d
        kv = self._gather_ctx(s, 2 * kvw, k.device)
        for row in range(b):
            g, k_full, v_full = self._gather_row(kv, k, v, row)
            kv.wait_gathered(g)                                  # the backward kernels read plain memory
            part = kv.next_slot()                                # this rank's partial dK | dV for all S keys
            dk_full = part.full[:, :kvw].view(1, s, hkv, d)
            dv_full = part.full[:, kvw:].view(1, s, hkv, d)
            attn_ops.flash_attention_backward(
                q[row:row + 1], k_full, v_full, o[row:row + 1], do[row:row + 1], lse[row:row + 1],
                self._row_meta(ctx["meta"], row), dq=dq[row:row + 1], dk=dk_full, dv=dv_full, q_offset=ctx["q_off"])
            mine = kv.reduce_scatter_rows(part)                  # [n, 2 kvw]: the key slice this rank projected
            dk[row].copy_(mine[:, :kvw].view(n, hkv, d))
            dv[row].copy_(mine[:, kvw:].view(n, hkv, d))
            self._count(9)


class SpLayerwiseEngine(SequenceParallelAttention, LayerwiseEngine):
    """Sequence parallelism on the plain layer schedule (every rank holds all heads)."""

    def __init__(self, cfg: ModelConfig, sp_group, provider, options: EngineOptions | None = None, fused: bool = True):
        LayerwiseEngine.__init__(self, cfg, provider, options)
        self._init_sp(sp_group, fused)


def sp_tp_engine(full_cfg: ModelConfig, tp_group, sp_group, provider, options: EngineOptions | None = None,
                 fused: bool = True):
    """Sequence x tensor parallelism: the tensor-parallel schedule on this rank's token slice, its
    attention seeing the whole row through the sp gather."""
    from .tp_engine import TpLayerwiseEngine

    class SpTpLayerwiseEngine(SequenceParallelAttention, TpLayerwiseEngine):
        def __init__(self):
            TpLayerwiseEngine.__init__(self, full_cfg, tp_group, provider, options, fused=fused)
            self._init_sp(sp_group, fused)

    return SpTpLayerwiseEngine()
