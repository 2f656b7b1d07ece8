"""Sequence-parallel engine: every rank of the ``sp`` group computes a contiguous slice of the
tokens of each row; attention sees the whole row through all-gathered keys and values.

This is the reference's sequence (context) parallelism: Q, O and the log-sum-exp are sharded over
``sp`` while K / V are replicated over it, and the partial dK / dV of the ranks are summed
(src/causal_trainer/kernels/efficient_attention.py:296-310, 1713-1774; src/causal_trainer/
modeling/attention.py:182-198).  Everything that is per token -- embedding, norms, projections,
MLP, the loss -- runs on the local slice unchanged; only attention communicates:

* forward: all-gather of the layer's K / V slices over ``sp`` (NCCL), then the flash kernel over
  the local query range against all keys (``ops.attention.flash_attention_forward(q_offset=...)``);
* backward: the dQ kernel on the local queries, the dK/dV kernel on all keys (partial sums over
  the local queries), then a reduce-scatter of dK / dV back to the owners of the key slices.

Parameters are not replicated over ``sp``: the sp ranks are further FSDP ranks (each sees
different tokens), so gradients are reduced and optimizer state is sharded over them as well.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..ops import attention as attn_ops
from .engine import EngineOptions, LayerwiseEngine


class SpLayerwiseEngine(LayerwiseEngine):
    def __init__(self, cfg: ModelConfig, sp_group, provider, options: EngineOptions | None = None):
        super().__init__(cfg, provider, options)
        self.sp_group = sp_group
        self.sp_world = dist.get_world_size(sp_group)
        self.sp_rank = dist.get_rank(sp_group)
        self._slice = slice(None)
        if self.options.attention_options is not None and self.options.attention_options.method == "moba":
            raise ValueError("MoBA and sequence parallelism (sp > 1) cannot be combined: shard long rows over tp instead")

    # ------------------------------------------------------------------ token slice
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

    def _uses_moba(self, li: int, seq: int) -> bool:
        return False

    # ------------------------------------------------------------------ attention
    def _attention_forward(self, q, k, v, ctx, li):
        b, n, hkv, d = k.shape
        p, s = self.sp_world, ctx["seq_full"]
        kvw = hkv * d
        local = torch.cat([k.reshape(b, n, kvw), v.reshape(b, n, kvw)], dim=-1)          # [B, n, 2 kvw]
        gathered = torch.empty((p, b, n, 2 * kvw), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(gathered, local, group=self.sp_group)
        full = gathered.permute(1, 0, 2, 3).reshape(b, s, 2 * kvw)                     # rows back in order
        k_full = full[..., :kvw].view(b, s, hkv, d)
        v_full = full[..., kvw:].view(b, s, hkv, d)
        o, lse = attn_ops.flash_attention_forward(q, k_full, v_full, ctx["meta"], q_offset=ctx["q_off"])
        self._count(4)
        return o, lse, {"kv": full}

    def _attention_backward(self, q, k, v, o, do, lse, aux, ctx, dq, dk, dv) -> None:
        b, n, hkv, d = k.shape
        p, s = self.sp_world, ctx["seq_full"]
        kvw = hkv * d
        full = aux["kv"]
        k_full = full[..., :kvw].view(b, s, hkv, d)
        v_full = full[..., kvw:].view(b, s, hkv, d)
        dfull = torch.empty_like(full)
        dk_full = dfull[..., :kvw].view(b, s, hkv, d)
        dv_full = dfull[..., kvw:].view(b, s, hkv, d)
        attn_ops.flash_attention_backward(q, k_full, v_full, o, do, lse, ctx["meta"], dq=dq, dk=dk_full, dv=dv_full,
                                          q_offset=ctx["q_off"])
        # sum the ranks' partial dK / dV; every rank keeps the slice of the keys it projected
        parts = dfull.view(b, p, n, 2 * kvw).permute(1, 0, 2, 3).contiguous()
        mine = torch.empty((b, n, 2 * kvw), dtype=dfull.dtype, device=dfull.device)
        dist.reduce_scatter_tensor(mine, parts, group=self.sp_group)
        dk.copy_(mine[..., :kvw].view(b, n, hkv, d))
        dv.copy_(mine[..., kvw:].view(b, n, hkv, d))
        self._count(6)
