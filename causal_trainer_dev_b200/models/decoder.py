"""Llama-family decoder, stated in plain PyTorch (autograd) — the numerical oracle.

This is the CPU / fp32 path and the reference every sm_100a kernel and the layerwise GPU
engine are tested against.  Pre-norm blocks: RMSNorm -> QKV (+bias) -> RoPE -> attention
-> O -> residual -> RMSNorm -> SwiGLU -> residual, then a final RMSNorm
(src/causal_trainer/modeling/architecture.py:275-424, 537-863).  Segment ids are
canonicalised by contiguous runs and positions reset per segment unless given
(src/causal_trainer/modeling/rotary.py:13-50, 82-110).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Callable

import torch

from ..ops import attention as attn_ops
from ..ops import elementwise as ew
from .config import ModelConfig
from .params import ModelParams


# ----------------------------------------------------------------------------- segments / positions
def canonicalize_segment_ids(attention_mask: torch.Tensor, segment_ids: torch.Tensor | None = None) -> torch.Tensor:
    """One-based ids of contiguous valid runs, zero for padding.

    A label change or a masked token starts a new run, so a reused label after another run
    is a new segment and a valid run labelled 0 is a real segment.
    """
    valid = attention_mask.to(torch.bool)
    if valid.dim() != 2:
        raise ValueError(f"attention_mask must have shape [batch, sequence], got {tuple(valid.shape)}")
    labels = torch.zeros_like(valid, dtype=torch.int32) if segment_ids is None else segment_ids.to(torch.int32)
    if labels.shape != valid.shape:
        raise ValueError(f"segment_ids must have shape {tuple(valid.shape)}, got {tuple(labels.shape)}")
    prev_valid = torch.cat([torch.zeros_like(valid[:, :1]), valid[:, :-1]], dim=1)
    prev_labels = torch.cat([labels[:, :1], labels[:, :-1]], dim=1)
    starts = valid & (~prev_valid | (labels != prev_labels))
    runs = torch.cumsum(starts.to(torch.int32), dim=1, dtype=torch.int32)
    return torch.where(valid, runs, torch.zeros_like(runs))


def make_position_ids(attention_mask: torch.Tensor, segment_ids: torch.Tensor | None = None,
                      canonical: bool = False) -> torch.Tensor:
    """Zero-based positions that restart at every segment; padding gets 0."""
    valid = attention_mask.to(torch.bool)
    seg = segment_ids.to(torch.int32) if canonical else canonicalize_segment_ids(valid, segment_ids)
    b, s = valid.shape
    idx = torch.arange(s, device=valid.device, dtype=torch.int32).expand(b, s)
    prev = torch.cat([torch.zeros_like(seg[:, :1]), seg[:, :-1]], dim=1)
    starts = valid & ((seg != prev) | (prev == 0))
    start_idx = torch.cummax(torch.where(starts, idx, torch.zeros_like(idx)), dim=1).values
    return torch.where(valid, idx - start_idx, torch.zeros_like(idx))


# ----------------------------------------------------------------------------- options
@dataclass
class ForwardOptions:
    attn_mechanism: str = "vanilla"           # "vanilla" (oracle) | "efficient" (sm_100a flash kernels)
    gradient_checkpointing: bool = False      # recompute each layer in the backward pass
    mlp_chunk_size: int = 0                   # rows per MLP tile (0 = untiled)
    attention_options: object | None = None   # MoBA options (models.moba.AttentionOptions) or None
    optimizer_step: int | None = None         # for dense_after_step
    lora: object | None = None                # models.lora.LoraState or None
    compute_dtype: torch.dtype | None = None


def _linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, lora_pair=None) -> torch.Tensor:
    y = x @ w.t().to(x.dtype)
    if lora_pair is not None:
        a, bb = lora_pair            # a [in, r], bb [r, out]; no alpha: kernel + A @ B
        y = y + (x @ a.to(x.dtype)) @ bb.to(x.dtype)
    if b is not None:
        y = y + b.to(x.dtype)
    return y


def _mlp(x: torch.Tensor, gu_w: torch.Tensor, down_w: torch.Tensor, lora, li: int, chunk: int) -> torch.Tensor:
    f = gu_w.shape[0] // 2

    def run(rows: torch.Tensor) -> torch.Tensor:
        gate = _linear(rows, gu_w[:f], None, lora.pair(li, "gate_proj") if lora else None)
        up = _linear(rows, gu_w[f:], None, lora.pair(li, "up_proj") if lora else None)
        act = torch.nn.functional.silu(gate.float()).to(rows.dtype) * up
        return _linear(act, down_w, None, lora.pair(li, "down_proj") if lora else None)

    if chunk <= 0 or x.shape[1] <= chunk:
        return run(x)
    return torch.cat([run(x[:, s0:s0 + chunk]) for s0 in range(0, x.shape[1], chunk)], dim=1)


def _attention(q, k, v, seg, attention_end, meta, opts: ForwardOptions, layer_index: int, cfg: ModelConfig):
    scale = 1.0 / math.sqrt(cfg.head_dim)
    ao = opts.attention_options
    if ao is not None and ao.applies_to_layer(layer_index, cfg.num_hidden_layers, opts.optimizer_step):
        from . import moba

        return moba.moba_attention(q, k, v, seg, ao, scale, meta)
    if opts.attn_mechanism == "vanilla" or not q.is_cuda:
        return attn_ops.vanilla_attention(q, k, v, seg, attention_end, scale)
    return attn_ops.flash_attention(q, k, v, meta, scale)


def decoder_layer(h: torch.Tensor, unit_views: dict[str, torch.Tensor], cfg: ModelConfig, cos, sin, seg,
                  attention_end, meta, opts: ForwardOptions, li: int) -> torch.Tensor:
    b, s, d = h.shape
    q_w, kv_w = cfg.query_width, cfg.key_value_width
    lora = opts.lora
    x = ew.rmsnorm_reference(h, unit_views["ln1"], cfg.rms_norm_eps)
    qkv_w, qkv_b = unit_views["qkv_w"], unit_views.get("qkv_b")
    if lora is None:
        qkv = _linear(x, qkv_w, qkv_b)
        q, k, v = qkv[..., :q_w], qkv[..., q_w:q_w + kv_w], qkv[..., q_w + kv_w:]
    else:
        bq = bk = bv = None
        if qkv_b is not None:
            bq, bk, bv = qkv_b[:q_w], qkv_b[q_w:q_w + kv_w], qkv_b[q_w + kv_w:]
        q = _linear(x, qkv_w[:q_w], bq, lora.pair(li, "q_proj"))
        k = _linear(x, qkv_w[q_w:q_w + kv_w], bk, lora.pair(li, "k_proj"))
        v = _linear(x, qkv_w[q_w + kv_w:], bv, lora.pair(li, "v_proj"))
    q = q.reshape(b * s, cfg.num_attention_heads, cfg.head_dim)
    k = k.reshape(b * s, cfg.num_key_value_heads, cfg.head_dim)
    q = ew.rope_reference(q, cos, sin, cfg.rotary_dim, cfg.rope_style).view(b, s, -1, cfg.head_dim)
    k = ew.rope_reference(k, cos, sin, cfg.rotary_dim, cfg.rope_style).view(b, s, -1, cfg.head_dim)
    v = v.reshape(b, s, cfg.num_key_value_heads, cfg.head_dim)
    ctx = _attention(q.contiguous(), k.contiguous(), v.contiguous(), seg, attention_end, meta, opts, li, cfg)
    h = h + _linear(ctx.reshape(b, s, q_w), unit_views["o_w"], None, lora.pair(li, "o_proj") if lora else None)
    x = ew.rmsnorm_reference(h, unit_views["ln2"], cfg.rms_norm_eps)
    return h + _mlp(x, unit_views["gu_w"], unit_views["down_w"], lora, li, opts.mlp_chunk_size)


def _unit_views(params: ModelParams, name: str) -> dict[str, torch.Tensor]:
    unit = params.units[name]
    return {seg.name: unit.view(seg.name) for seg in unit.layout.segments}


def embedding_lookup(table: torch.Tensor, input_ids: torch.Tensor, pad_token_id: int) -> torch.Tensor:
    """Returns the stored rows (the pad row included); the pad row receives no gradient."""
    out = torch.nn.functional.embedding(input_ids, table)
    if table.requires_grad and torch.is_grad_enabled():
        keep = (input_ids != pad_token_id).unsqueeze(-1).to(out.dtype)
        out = out * keep + (out * (1 - keep)).detach()
    return out


def decoder_forward(
    params: ModelParams,
    input_ids: torch.Tensor,
    attention_mask: torch.Tensor,
    segment_ids: torch.Tensor | None = None,
    position_ids: torch.Tensor | None = None,
    attention_end: torch.Tensor | None = None,
    options: ForwardOptions | None = None,
) -> torch.Tensor:
    """Final-norm hidden states ``[B,S,d]`` for token ids ``[B,S]``."""
    cfg = params.config
    opts = options or ForwardOptions()
    seg = canonicalize_segment_ids(attention_mask, segment_ids)
    if position_ids is None:
        position_ids = make_position_ids(attention_mask, seg, canonical=True)
    dtype = opts.compute_dtype or params.dtype
    inv_freq = ew.inverse_frequencies(cfg.rotary_dim, cfg.rope_theta, device=input_ids.device)
    cos, sin = ew.rope_table_reference(position_ids.to(input_ids.device), inv_freq, dtype)
    meta = None
    needs_meta = input_ids.is_cuda and (opts.attn_mechanism != "vanilla" or opts.attention_options is not None)
    if needs_meta and seg.shape[1] % attn_ops.BLOCK == 0:
        meta = attn_ops.build_attention_meta(seg, attention_end)
    elif opts.attn_mechanism != "vanilla" and input_ids.is_cuda:
        raise ValueError("the efficient attention backend needs a sequence length that is a multiple of 128")
    embed = params.units["embed"].view("embed")
    if opts.lora is not None and opts.lora.train_embed_and_lm_head:
        embed = opts.lora.embed
    h = embedding_lookup(embed, input_ids, cfg.pad_token_id).to(dtype)
    for li in range(cfg.num_hidden_layers):
        views = _unit_views(params, f"layer.{li}")
        fn: Callable = decoder_layer
        if opts.gradient_checkpointing and torch.is_grad_enabled():
            from torch.utils.checkpoint import checkpoint

            h = checkpoint(fn, h, views, cfg, cos, sin, seg, attention_end, meta, opts, li, use_reentrant=False)
        else:
            h = fn(h, views, cfg, cos, sin, seg, attention_end, meta, opts, li)
    return ew.rmsnorm_reference(h, params.units["final"].view("norm"), cfg.rms_norm_eps)


def lm_head_logits(params: ModelParams, hidden: torch.Tensor) -> torch.Tensor:
    """Full logits (tests and tiny models only)."""
    return hidden @ params.units["final"].view("lm_head").t().to(hidden.dtype)
