"""Loss front-end: shifted next-token targets, aligned (MaskGIT) targets, backend dispatch.

A shifted target at position t+1 is supervised only when both tokens of the edge are
valid, the edge stays inside one canonical segment, and the label is not ``ignore_index``;
assistant masks and fractional loss weights are read at the *target* position
(src/causal_trainer/training/losses.py:21-85).  The targets are always padded back to the
full sequence with one zero-weight column (the reference does this only under sequence
parallelism, losses.py:211-218), so every backend sees ``B*S`` rows and the last position
gets exactly zero gradient.  Results are sums ``(nll_sum, weight_sum)``; normalisation is
global and happens in the step function.
"""
from __future__ import annotations

import torch

from ..models.decoder import canonicalize_segment_ids
from ..ops import cross_entropy as ce


def shifted_targets_and_weights(
    input_ids: torch.Tensor,
    attention_mask: torch.Tensor | None,
    segment_ids: torch.Tensor | None = None,
    assistant_mask: torch.Tensor | None = None,
    loss_mask: torch.Tensor | None = None,
    labels: torch.Tensor | None = None,
    *,
    ignore_index: int = -100,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns ``(targets [B,S-1] int64, weights [B,S-1] fp32)``; masked targets are 0."""
    tokens = input_ids.long()
    if tokens.dim() != 2:
        raise ValueError(f"input_ids must have shape [batch, sequence], got {tuple(tokens.shape)}")
    labels = tokens if labels is None else labels.long()
    if labels.shape != tokens.shape:
        raise ValueError(f"labels must have shape {tuple(tokens.shape)}, got {tuple(labels.shape)}")
    valid_tokens = torch.ones_like(tokens, dtype=torch.bool) if attention_mask is None else (attention_mask == 1)
    if valid_tokens.shape != tokens.shape:
        raise ValueError(f"attention_mask must have shape {tuple(tokens.shape)}")
    targets = labels[:, 1:]
    valid = valid_tokens[:, :-1] & valid_tokens[:, 1:] & (targets != ignore_index)
    if segment_ids is not None:
        if segment_ids.shape != tokens.shape:
            raise ValueError(f"segment_ids must have shape {tuple(tokens.shape)}")
        seg = canonicalize_segment_ids(valid_tokens, segment_ids)
        valid &= (seg[:, :-1] == seg[:, 1:]) & (seg[:, 1:] != 0)
    weights = valid.float()
    if assistant_mask is not None:
        if assistant_mask.shape != tokens.shape:
            raise ValueError(f"assistant_mask must have shape {tuple(tokens.shape)}")
        weights = weights * (assistant_mask[:, 1:] != 0).float()
    if loss_mask is not None:
        if loss_mask.shape != tokens.shape:
            raise ValueError(f"loss_mask must have shape {tuple(tokens.shape)}")
        weights = weights * loss_mask[:, 1:].float()
    return torch.where(weights > 0, targets, torch.zeros_like(targets)), weights


def aligned_targets_and_weights(batch: dict[str, torch.Tensor]) -> tuple[torch.Tensor, torch.Tensor]:
    """Targets/weights aligned to hidden-state positions, ``[B,S]`` each.

    Uses ``prediction_targets``/``prediction_weights`` when the batch carries them (mixed
    AR + MaskGIT), otherwise the shifted rule padded with one zero-weight column.
    """
    if ("prediction_targets" in batch) != ("prediction_weights" in batch):
        raise ValueError("prediction_targets and prediction_weights must be supplied together")
    if "prediction_targets" in batch:
        weights = batch["prediction_weights"].float()
        targets = torch.where(weights > 0, batch["prediction_targets"].long(), torch.zeros_like(weights).long())
        if targets.shape != batch["input_ids"].shape:
            raise ValueError("prediction targets/weights must match [batch, sequence]")
        return targets, weights
    targets, weights = shifted_targets_and_weights(
        batch["input_ids"], batch.get("attention_mask"), batch.get("segment_ids"),
        assistant_mask=None, loss_mask=batch.get("loss_weights"),
    )
    pad_t = torch.zeros_like(targets[:, :1])
    pad_w = torch.zeros_like(weights[:, :1])
    return torch.cat([targets, pad_t], dim=1), torch.cat([weights, pad_w], dim=1)


def linear_cross_entropy(hidden: torch.Tensor, head: torch.Tensor, targets: torch.Tensor, weights: torch.Tensor, *,
                         implementation: str = "xla", token_budget: int = 4096, cut_chunk_size: int = 0):
    """``(nll_sum, weight_sum)`` of ``hidden [rows,d] @ head[vocab,d]^T`` under one of the backends.

    ``cut``: projection-fused tcgen05 kernels (GPU bf16 only); ``pallas``/``xla``: chunked
    logits with per-chunk recompute (any device).  On CPU every name maps to the chunked path.
    """
    if implementation not in ("auto", "cut", "pallas", "xla"):
        raise ValueError(f"unknown loss implementation {implementation!r}")
    use_cut = implementation in ("auto", "cut") and hidden.is_cuda and hidden.dtype == torch.bfloat16
    if implementation == "cut" and not use_cut:
        raise ValueError("the cut loss backend needs bf16 tensors on a CUDA device")
    if use_cut:
        return ce.cut_cross_entropy(hidden.contiguous(), head, targets, weights, cut_chunk_size or 4096)
    return ce.chunked_cross_entropy(hidden, head, targets, weights, token_budget)


def causal_lm_loss(hidden_states: torch.Tensor, head: torch.Tensor, batch: dict[str, torch.Tensor], **kw):
    """Loss sums for final-norm hidden states ``[B,S,d]``."""
    targets, weights = aligned_targets_and_weights(batch)
    b, s, d = hidden_states.shape
    return linear_cross_entropy(hidden_states.reshape(b * s, d), head, targets.reshape(-1), weights.reshape(-1), **kw)


def shifted_loss_mask(input_ids, attention_mask, segment_ids=None, assistant_mask=None, loss_mask=None, labels=None, *,
                      ignore_index: int = -100) -> tuple[torch.Tensor, torch.Tensor]:
    """``(targets, supervised)``: the shifted targets and a boolean mask of the positions that carry
    any weight (src/causal_trainer/training/losses.py:88-109)."""
    targets, weights = shifted_targets_and_weights(input_ids, attention_mask, segment_ids, assistant_mask, loss_mask,
                                                   labels, ignore_index=ignore_index)
    return targets, weights > 0


def chunked_causal_lm_loss(hidden_states: torch.Tensor, lm_head: torch.Tensor, input_ids: torch.Tensor,
                           attention_mask: torch.Tensor | None, segment_ids: torch.Tensor | None = None,
                           assistant_mask: torch.Tensor | None = None, loss_weights: torch.Tensor | None = None, *,
                           token_budget: int = 128, loss_implementation: str = "xla", cut_chunk_size: int = 0,
                           prediction_targets: torch.Tensor | None = None,
                           prediction_weights: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """``(nll_sum, weight_sum)`` from separate tensors instead of a batch dictionary, without ever
    holding full-sequence logits (src/causal_trainer/training/losses.py:152-231).  ``lm_head`` is
    ``[vocab, hidden]`` (the Hugging Face orientation).  The shifted rule multiplies padding,
    segment-boundary, assistant and fractional weights; explicit ``prediction_targets`` /
    ``prediction_weights`` (aligned to hidden-state positions) replace it."""
    if (prediction_targets is None) != (prediction_weights is None):
        raise ValueError("prediction_targets and prediction_weights must be supplied together")
    b, s, d = hidden_states.shape
    if prediction_targets is not None:
        targets, weights = aligned_targets_and_weights({"input_ids": input_ids, "prediction_targets": prediction_targets,
                                                        "prediction_weights": prediction_weights})
    else:
        t, w = shifted_targets_and_weights(input_ids, attention_mask, segment_ids, assistant_mask, loss_weights)
        targets = torch.cat([t, torch.zeros_like(t[:, :1])], dim=1)
        weights = torch.cat([w, torch.zeros_like(w[:, :1])], dim=1)
    return linear_cross_entropy(hidden_states.reshape(b * s, d), lm_head, targets.reshape(-1), weights.reshape(-1),
                                implementation=loss_implementation, token_budget=token_budget,
                                cut_chunk_size=cut_chunk_size)


def mean_loss(nll_sum: torch.Tensor, token_count: torch.Tensor) -> torch.Tensor:
    return nll_sum / torch.clamp(token_count, min=1.0)
