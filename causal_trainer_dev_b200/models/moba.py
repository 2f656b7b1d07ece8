"""MoBA (mixture of block attention): options, routing and the attention operators.

Semantics (src/causal_trainer/modeling/approximate_attention.py:29-127 and the slow oracle of
tests/modeling/test_approximate_attention.py:40-62): inside each packed document, keys are cut
into blocks of ``moba_block_size`` tokens counted from the document start.  A query in block
``c`` scores every *completed* block ``< c`` of its own document with ``q . mean(K_block)``
(fp32, per query head against its KV head), keeps the ``top_k - 1`` best, adds its own block
causally and runs ONE softmax over the union.  ``top_k`` therefore includes the current
block, and ``top_k * block >= S`` is exactly dense attention.

Two operators share the routing:

* ``reference``: an explicit visibility mask and an fp32 softmax (any device, autograd);
* native (``auto``/``pallas`` on CUDA): routing runs on the GPU in PyTorch, attention runs on
  the tcgen05 flash kernels tile by tile with a per-(query, head) block-selection bitmask, so
  only key tiles that at least one query of the tile selected are ever loaded.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class AttentionOptions:
    method: str = "dense"
    backend: str = "auto"
    query_chunk_size: int = 128
    key_chunk_size: int = 512
    moba_block_size: int = 4096
    moba_top_k: int = 12
    dense_prefix_layers: int = 0
    dense_suffix_layers: int = 0
    dense_after_step: int | None = None

    def __post_init__(self) -> None:
        if self.method not in ("dense", "moba"):
            raise ValueError(f"unknown attention method: {self.method!r}")
        if self.backend not in ("auto", "pallas", "reference"):
            raise ValueError(f"unknown sparse attention backend: {self.backend!r}")
        for name in ("query_chunk_size", "key_chunk_size", "moba_block_size", "moba_top_k"):
            value = getattr(self, name)
            if type(value) is not int or value < 1:
                raise ValueError(f"{name} must be a positive integer")
        for name in ("dense_prefix_layers", "dense_suffix_layers"):
            value = getattr(self, name)
            if type(value) is not int or value < 0:
                raise ValueError(f"{name} must be a nonnegative integer")
        if self.dense_after_step is not None and (type(self.dense_after_step) is not int or self.dense_after_step < 0):
            raise ValueError("dense_after_step must be a nonnegative integer or None")
        if self.method == "dense" and (self.dense_prefix_layers or self.dense_suffix_layers
                                       or self.dense_after_step is not None):
            raise ValueError("dense layer/recovery options require moba")

    def validate_layers(self, layers: int) -> None:
        if self.dense_prefix_layers + self.dense_suffix_layers > layers:
            raise ValueError("dense prefix/suffix layer counts cannot exceed num_hidden_layers")

    @property
    def needs_dense_backend(self) -> bool:
        return (self.method == "dense" or self.dense_prefix_layers > 0 or self.dense_suffix_layers > 0
                or self.dense_after_step is not None)

    def applies_to_layer(self, layer: int, num_layers: int, optimizer_step: int | None) -> bool:
        """Whether ``layer`` runs MoBA at this optimizer step (dense prefix/suffix/recovery excluded)."""
        if self.method != "moba":
            return False
        if layer < self.dense_prefix_layers or layer >= num_layers - self.dense_suffix_layers:
            return False
        if self.dense_after_step is not None and optimizer_step is not None and optimizer_step >= self.dense_after_step:
            return False
        return True


# ----------------------------------------------------------------------------------------- routing
def segment_starts(segments: torch.Tensor) -> torch.Tensor:
    """Index of the first token of each token's document (0 for padding)."""
    b, s = segments.shape
    idx = torch.arange(s, device=segments.device).expand(b, s)
    prev = torch.cat([torch.zeros_like(segments[:, :1]), segments[:, :-1]], dim=1)
    first = (segments != 0) & (segments != prev)
    return torch.cummax(torch.where(first, idx, torch.zeros_like(idx)), dim=1).values


def block_means(key: torch.Tensor, segments: torch.Tensor, starts: torch.Tensor, block: int) -> torch.Tensor:
    """Mean key of every *complete* document-relative block: ``[B, S/…]`` indexed by block end.

    Returns ``means [B,S,Hkv,D]`` where ``means[b, e]`` is the mean over the block that ends at
    token ``e`` (only meaningful where ``(e - start + 1) % block == 0``).  Sums stay inside one
    block, so other documents cannot perturb the rounding of a routing score.  No gradient.
    """
    with torch.no_grad():
        kf = key.float()
        b, s = segments.shape
        idx = torch.arange(s, device=key.device).expand(b, s)
        rel = idx - starts
        csum = torch.cumsum(kf, dim=1)
        block_first = idx - (rel % block)                     # first token of my block
        before = torch.gather(
            torch.cat([torch.zeros_like(csum[:, :1]), csum], dim=1), 1,
            block_first[:, :, None, None].expand(-1, -1, kf.shape[2], kf.shape[3]),
        )
        return (csum - before) / block


def moba_selected_blocks(query: torch.Tensor, key: torch.Tensor, segments: torch.Tensor, block: int, top_k: int):
    """Per (token, query head): current block id and up to ``top_k-1`` selected earlier block ids.

    Returns ``(current [B,S], previous [B,S,Hq,top_k-1] with -1 for unused, starts [B,S])``.
    """
    b, s, hq, d = query.shape
    hkv = key.shape[2]
    g = hq // hkv
    starts = segment_starts(segments)
    idx = torch.arange(s, device=query.device).expand(b, s)
    current = torch.where(segments != 0, (idx - starts) // block, torch.zeros_like(idx))
    candidates = (s + block - 1) // block
    count = min(top_k - 1, max(candidates - 1, 0))
    if count == 0:
        return current, torch.empty((b, s, hq, 0), dtype=torch.long, device=query.device), starts
    means = block_means(key, segments, starts, block)                               # [B,S,Hkv,D]
    blk = torch.arange(candidates, device=query.device)
    ends = (starts[:, :, None] + (blk[None, None, :] + 1) * block - 1).clamp(0, s - 1)  # [B,S,C]
    gathered = means[torch.arange(b, device=query.device)[:, None, None], ends]       # [B,S,C,Hkv,D]
    qf = query.float().view(b, s, hkv, g, d)
    scores = torch.einsum("bshgd,bschd->bshgc", qf, gathered).reshape(b, s, hq, candidates)
    completed = blk[None, None, None, :] < current[:, :, None, None]
    scores = torch.where(completed, scores, torch.full_like(scores, float("-inf")))
    # stable order for ties: sort by (-score, block id)
    order = torch.sort(-scores, dim=-1, stable=True).indices[..., :count]
    chosen = torch.gather(scores, -1, order)
    previous = torch.where(torch.isfinite(chosen), order, torch.full_like(order, -1))
    return current, previous, starts


def moba_visibility(query: torch.Tensor, key: torch.Tensor, segments: torch.Tensor, block: int, top_k: int):
    """Dense boolean mask ``[B,Hq,S,S]`` of the MoBA graph (oracle / small shapes only)."""
    b, s, hq, _ = query.shape
    current, previous, starts = moba_selected_blocks(query.detach(), key.detach(), segments, block, top_k)
    idx = torch.arange(s, device=query.device)
    same = (segments[:, :, None] == segments[:, None, :]) & (segments[:, :, None] != 0)   # [B,Sq,Sk]
    key_block = torch.where(same, (idx[None, None, :] - starts[:, :, None]) // block, torch.full_like(same, -2, dtype=torch.long))
    causal = idx[None, None, :] <= idx[None, :, None]
    in_current = (key_block == current[:, :, None]) & causal & same                        # [B,Sq,Sk]
    mask = in_current[:, None].expand(b, hq, s, s).clone()
    for r in range(previous.shape[-1]):
        sel = previous[..., r].permute(0, 2, 1)                                            # [B,Hq,Sq]
        mask |= (key_block[:, None] == sel[..., None]) & (sel[..., None] >= 0) & same[:, None]
    return mask


def _masked_attention(query, key, value, mask, scale):
    b, s, hq, d = query.shape
    hkv = key.shape[2]
    g = hq // hkv
    qf = query.float().view(b, s, hkv, g, d)
    scores = torch.einsum("bqhgd,bkhd->bhgqk", qf, key.float()) * scale
    m = mask.view(b, hkv, g, s, s)
    scores = scores.masked_fill(~m, torch.finfo(torch.float32).min)
    probs = torch.softmax(scores, dim=-1) * m
    out = torch.einsum("bhgqk,bkhd->bqhgd", probs, value.float())
    return out.reshape(b, s, hq, d).to(query.dtype)


def _native_available() -> bool:
    try:
        from ..ops import moba as _  # noqa: F401
    except ImportError:
        return False
    return True


def moba_attention(query, key, value, segments, options: AttentionOptions, scale: float, meta=None):
    """MoBA attention for ``[B,S,H,D]`` operands; dispatches on ``options.backend`` and device."""
    s = query.shape[1]
    block = min(options.moba_block_size, s)
    if options.moba_top_k * block >= s:
        # every document history fits the budget: the graph is exactly dense
        from ..ops import attention as attn_ops

        if query.is_cuda and meta is not None and options.backend != "reference":
            return attn_ops.flash_attention(query, key, value, meta, scale)
        return attn_ops.vanilla_attention(query, key, value, segments, None, scale)
    native = _native_available() and query.is_cuda and options.backend != "reference" \
        and query.dtype == torch.bfloat16 and s % 128 == 0 and block >= 128
    if native:
        from ..ops import moba as moba_ops

        return moba_ops.moba_flash_attention(query, key, value, segments, block, options.moba_top_k, scale, meta)
    mask = moba_visibility(query, key, segments, block, options.moba_top_k)
    return _masked_attention(query, key, value, mask, scale)
