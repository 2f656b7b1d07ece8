"""Component freezing for full-rank training: ``--frozen_parameters lm_head|embed|norm``.

``embed`` is the token embedding, ``lm_head`` the output projection, and ``norm`` the final
RMSNorm together with both norms of every decoder layer; attention and MLP weights always
train (src/causal_trainer/modeling/freezing.py:75-120).  With flat unit buffers a frozen
component is simply a set of ``(unit, segment)`` pairs that get no optimizer region and, on
the GPU engine, no gradient kernel.
"""
from __future__ import annotations

from .config import ModelConfig

SUPPORTED_COMPONENTS = ("lm_head", "embed", "norm")


def frozen_segments(cfg: ModelConfig, components: tuple[str, ...]) -> set[tuple[str, str]]:
    """``{(unit name, segment name)}`` that must not be updated."""
    unknown = set(components) - set(SUPPORTED_COMPONENTS)
    if unknown:
        raise ValueError(f"unsupported frozen components: {sorted(unknown)!r}")
    out: set[tuple[str, str]] = set()
    if "embed" in components:
        out.add(("embed", "embed"))
    if "lm_head" in components:
        out.add(("final", "lm_head"))
    if "norm" in components:
        out.add(("final", "norm"))
        for i in range(cfg.num_hidden_layers):
            out.add((f"layer.{i}", "ln1"))
            out.add((f"layer.{i}", "ln2"))
    return out


def split_trainable(cfg: ModelConfig, components: tuple[str, ...], hf_names: list[str]) -> tuple[list[str], list[str]]:
    """HF tensor names split into (frozen, trainable) for reporting and export plans."""
    frozen, trainable = [], []
    for name in hf_names:
        is_norm = name.endswith("layernorm.weight") or name == "model.norm.weight"
        hit = (("embed" in components and name == "model.embed_tokens.weight")
               or ("lm_head" in components and name == "lm_head.weight") or ("norm" in components and is_norm))
        (frozen if hit else trainable).append(name)
    return frozen, trainable
