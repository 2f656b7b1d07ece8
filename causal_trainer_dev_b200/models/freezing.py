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


# ------------------------------------------------------------------ nested parameter trees
# The same split for parameters held as a nested tree (``embed_tokens / layers[i] / norm / lm_head``,
# the layout of src/causal_trainer/modeling/architecture.py:58-99), for tools that keep that layout:
# export plans, checkpoint converters, anything written against
# src/causal_trainer/modeling/freezing.py:75-219.  Leaves are opaque (tensors, shapes, shardings).
_TOP_KEYS = ("embed_tokens", "layers", "norm", "lm_head")
_LAYER_KEYS = ("attention", "mlp", "input_layernorm", "post_attention_layernorm")
_LAYER_NORMS = ("input_layernorm", "post_attention_layernorm")
_FROZEN_TOP = {"embed": "embed_tokens", "lm_head": "lm_head", "norm": "norm"}


def _check_keys(node, allowed: tuple[str, ...], what: str, required: bool = True) -> None:
    if not isinstance(node, dict):
        raise TypeError(f"{what} must be a mapping")
    missing = [k for k in allowed if k not in node] if required else []
    unexpected = [k for k in node if k not in allowed]
    if missing or unexpected:
        raise ValueError(f"{what} has invalid keys: missing {missing!r}, unexpected {unexpected!r}")


def _check_components(components) -> tuple[str, ...]:
    components = tuple(components)
    if not components:
        raise ValueError("frozen components must not be empty")
    unknown = set(components) - set(SUPPORTED_COMPONENTS)
    if unknown:
        raise ValueError(f"unsupported frozen components: {sorted(unknown)!r}")
    return components


def split_full_trainable_params(params: dict, components) -> tuple[dict, dict]:
    """``(frozen, trainable)`` trees with disjoint leaf paths whose union is ``params``; the
    ``layers`` sequence keeps its type and length in both, leaves are passed on by identity."""
    components = _check_components(components)
    _check_keys(params, _TOP_KEYS, "params")
    layers = params["layers"]
    if not isinstance(layers, (tuple, list)):
        raise TypeError("params['layers'] must be a tuple or list")
    frozen: dict = {}
    trainable: dict = {}
    for component, key in _FROZEN_TOP.items():
        (frozen if component in components else trainable)[key] = params[key]
    frozen_layers, trainable_layers = [], []
    for i, layer in enumerate(layers):
        _check_keys(layer, _LAYER_KEYS, f"params['layers'][{i}]")
        norms = {k: layer[k] for k in _LAYER_NORMS}
        rest = {k: layer[k] for k in layer if k not in _LAYER_NORMS}
        frozen_layers.append(norms if "norm" in components else {})
        trainable_layers.append(rest if "norm" in components else {**rest, **norms})
    frozen["layers"] = type(layers)(frozen_layers)
    trainable["layers"] = type(layers)(trainable_layers)
    return frozen, trainable


def compose_full_trainable_params(frozen: dict, trainable: dict) -> dict:
    """Inverse of :func:`split_full_trainable_params`: one tree in the canonical key order."""
    _check_keys(frozen, _TOP_KEYS, "frozen", required=False)
    _check_keys(trainable, _TOP_KEYS, "trainable", required=False)
    fl, tl = frozen.get("layers"), trainable.get("layers")
    for name, value in (("frozen", fl), ("trainable", tl)):
        if not isinstance(value, (tuple, list)):
            raise TypeError(f"{name}['layers'] must be a tuple or list")
    if type(fl) is not type(tl):
        raise TypeError("frozen and trainable layers must use the same sequence type")
    if len(fl) != len(tl):
        raise ValueError("frozen and trainable must have the same number of layers")
    out: dict = {}
    for key in _TOP_KEYS:
        if key == "layers":
            merged = []
            for i, (f, t) in enumerate(zip(fl, tl)):
                _check_keys(f, _LAYER_KEYS, f"frozen['layers'][{i}]", required=False)
                _check_keys(t, _LAYER_KEYS, f"trainable['layers'][{i}]", required=False)
                both = sorted(set(f) & set(t))
                if both:
                    raise ValueError(f"layer {i} overlaps between frozen and trainable: {both!r}")
                layer = {k: (f[k] if k in f else t[k]) for k in _LAYER_KEYS if k in f or k in t}
                _check_keys(layer, _LAYER_KEYS, f"composed layer {i}")
                merged.append(layer)
            out[key] = type(fl)(merged)
            continue
        if (key in frozen) == (key in trainable):
            state = "overlaps between" if key in frozen else "is missing from"
            raise ValueError(f"{key!r} {state} frozen and trainable")
        out[key] = frozen[key] if key in frozen else trainable[key]
    return out
