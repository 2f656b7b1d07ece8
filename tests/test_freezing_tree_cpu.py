"""Freezing split / compose over nested parameter trees (opaque leaves)."""
import pytest

from causal_trainer_dev_b200.models.freezing import compose_full_trainable_params, split_full_trainable_params


def _proj(bias=False):
    return {"kernel": object(), **({"bias": object()} if bias else {})}


def _layer():
    return {"attention": {"q_proj": _proj(True), "k_proj": _proj(True), "v_proj": _proj(True), "o_proj": _proj()},
            "mlp": {"gate_proj": _proj(), "up_proj": _proj(), "down_proj": _proj()},
            "input_layernorm": {"scale": object()}, "post_attention_layernorm": {"scale": object()}}


def _params(container=tuple):
    return {"embed_tokens": {"embedding": object()}, "layers": container([_layer(), _layer()]),
            "norm": {"scale": object()}, "lm_head": {"kernel": object()}}


def _leaves(node, prefix=()):
    if isinstance(node, dict):
        return {p: v for k, c in node.items() for p, v in _leaves(c, (*prefix, k)).items()}
    if isinstance(node, (tuple, list)):
        return {p: v for i, c in enumerate(node) for p, v in _leaves(c, (*prefix, str(i))).items()}
    return {prefix: node}


@pytest.mark.parametrize("container", [tuple, list])
@pytest.mark.parametrize("components", [("lm_head",), ("embed",), ("norm",), ("lm_head", "embed", "norm")])
def test_split_is_a_partition_and_compose_restores_every_leaf(container, components):
    params = _params(container)
    frozen, trainable = split_full_trainable_params(params, components)
    expected = set()
    if "embed" in components:
        expected.add(("embed_tokens", "embedding"))
    if "lm_head" in components:
        expected.add(("lm_head", "kernel"))
    if "norm" in components:
        expected |= {("norm", "scale")} | {("layers", str(i), n, "scale") for i in range(2)
                                           for n in ("input_layernorm", "post_attention_layernorm")}
    assert set(_leaves(frozen)) == expected
    assert set(_leaves(frozen)).isdisjoint(_leaves(trainable))
    assert isinstance(frozen["layers"], container) and isinstance(trainable["layers"], container)
    composed = compose_full_trainable_params(frozen, trainable)
    assert list(composed) == list(params) and type(composed["layers"]) is container
    original = _leaves(params)
    restored = _leaves(composed)
    assert set(restored) == set(original) and all(restored[p] is leaf for p, leaf in original.items())


def test_split_rejects_malformed_trees():
    missing = _params()
    missing.pop("norm")
    with pytest.raises(ValueError, match=r"params has invalid keys: missing \['norm'\]"):
        split_full_trainable_params(missing, ("norm",))
    with pytest.raises(ValueError, match="unexpected"):
        split_full_trainable_params({**_params(), "extra": {}}, ("norm",))
    broken = _params(list)
    broken["layers"][0].pop("post_attention_layernorm")
    with pytest.raises(ValueError, match="post_attention_layernorm"):
        split_full_trainable_params(broken, ("norm",))
    with pytest.raises(TypeError, match="must be a tuple or list"):
        split_full_trainable_params({**_params(), "layers": {"0": _layer()}}, ("norm",))
    with pytest.raises(ValueError, match="must not be empty"):
        split_full_trainable_params(_params(), ())
    with pytest.raises(ValueError, match="unsupported frozen components"):
        split_full_trainable_params(_params(), ("attention",))


def test_compose_rejects_overlap_and_mismatch():
    frozen, trainable = split_full_trainable_params(_params(list), ("lm_head", "embed", "norm"))
    frozen["layers"][0]["attention"] = {"q_proj": _proj()}
    with pytest.raises(ValueError, match=r"overlaps.*attention"):
        compose_full_trainable_params(frozen, trainable)
    frozen, trainable = split_full_trainable_params(_params(), ("lm_head", "embed", "norm"))
    with pytest.raises(ValueError, match="same number of layers"):
        compose_full_trainable_params(frozen, {**trainable, "layers": trainable["layers"][:-1]})
    with pytest.raises(TypeError, match="same sequence type"):
        compose_full_trainable_params(frozen, {**trainable, "layers": list(trainable["layers"])})
    with pytest.raises(ValueError, match="overlaps"):
        compose_full_trainable_params(frozen, {**trainable, "norm": {"scale": object()}})
