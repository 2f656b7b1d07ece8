"""Parameter storage: flat per-unit buffers with Hugging Face named views.

The reference keeps a pytree of per-projection arrays in JAX ``[in,out]`` layout and
transposes on checkpoint I/O (src/causal_trainer/modeling/architecture.py:58-152,
src/causal_trainer/checkpointing/huggingface.py:108-140).  Here every *unit* (the embedding,
each decoder layer, the final norm + LM head) owns ONE contiguous buffer in the
``nn.Linear`` ``[out,in]`` layout that checkpoints use, so

* FSDP shards, gathers and reduce-scatters a unit with a single contiguous transfer;
* the optimizer sweeps a unit with one or two fused launches (vectors first, no decay;
  matrices after, decayed);
* Q/K/V and gate/up are stored adjacently and consumed as one ``[q+2kv, d]`` / ``[2f, d]``
  GEMM operand, while ``q_proj.weight`` ... stay addressable as row-slice views for I/O.

Initialisation matches ``init_params``: N(0, initializer_range) for matrices, the padding
row of the embedding zeroed, norm scales one, biases zero.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterator

import torch

from .config import ModelConfig

ALIGN = 64  # elements; keeps every segment 128-byte aligned for TMA and vector access


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


@dataclass(frozen=True)
class Segment:
    name: str            # internal name inside the unit ("qkv_w", "ln1", ...)
    shape: tuple[int, ...]
    offset: int          # element offset inside the unit buffer
    decay: bool          # weight decay applies (ndim > 1)

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


@dataclass(frozen=True)
class UnitLayout:
    name: str
    segments: tuple[Segment, ...]
    numel: int           # padded total
    vector_numel: int    # leading region holding the 1-D segments (no decay)

    def segment(self, name: str) -> Segment:
        for seg in self.segments:
            if seg.name == name:
                return seg
        raise KeyError(name)


def _layout(name: str, entries: list[tuple[str, tuple[int, ...]]]) -> UnitLayout:
    vectors = [(n, s) for n, s in entries if len(s) == 1]
    matrices = [(n, s) for n, s in entries if len(s) > 1]
    segs, off = [], 0
    for n, s in vectors:
        segs.append(Segment(n, s, off, False))
        off = _round_up(off + segs[-1].numel, ALIGN)
    vector_numel = off
    for n, s in matrices:
        segs.append(Segment(n, s, off, True))
        off = _round_up(off + segs[-1].numel, ALIGN)
    return UnitLayout(name, tuple(segs), off, vector_numel)


def layer_layout(cfg: ModelConfig, index: int) -> UnitLayout:
    d, f, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.query_width, cfg.key_value_width
    entries: list[tuple[str, tuple[int, ...]]] = [("ln1", (d,)), ("ln2", (d,))]
    if cfg.attention_bias:
        entries.append(("qkv_b", (q + 2 * kv,)))
    entries += [("qkv_w", (q + 2 * kv, d)), ("o_w", (d, q)), ("gu_w", (2 * f, d)), ("down_w", (d, f))]
    return _layout(f"layer.{index}", entries)


def embed_layout(cfg: ModelConfig) -> UnitLayout:
    return _layout("embed", [("embed", (cfg.vocab_size, cfg.hidden_size))])


def final_layout(cfg: ModelConfig) -> UnitLayout:
    return _layout("final", [("norm", (cfg.hidden_size,)), ("lm_head", (cfg.vocab_size, cfg.hidden_size))])


def unit_layouts(cfg: ModelConfig) -> list[UnitLayout]:
    return [embed_layout(cfg)] + [layer_layout(cfg, i) for i in range(cfg.num_hidden_layers)] + [final_layout(cfg)]


# HF name -> (unit, segment, row_start, row_count) ; rows index dim 0 of the segment.
def hf_name_map(cfg: ModelConfig) -> dict[str, tuple[str, str, int, int]]:
    q, kv, f = cfg.query_width, cfg.key_value_width, cfg.intermediate_size
    out: dict[str, tuple[str, str, int, int]] = {"model.embed_tokens.weight": ("embed", "embed", 0, cfg.vocab_size)}
    for i in range(cfg.num_hidden_layers):
        u, p = f"layer.{i}", f"model.layers.{i}."
        out[p + "input_layernorm.weight"] = (u, "ln1", 0, cfg.hidden_size)
        out[p + "post_attention_layernorm.weight"] = (u, "ln2", 0, cfg.hidden_size)
        out[p + "self_attn.q_proj.weight"] = (u, "qkv_w", 0, q)
        out[p + "self_attn.k_proj.weight"] = (u, "qkv_w", q, kv)
        out[p + "self_attn.v_proj.weight"] = (u, "qkv_w", q + kv, kv)
        if cfg.attention_bias:
            out[p + "self_attn.q_proj.bias"] = (u, "qkv_b", 0, q)
            out[p + "self_attn.k_proj.bias"] = (u, "qkv_b", q, kv)
            out[p + "self_attn.v_proj.bias"] = (u, "qkv_b", q + kv, kv)
        out[p + "self_attn.o_proj.weight"] = (u, "o_w", 0, cfg.hidden_size)
        out[p + "mlp.gate_proj.weight"] = (u, "gu_w", 0, f)
        out[p + "mlp.up_proj.weight"] = (u, "gu_w", f, f)
        out[p + "mlp.down_proj.weight"] = (u, "down_w", 0, cfg.hidden_size)
    out["model.norm.weight"] = ("final", "norm", 0, cfg.hidden_size)
    out["lm_head.weight"] = ("final", "lm_head", 0, cfg.vocab_size)
    return out


def hf_export_order(cfg: ModelConfig) -> list[str]:
    """Tensor order inside ``model.safetensors``.

    The reference writes leaves in the flatten order of its parameter tree, i.e. sorted
    keys: embedding, then per layer attention.{k,o,q,v}_proj (bias before kernel),
    input_layernorm, mlp.{down,gate,up}_proj, post_attention_layernorm, then lm_head, then
    the final norm (src/causal_trainer/checkpointing/huggingface.py:1156).
    """
    names = ["model.embed_tokens.weight"]
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        for proj in ("k_proj", "o_proj", "q_proj", "v_proj"):
            if cfg.attention_bias and proj != "o_proj":
                names.append(p + f"self_attn.{proj}.bias")
            names.append(p + f"self_attn.{proj}.weight")
        names.append(p + "input_layernorm.weight")
        names += [p + f"mlp.{m}.weight" for m in ("down_proj", "gate_proj", "up_proj")]
        names.append(p + "post_attention_layernorm.weight")
    names += ["lm_head.weight", "model.norm.weight"]
    return names


@dataclass
class Unit:
    layout: UnitLayout
    data: torch.Tensor                    # flat [numel]
    grad: torch.Tensor | None = None      # flat, same layout (bf16 or fp32)
    views: dict[str, torch.Tensor] = field(default_factory=dict)

    def view(self, name: str, of: torch.Tensor | None = None) -> torch.Tensor:
        seg = self.layout.segment(name)
        base = self.data if of is None else of
        return base[seg.offset:seg.offset + seg.numel].view(seg.shape)


class ModelParams:
    """All units of one model replica (or, under FSDP, the gathered full views)."""

    def __init__(self, cfg: ModelConfig, dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu",
                 allocate: bool = True):
        self.config = cfg
        self.dtype = dtype
        self.device = torch.device(device)
        self.units: dict[str, Unit] = {}
        for lay in unit_layouts(cfg):
            data = torch.zeros(lay.numel, dtype=dtype, device=self.device) if allocate else torch.empty(0)
            self.units[lay.name] = Unit(lay, data)
        self._map = hf_name_map(cfg)

    # ---- construction ----
    @classmethod
    def init_random(cls, cfg: ModelConfig, seed: int = 0, dtype=torch.bfloat16, device="cpu") -> "ModelParams":
        self = cls(cfg, dtype, device)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        for name in hf_export_order(cfg):
            t = self.tensor(name)
            if name.endswith("layernorm.weight") or name == "model.norm.weight":
                t.fill_(1.0)
            elif name.endswith(".bias"):
                t.zero_()
            else:
                # generate in bounded slices so a 128k x 4096 matrix never needs a second fp32 copy
                rows = max(1, (1 << 24) // t.shape[1])
                for r0 in range(0, t.shape[0], rows):
                    block = torch.empty((min(rows, t.shape[0] - r0), t.shape[1]), dtype=torch.float32)
                    block.normal_(0.0, cfg.initializer_range, generator=gen)
                    t[r0:r0 + block.shape[0]].copy_(block)
        self.tensor("model.embed_tokens.weight")[cfg.pad_token_id].zero_()
        return self

    # ---- access ----
    def tensor(self, hf_name: str) -> torch.Tensor:
        unit, seg, r0, rn = self._map[hf_name]
        return self.units[unit].view(seg)[r0:r0 + rn]

    def grad_tensor(self, hf_name: str) -> torch.Tensor | None:
        unit, seg, r0, rn = self._map[hf_name]
        u = self.units[unit]
        if u.grad is None:
            return None
        return u.view(seg, of=u.grad)[r0:r0 + rn]

    def named_tensors(self) -> Iterator[tuple[str, torch.Tensor]]:
        for name in hf_export_order(self.config):
            yield name, self.tensor(name)

    def hf_names(self) -> list[str]:
        return hf_export_order(self.config)

    def layer(self, i: int) -> Unit:
        return self.units[f"layer.{i}"]

    def numel(self) -> int:
        return sum(t.numel() for _, t in self.named_tensors())

    def to(self, device) -> "ModelParams":
        self.device = torch.device(device)
        for u in self.units.values():
            u.data = u.data.to(self.device)
            if u.grad is not None:
                u.grad = u.grad.to(self.device)
        return self

    def requires_grad_(self, flag: bool = True) -> "ModelParams":
        for u in self.units.values():
            u.data.requires_grad_(flag)
        return self

    def state_dict(self) -> dict[str, torch.Tensor]:
        return {name: t for name, t in self.named_tensors()}

    def load_state_dict(self, tensors: dict[str, torch.Tensor], strict: bool = True) -> None:
        missing = [n for n in self.hf_names() if n not in tensors]
        if strict and missing:
            raise KeyError(f"missing tensors: {missing[:4]}{'...' if len(missing) > 4 else ''}")
        with torch.no_grad():
            for name in self.hf_names():
                if name in tensors:
                    dst = self.tensor(name)
                    src = tensors[name]
                    if tuple(src.shape) != tuple(dst.shape):
                        raise ValueError(f"{name}: shape {tuple(src.shape)} != {tuple(dst.shape)}")
                    dst.copy_(src.to(dst.dtype))
