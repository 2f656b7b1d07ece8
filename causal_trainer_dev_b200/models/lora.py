"""LoRA adapters on the seven decoder projections.

Math and formats follow the reference (src/causal_trainer/modeling/lora.py): an adapted
projection computes ``x @ W^T + (x @ A) @ B`` with **no alpha multiplier** (``:1-9``), ``A`` is
``[in, r]`` He-uniform on ``[-sqrt(6/in), sqrt(6/in)]`` and ``B`` is ``[r, out]`` zeros, so step 0
is the base model (``:109-154``).  Export either merges ``W += (A @ B)^T`` leaf by leaf
(``:279-356``) or writes a PEFT adapter: keys ``base_model.model.model.layers.N.<module>.
lora_A.weight`` (= ``A^T``) / ``lora_B.weight`` (= ``B^T``) and ``lora_alpha = r`` so PEFT's
``alpha/r`` scaling reproduces the same model (``:428-487``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Iterator

import torch

from .config import ModelConfig

LORA_PROJECTIONS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
_MODULE_OF = {"q_proj": "self_attn", "k_proj": "self_attn", "v_proj": "self_attn", "o_proj": "self_attn",
              "gate_proj": "mlp", "up_proj": "mlp", "down_proj": "mlp"}


def projection_dimensions(cfg: ModelConfig) -> dict[str, tuple[int, int]]:
    """``name -> (in_features, out_features)``."""
    d, f, q, kv = cfg.hidden_size, cfg.intermediate_size, cfg.query_width, cfg.key_value_width
    return {"q_proj": (d, q), "k_proj": (d, kv), "v_proj": (d, kv), "o_proj": (q, d), "gate_proj": (d, f),
            "up_proj": (d, f), "down_proj": (f, d)}


def validate_rank(rank: Any) -> int:
    if isinstance(rank, bool) or not isinstance(rank, int) or rank <= 0:
        raise ValueError("lora_rank must be a positive integer")
    return rank


def lora_parameter_shapes(cfg: ModelConfig, rank: int) -> dict[str, tuple[int, ...]]:
    """``"layers/<i>/<projection>/lora_a|lora_b" -> shape`` for every adapter leaf, in the stable
    order of :meth:`LoraState.named_tensors` (A is ``[in, r]``, B is ``[r, out]``)."""
    rank = validate_rank(rank)
    dims = projection_dimensions(cfg)
    out: dict[str, tuple[int, ...]] = {}
    for layer in range(cfg.num_hidden_layers):
        for name in LORA_PROJECTIONS:
            fin, fout = dims[name]
            out[f"layers/{layer}/{name}/lora_a"] = (fin, rank)
            out[f"layers/{layer}/{name}/lora_b"] = (rank, fout)
    return out


def _check_pair(a: torch.Tensor, b: torch.Tensor) -> None:
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[0]:
        raise ValueError(f"adapter shapes {tuple(a.shape)} and {tuple(b.shape)} do not form a rank-r product")


def lora_linear_delta(x: torch.Tensor, a: torch.Tensor, b: torch.Tensor,
                      compute_dtype: torch.dtype | None = None) -> torch.Tensor:
    """``(x @ A) @ B`` without forming ``A @ B`` and without an alpha multiplier
    (src/causal_trainer/modeling/lora.py:218-242)."""
    _check_pair(a, b)
    if x.shape[-1] != a.shape[0]:
        raise ValueError(f"input width {x.shape[-1]} does not match lora_a input width {a.shape[0]}")
    dtype = x.dtype if compute_dtype is None else compute_dtype
    return (x.to(dtype) @ a.to(dtype)) @ b.to(dtype)


def merge_lora_kernel(kernel: torch.Tensor, a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``kernel + A @ B`` for a kernel in ``[in, out]`` layout, product accumulated in fp32, result
    in the kernel's dtype (src/causal_trainer/modeling/lora.py:279-295)."""
    _check_pair(a, b)
    if kernel.dim() != 2:
        raise ValueError(f"a merged projection kernel must be rank two, got shape {tuple(kernel.shape)}")
    if tuple(kernel.shape) != (a.shape[0], b.shape[1]):
        raise ValueError(f"kernel shape {tuple(kernel.shape)} is incompatible with adapter shapes "
                         f"{tuple(a.shape)} and {tuple(b.shape)}")
    return (kernel.float() + a.float() @ b.float()).to(kernel.dtype)


def lora_parameter_to_peft_key(path: str) -> tuple[str, bool]:
    """``(PEFT tensor name, transposed)`` of an adapter leaf path as :meth:`LoraState.named_tensors`
    spells it (src/causal_trainer/modeling/lora.py:428-456): ``lora_A`` is ``A^T`` and ``lora_B`` is
    ``B^T``; the embedding and LM-head copies are stored in the Hugging Face orientation already."""
    parts = [p for p in path.split("/") if p]
    if parts[:1] == ["adapters"]:
        parts = parts[1:]
    if parts == ["embed_tokens", "embedding"]:
        return "base_model.model.model.embed_tokens.weight", False
    if parts == ["lm_head", "kernel"]:
        return "base_model.model.lm_head.weight", False
    if len(parts) == 4 and parts[0] == "layers" and parts[1].isdigit() and parts[2] in LORA_PROJECTIONS \
            and parts[3] in ("lora_a", "lora_b"):
        leaf = "lora_A" if parts[3] == "lora_a" else "lora_B"
        return f"base_model.model.model.layers.{int(parts[1])}.{_MODULE_OF[parts[2]]}.{parts[2]}.{leaf}.weight", True
    raise KeyError(f"unknown adapter parameter path {path!r}")


@dataclass
class LoraState:
    """All adapter tensors of a model plus, optionally, trainable copies of embedding and head."""

    config: ModelConfig
    rank: int
    a: dict[tuple[int, str], torch.Tensor] = field(default_factory=dict)
    b: dict[tuple[int, str], torch.Tensor] = field(default_factory=dict)
    train_embed_and_lm_head: bool = False
    embed: torch.Tensor | None = None
    lm_head: torch.Tensor | None = None

    @classmethod
    def init(cls, cfg: ModelConfig, rank: int, *, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
             device: str | torch.device = "cpu", train_embed_and_lm_head: bool = False, base=None) -> "LoraState":
        rank = validate_rank(rank)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self = cls(cfg, rank, train_embed_and_lm_head=train_embed_and_lm_head)
        dims = projection_dimensions(cfg)
        for layer in range(cfg.num_hidden_layers):
            for name in LORA_PROJECTIONS:
                fin, fout = dims[name]
                limit = math.sqrt(6.0 / fin)
                a = (torch.rand((fin, rank), generator=gen, dtype=torch.float32) * 2 - 1) * limit
                self.a[(layer, name)] = a.to(dtype).to(device).requires_grad_()
                self.b[(layer, name)] = torch.zeros((rank, fout), dtype=dtype, device=device).requires_grad_()
        if train_embed_and_lm_head:
            if base is None:
                raise ValueError("training the embedding and LM head next to LoRA needs the base parameters")
            self.embed = base.tensor("model.embed_tokens.weight").detach().clone().requires_grad_()
            self.lm_head = base.tensor("lm_head.weight").detach().clone().requires_grad_()
        return self

    def pair(self, layer: int, name: str) -> tuple[torch.Tensor, torch.Tensor]:
        return self.a[(layer, name)], self.b[(layer, name)]

    def named_tensors(self) -> Iterator[tuple[str, torch.Tensor]]:
        """Adapter leaves in a stable order (layer, projection, A then B), then embedding / head."""
        for layer in range(self.config.num_hidden_layers):
            for name in LORA_PROJECTIONS:
                yield f"layers/{layer}/{name}/lora_a", self.a[(layer, name)]
                yield f"layers/{layer}/{name}/lora_b", self.b[(layer, name)]
        if self.train_embed_and_lm_head:
            yield "embed_tokens/embedding", self.embed
            yield "lm_head/kernel", self.lm_head

    def trainable(self) -> list[tuple[str, torch.Tensor]]:
        return list(self.named_tensors())

    # ---- export ----
    def pair_of_tensor(self, hf_name: str):
        """``(A, B)`` of the adapter on projection weight ``hf_name``, else ``None``."""
        parts = hf_name.split(".")
        if len(parts) == 6 and parts[0] == "model" and parts[1] == "layers" and parts[-1] == "weight" \
                and parts[4] in LORA_PROJECTIONS:
            return self.pair(int(parts[2]), parts[4])
        return None

    def merged_delta(self, hf_name: str) -> torch.Tensor | None:
        """``(A @ B)^T`` in HF ``[out,in]`` layout for a projection weight name, else ``None``."""
        parts = hf_name.split(".")
        if len(parts) == 6 and parts[0] == "model" and parts[1] == "layers" and parts[-1] == "weight" \
                and parts[4] in LORA_PROJECTIONS:
            a, b = self.pair(int(parts[2]), parts[4])
            return (a.detach().float() @ b.detach().float()).t()
        return None

    def export_transform(self):
        """``(name, tensor) -> tensor`` hook that merges adapters while a checkpoint streams out."""
        def transform(name: str, t: torch.Tensor) -> torch.Tensor:
            if self.train_embed_and_lm_head and name == "model.embed_tokens.weight":
                return self.embed.detach().to(t.dtype)
            if self.train_embed_and_lm_head and name == "lm_head.weight":
                return self.lm_head.detach().to(t.dtype)
            pair = self.pair_of_tensor(name)
            if pair is not None and t.is_cuda and t.dtype == torch.bfloat16:
                from ..ops.gemm import lora_merge      # rank-r update on the tcgen05 GEMM

                return lora_merge(t, pair[0].detach().to(t.device), pair[1].detach().to(t.device))
            delta = self.merged_delta(name)
            if delta is None:
                return t
            return (t.float() + delta.to(t.device)).to(t.dtype)
        return transform

    def peft_tensors(self) -> dict[str, torch.Tensor]:
        out: dict[str, torch.Tensor] = {}
        for layer in range(self.config.num_hidden_layers):
            for name in LORA_PROJECTIONS:
                prefix = f"base_model.model.model.layers.{layer}.{_MODULE_OF[name]}.{name}"
                a, b = self.pair(layer, name)
                out[f"{prefix}.lora_A.weight"] = a.detach().t().contiguous()
                out[f"{prefix}.lora_B.weight"] = b.detach().t().contiguous()
        if self.train_embed_and_lm_head:
            out["base_model.model.model.embed_tokens.weight"] = self.embed.detach()
            out["base_model.model.lm_head.weight"] = self.lm_head.detach()
        return out

    def load_peft_tensors(self, tensors: dict[str, torch.Tensor]) -> None:
        with torch.no_grad():
            for key, value in self.peft_tensors().items():
                if key not in tensors:
                    raise KeyError(f"adapter checkpoint is missing {key}")
            for layer in range(self.config.num_hidden_layers):
                for name in LORA_PROJECTIONS:
                    prefix = f"base_model.model.model.layers.{layer}.{_MODULE_OF[name]}.{name}"
                    a, b = self.pair(layer, name)
                    a.copy_(tensors[f"{prefix}.lora_A.weight"].t().to(a.dtype))
                    b.copy_(tensors[f"{prefix}.lora_B.weight"].t().to(b.dtype))
            if self.train_embed_and_lm_head:
                self.embed.copy_(tensors["base_model.model.model.embed_tokens.weight"].to(self.embed.dtype))
                self.lm_head.copy_(tensors["base_model.model.lm_head.weight"].to(self.lm_head.dtype))


def peft_adapter_config(base_model_name_or_path: str, rank: int, *, train_embed_and_lm_head: bool,
                        revision: str | None = None) -> dict[str, Any]:
    rank = validate_rank(rank)
    return {
        "base_model_name_or_path": str(base_model_name_or_path), "bias": "none", "fan_in_fan_out": False,
        "inference_mode": True, "init_lora_weights": True, "lora_alpha": rank, "lora_dropout": 0.0,
        "modules_to_save": ["embed_tokens", "lm_head"] if train_embed_and_lm_head else None, "peft_type": "LORA",
        "r": rank, "revision": revision, "target_modules": list(LORA_PROJECTIONS), "task_type": "CAUSAL_LM",
        "use_dora": False, "use_rslora": False,
    }
