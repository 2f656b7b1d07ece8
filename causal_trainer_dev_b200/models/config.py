"""Decoder architecture description.

The reference trainer accepts exactly one architecture (40 layers, one KV head,
head_dim 128, partial rotary 0.5; src/causal_trainer/modeling/config.py:35-145 and the
gate at src/causal_trainer/training/runner.py:190-216).  This framework keeps the same
field names and the same read-side normalisation of Hugging Face ``config.json``
(v4 ``torch_dtype``/``rope_scaling`` and v5 ``dtype``/``rope_parameters`` spellings) but
admits the whole Llama family: any GQA ratio, head_dim 64 or 128, full or partial
rotary, either RoPE pairing and optional QKV bias.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, fields
from pathlib import Path
from typing import Any, Mapping, Literal

ROPE_STYLES = ("gpt-j", "gpt-neox")
RopeStyle = Literal["gpt-j", "gpt-neox"]     # adjacent-pair or half-split rotary channel pairing

# model_type -> (rope pairing, QKV bias) used when config.json does not say.
_FAMILY_DEFAULTS = {
    "llama": ("gpt-neox", False),
    "mistral": ("gpt-neox", False),
    "qwen2": ("gpt-neox", True),
    "qwen3": ("gpt-neox", False),
    "glm": ("gpt-j", True),
    "glm4": ("gpt-j", True),
}
# A config of any other model type follows the reference, whose single architecture pairs
# adjacent channels (src/causal_trainer/modeling/config.py: rope_style defaults to "gpt-j").
_OTHER_FAMILY = ("gpt-j", False)


def _is_pos_int(value: Any) -> bool:
    return isinstance(value, int) and not isinstance(value, bool) and value > 0


@dataclass(frozen=True)
class ModelConfig:
    vocab_size: int = 32000
    hidden_size: int = 4096
    intermediate_size: int = 11008
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 32
    head_dim: int = 128
    hidden_act: str = "silu"
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    partial_rotary_factor: float = 1.0
    rope_style: str = "gpt-neox"
    rope_scaling: Mapping[str, Any] | None = None
    attention_bias: bool = False
    attention_dropout: float = 0.0
    initializer_range: float = 0.02
    max_position_embeddings: int = 2_097_152
    pad_token_id: int = 0
    eos_token_id: int | tuple[int, ...] = 2
    tie_word_embeddings: bool = False
    torch_dtype: str | None = "bfloat16"
    use_cache: bool = True
    sliding_window: int | None = None
    use_sliding_window: bool = False
    model_type: str = "llama"

    def __post_init__(self) -> None:
        if isinstance(self.eos_token_id, list):
            object.__setattr__(self, "eos_token_id", tuple(self.eos_token_id))
        for name in (
            "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "max_position_embeddings",
        ):
            if not _is_pos_int(getattr(self, name)):
                raise ValueError(f"{name} must be a positive integer, got {getattr(self, name)!r}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim not in (64, 128):
            raise ValueError("head_dim must be 64 or 128 (the sizes the sm_100a attention kernels are built for)")
        if isinstance(self.pad_token_id, bool) or not isinstance(self.pad_token_id, int):
            raise ValueError("pad_token_id must be an integer")
        if not 0 <= self.pad_token_id < self.vocab_size:
            raise ValueError("pad_token_id must index the embedding vocabulary")
        eos = self.eos_token_id if isinstance(self.eos_token_id, tuple) else (self.eos_token_id,)
        if not eos or any(isinstance(t, bool) or not isinstance(t, int) or not 0 <= t < self.vocab_size for t in eos):
            raise ValueError("eos_token_id must contain valid vocabulary indices")
        if not 0.0 < self.partial_rotary_factor <= 1.0:
            raise ValueError("partial_rotary_factor must be in (0, 1]")
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError("int(head_dim * partial_rotary_factor) must be positive and even")
        if self.hidden_act != "silu":
            raise ValueError("only the silu gated MLP is supported")
        if not 0.0 <= self.attention_dropout < 1.0:
            raise ValueError("attention_dropout must be in [0, 1)")
        if self.initializer_range <= 0.0 or self.rms_norm_eps <= 0.0 or self.rope_theta <= 0.0:
            raise ValueError("initializer_range, rms_norm_eps and rope_theta must be positive")
        if self.rope_style not in ROPE_STYLES:
            raise ValueError("rope_style must be 'gpt-j' or 'gpt-neox'")
        if self.rope_scaling is not None:
            raise ValueError("scaled RoPE variants are not supported")
        if self.use_sliding_window or self.sliding_window is not None:
            raise ValueError("sliding-window attention is not supported")
        if self.tie_word_embeddings:
            raise ValueError("tied input/output embeddings are not supported (the head is a separate tensor)")

    # ---- derived sizes (src/causal_trainer/modeling/config.py:129-145) ----
    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def query_width(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def key_value_width(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def key_value_groups(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    def parameter_count(self) -> int:
        d, f, q, kv = self.hidden_size, self.intermediate_size, self.query_width, self.key_value_width
        per_layer = d * q + 2 * d * kv + q * d + 3 * d * f + 2 * d
        if self.attention_bias:
            per_layer += q + 2 * kv
        return self.num_hidden_layers * per_layer + 2 * self.vocab_size * d + d

    def flops_per_token(self, seq_len: int, causal: bool = True) -> float:
        """Model FLOPs per trained token (forward + backward, no recompute)."""
        d, f, q, kv = self.hidden_size, self.intermediate_size, self.query_width, self.key_value_width
        matmul_params = self.num_hidden_layers * (d * q + 2 * d * kv + q * d + 3 * d * f) + self.vocab_size * d
        attn = self.num_hidden_layers * 2 * 2 * seq_len * q * (0.5 if causal else 1.0)  # QK^T and PV, forward
        return 6.0 * matmul_params + 3.0 * attn

    # ---- I/O ----
    @classmethod
    def from_dict(cls, values: Mapping[str, Any]) -> "ModelConfig":
        norm = dict(values)
        if "dtype" in norm:
            if norm["dtype"] is not None:
                norm["torch_dtype"] = norm["dtype"]
            elif "torch_dtype" not in norm:
                norm["torch_dtype"] = None
        family = _FAMILY_DEFAULTS.get(str(norm.get("model_type", "llama")), _OTHER_FAMILY)
        norm.setdefault("rope_style", family[0])
        norm.setdefault("attention_bias", family[1])
        if "head_dim" not in norm or norm["head_dim"] is None:
            if "hidden_size" in norm and "num_attention_heads" in norm:
                norm["head_dim"] = int(norm["hidden_size"]) // int(norm["num_attention_heads"])
        if norm.get("num_key_value_heads") is None and "num_attention_heads" in norm:
            norm["num_key_value_heads"] = norm["num_attention_heads"]
        if norm.get("pad_token_id") is None:
            norm["pad_token_id"] = 0
        rope_parameters = norm.get("rope_parameters")
        rope_scaling = norm.get("rope_scaling")
        if rope_parameters is not None and not isinstance(rope_parameters, Mapping):
            raise ValueError("rope_parameters must be a mapping")
        effective: Mapping[str, Any] | None = None
        if isinstance(rope_scaling, Mapping) and rope_scaling:
            effective = rope_scaling
        elif isinstance(rope_parameters, Mapping):
            effective = rope_parameters
        elif isinstance(rope_scaling, Mapping):
            effective = rope_scaling
        if effective is not None:
            rope_type = effective.get("rope_type", effective.get("type", "default"))
            if rope_type != "default":
                raise ValueError(f"only unscaled default RoPE is supported, got rope_type={rope_type!r}")
            norm["rope_theta"] = effective.get("rope_theta", norm.get("rope_theta", 10_000.0))
            norm["partial_rotary_factor"] = effective.get(
                "partial_rotary_factor", norm.get("partial_rotary_factor", 1.0)
            )
            norm["rope_scaling"] = None
        accepted = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in norm.items() if k in accepted})

    @classmethod
    def from_json_file(cls, path: str | Path) -> "ModelConfig":
        values = json.loads(Path(path).read_text(encoding="utf-8"))
        if not isinstance(values, dict):
            raise ValueError("model config JSON must contain an object")
        return cls.from_dict(values)

    def to_dict(self) -> dict[str, Any]:
        values = asdict(self)
        if isinstance(values["eos_token_id"], tuple):
            values["eos_token_id"] = list(values["eos_token_id"])
        return values


def validate_splash_block_size(sequence_length: int, requested: int, name: str) -> int:
    """Block-size rule kept for ``--attn_mechanism splash`` / ``--block_size_q/k``.

    The effective tile is ``min(requested, S)``, must be a multiple of 128 and must divide
    the sequence (src/causal_trainer/modeling/config.py:13-31).  The flash kernel uses it
    as a tile hint only.
    """
    if not _is_pos_int(sequence_length):
        raise ValueError(f"sequence_length must be a positive integer, got {sequence_length!r}")
    if not _is_pos_int(requested):
        raise ValueError(f"{name} must be a positive integer, got {requested!r}")
    effective = min(requested, sequence_length)
    if effective % 128:
        raise ValueError(f"effective {name}={effective} must be a multiple of 128")
    if sequence_length % effective:
        raise ValueError(f"sequence length {sequence_length} must be divisible by effective {name}={effective}")
    return effective


# Named shapes used by the benchmarks and tests.
PRESETS: dict[str, dict[str, Any]] = {
    "tiny": dict(
        vocab_size=32000, hidden_size=256, intermediate_size=688, num_hidden_layers=2, num_attention_heads=4,
        num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0, eos_token_id=2, pad_token_id=0,
    ),
    "llama3-8b": dict(
        vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, num_attention_heads=32,
        num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=500000.0, eos_token_id=128001,
        pad_token_id=128002,
    ),
    "qwen2.5-7b": dict(
        vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
        num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, attention_bias=True,
        eos_token_id=151645, pad_token_id=151643, model_type="qwen2",
    ),
    "qwen2.5-1.5b-image": dict(
        vocab_size=151936 + 16384 + 64, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28,
        num_attention_heads=12, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6,
        attention_bias=True, eos_token_id=151645, pad_token_id=151643, model_type="qwen2",
    ),
}


def preset(name: str, **overrides: Any) -> ModelConfig:
    return ModelConfig(**{**PRESETS[name], **overrides})
