"""Shared builders for the CPU tests: a tiny word-level tokenizer directory and a tiny model directory."""
from __future__ import annotations

import json
from pathlib import Path

CHATML = (
    "{% for m in messages %}<|im_start|>{{ m['role'] }}\n"
    "{% if m['role'] == 'assistant' %}{% generation %}{{ m['content'] }}<|im_end|>{% endgeneration %}"
    "{% else %}{{ m['content'] }}<|im_end|>{% endif %}\n{% endfor %}"
)


def write_tokenizer(directory: Path, extra_tokens: list[str] | None = None, chat_template: str | None = CHATML) -> Path:
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers

    directory.mkdir(parents=True, exist_ok=True)
    words = ["<pad>", "<unk>", "</s>", "<|im_start|>", "<|im_end|>", "[MASK]", "\n", "user", "assistant", "system"]
    words += [f"w{i}" for i in range(40)] + [f"<|image_{i}|>" for i in range(16)] + (extra_tokens or [])
    vocab = {w: i for i, w in enumerate(words)}
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split(Regex(r"<\|[a-z_0-9]+\|>|\[MASK\]|\n|[^\s<\[]+"), behavior="isolated")
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(r"<\|[a-z_0-9]+\|>|\[MASK\]|\n"), behavior="isolated"),
        pre_tokenizers.Split(Regex(r"[ \t]+"), behavior="removed"),
    ])
    tok.decoder = decoders.Fuse()          # decode by plain concatenation, like a byte-level BPE would
    tok.save(str(directory / "tokenizer.json"))
    cfg = {"pad_token": "<pad>", "eos_token": "</s>", "unk_token": "<unk>"}
    if chat_template is not None:
        cfg["chat_template"] = chat_template
    (directory / "tokenizer_config.json").write_text(json.dumps(cfg))
    return directory


def write_model_dir(directory: Path, vocab_size: int = 80, **overrides) -> Path:
    write_tokenizer(directory)
    cfg = dict(model_type="llama", vocab_size=vocab_size, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
               num_attention_heads=2, num_key_value_heads=1, head_dim=64, rms_norm_eps=1e-6, rope_theta=10000.0,
               pad_token_id=0, eos_token_id=2, torch_dtype="float32")
    cfg.update(overrides)
    (directory / "config.json").write_text(json.dumps(cfg))
    return directory
