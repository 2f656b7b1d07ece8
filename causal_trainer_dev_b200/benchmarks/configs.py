"""Named benchmark configurations (model shape, sequence length, batch, parallel layout, data).

``bench.py --config <name>`` runs one of them through ``api.Trainer``:

* ``llama8b-pretrain``          Llama-3-8B shape, seq 4096, 32 rows, FSDP over all GPUs (headline)
* ``qwen7b-sft-fsdp4tp2``       Qwen2.5-7B shape, seq 8192, assistant-only ChatML, FSDP x TP 2
* ``llama8b-moba32k-fsdp2tp4``  Llama-3-8B shape, rows of 32768 tokens from 4 documents, MoBA block
                                4096 / top-3 + current, FSDP x TP 4 (``--attention dense`` for the
                                dense segment-masked comparison on the same rows)
* ``llama8b-moba32k-one-document`` / ``llama8b-moba128k-one-document``  the same model and MoBA settings on
                                rows that are one document (8 / 32 blocks: the router has something to drop)
* ``qwen1.5b-maskgit-fsdp8``    1.5B shape with image codes, seq 4096, mixed AR + MaskGIT, FSDP

The tensor-parallel degree is capped by the number of GPUs the run has (tp = min(named tp, N)), so
every configuration also runs on fewer GPUs; the layout actually used is reported in the result.
Data is synthetic (``data/synthetic.py``), weights are random N(0, 0.02).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import numpy as np

from ..data import synthetic
from ..models.config import ModelConfig, preset


@dataclass(frozen=True)
class BenchConfig:
    name: str
    metric: str
    model: str
    seq_len: int
    global_batch: int
    micro_batch: int
    tp: int                                   # tensor-parallel degree on 8 GPUs
    make_rows: Callable[[ModelConfig, int, int, int], dict[str, np.ndarray]]   # (cfg, rows, seq, seed) -> arrays
    moba: tuple[int, int] | None = None       # (block, top_k incl. the current block)
    data: str = ""


def _eos(cfg: ModelConfig) -> int:
    return int(cfg.eos_token_id if isinstance(cfg.eos_token_id, int) else cfg.eos_token_id[0])


def _pretrain(cfg, rows, seq, seed):
    return synthetic.pretraining_rows(rows, seq, cfg.vocab_size, eos_token_id=_eos(cfg), pad_token_id=cfg.pad_token_id,
                                      median_len=600.0, sigma=1.0, min_len=32, seed=seed)


def _chat(cfg, rows, seq, seed):
    # Qwen ChatML delimiters: <|im_start|> = 151644, <|im_end|> = 151645
    return synthetic.chat_rows(rows, seq, cfg.vocab_size, im_start=151644, im_end=151645, pad_token_id=cfg.pad_token_id,
                               median_turn=200.0, seed=seed)


def _long(cfg, rows, seq, seed):
    return synthetic.long_document_rows(rows, seq, cfg.vocab_size, docs_per_row=4, min_len=seq // 8, max_len=3 * seq // 8,
                                        eos_token_id=_eos(cfg), pad_token_id=cfg.pad_token_id, seed=seed)


def _one_document(cfg, rows, seq, seed):
    return synthetic.long_document_rows(rows, seq, cfg.vocab_size, docs_per_row=1, min_len=seq, max_len=seq,
                                        eos_token_id=_eos(cfg), pad_token_id=cfg.pad_token_id, seed=seed)


def _maskgit(cfg, rows, seq, seed):
    return synthetic.maskgit_rows(rows, seq, text_vocab=151000, code_base=151936, num_codes=16384,
                                  mask_id=151936 + 16384, im_start=151644, im_end=151645, newline_id=198,
                                  pad_token_id=cfg.pad_token_id, probability=0.5, seed=seed)


CONFIGS: dict[str, BenchConfig] = {c.name: c for c in (
    BenchConfig("llama8b-pretrain", "tokens/s Llama-3-8B-shape seq4096 FSDP bf16", "llama3-8b", 4096, 32, 4, 1, _pretrain,
                data="packed log-normal documents (median 600), uniform token ids"),
    BenchConfig("qwen7b-sft-fsdp4tp2", "tokens/s Qwen2.5-7B-shape seq8192 assistant-only SFT FSDPxTP2 bf16", "qwen2.5-7b",
                8192, 16, 2, 2, _chat, data="packed ChatML conversations of 2-6 turns, loss on assistant spans only"),
    BenchConfig("llama8b-moba32k-fsdp2tp4", "tokens/s Llama-3-8B-shape 32768-token rows MoBA block4096 top3+current "
                "FSDPxTP4 bf16", "llama3-8b", 32768, 2, 1, 4, _long, moba=(4096, 4),
                data="rows of 32768 tokens packed from 4 documents of 4096-12288 tokens"),
    BenchConfig("llama8b-moba32k-one-document", "tokens/s Llama-3-8B-shape 32768-token single-document rows MoBA "
                "block4096 top3+current FSDPxTP4 bf16", "llama3-8b", 32768, 2, 1, 4, _one_document, moba=(4096, 4),
                data="rows of one 32768-token document each"),
    BenchConfig("llama8b-moba128k-one-document", "tokens/s Llama-3-8B-shape 131072-token single-document rows MoBA "
                "block4096 top3+current FSDPxTP4 bf16", "llama3-8b", 131072, 2, 1, 4, _one_document, moba=(4096, 4),
                data="rows of one 131072-token document each"),
    BenchConfig("qwen1.5b-maskgit-fsdp8", "tokens/s 1.5B-shape seq4096 mixed AR+MaskGIT FSDP bf16", "qwen2.5-1.5b-image",
                4096, 64, 8, 1, _maskgit, data="conversations with 1-2 image-code grids (16x16 / 32x32) per assistant "
                "turn, maskgit_probability 0.5, cosine mask ratio"),
)}
DEFAULT = "llama8b-pretrain"


def executed_attention_flops_per_token(cfg: ModelConfig, arrays: dict[str, np.ndarray]) -> float:
    """Attention FLOPs (forward + backward, QK^T and PV) the segment-isolated rows actually need,
    per token: a query attends to the keys of its own document up to ``max(i, attention_end[i])``.
    The nominal ``ModelConfig.flops_per_token`` charges full-row causal attention instead."""
    seg = arrays["segment_ids"]
    rows, s = seg.shape
    idx = np.arange(s)[None, :]
    change = np.ones((rows, s), dtype=bool)
    change[:, 1:] = seg[:, 1:] != seg[:, :-1]
    start = np.maximum.accumulate(np.where(change, idx, 0), axis=1)
    lim = idx if "attention_end" not in arrays else np.maximum(idx, arrays["attention_end"])
    keys = np.where(seg != 0, lim - start + 1, 0).astype(np.float64)
    per_token_keys = keys.sum() / (rows * s)
    forward = cfg.num_hidden_layers * 2 * 2 * per_token_keys * cfg.query_width
    return 3.0 * forward


def executed_flops_per_token(cfg: ModelConfig, arrays: dict[str, np.ndarray], seq_len: int) -> float:
    nominal = cfg.flops_per_token(seq_len)
    nominal_attention = 3.0 * cfg.num_hidden_layers * 2 * 2 * seq_len * cfg.query_width * 0.5
    return nominal - nominal_attention + executed_attention_flops_per_token(cfg, arrays)


def model_of(config: BenchConfig, **overrides) -> ModelConfig:
    return preset(config.model, **overrides)
