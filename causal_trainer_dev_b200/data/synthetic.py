"""Synthetic corpora of the shapes the benchmarks name (no dataset or network needed).

``pretraining_rows`` draws documents with log-normal lengths, uniform token ids and an EOS
at each document end, then packs them with the production packer into fixed-length rows.
``chat_rows`` builds ChatML-like conversations with assistant-only loss weights.
"""
from __future__ import annotations

import numpy as np

from .packing import pack_examples

FIELDS_INT = ("input_ids", "attention_mask", "segment_ids", "position_ids")


def _rows_to_arrays(rows: list[dict], with_weights: bool) -> dict[str, np.ndarray]:
    out = {f: np.asarray([r[f] for r in rows], dtype=np.int32) for f in FIELDS_INT}
    if with_weights:
        out["loss_weights"] = np.asarray([r["loss_weights"] for r in rows], dtype=np.float32)
    return out


def pretraining_rows(num_rows: int, seq_len: int, vocab_size: int, *, eos_token_id: int, pad_token_id: int,
                     median_len: float = 600.0, sigma: float = 1.0, min_len: int = 32, seed: int = 0) -> dict[str, np.ndarray]:
    """``num_rows`` packed rows: document lengths log-normal (median ``median_len``) clipped to
    [min_len, seq_len], ids uniform in [3, vocab), EOS last."""
    rng = np.random.default_rng(seed)
    rows: list[dict] = []
    while len(rows) < num_rows:
        docs = []
        budget = (num_rows - len(rows) + 2) * seq_len
        while budget > 0:
            n = int(np.clip(rng.lognormal(np.log(median_len), sigma), min_len, seq_len))
            ids = rng.integers(3, vocab_size, size=n, dtype=np.int64)
            ids[-1] = eos_token_id
            docs.append({"input_ids": ids.tolist()})
            budget -= n
        rows.extend(pack_examples(docs, max_length=seq_len, pad_token_id=pad_token_id, packing_batch_size=1000))
    return _rows_to_arrays(rows[:num_rows], with_weights=False)


def chat_rows(num_rows: int, seq_len: int, vocab_size: int, *, im_start: int, im_end: int, pad_token_id: int,
              median_turn: float = 200.0, seed: int = 0) -> dict[str, np.ndarray]:
    """Packed ChatML conversations of 2-6 alternating turns; loss weight 1 only on assistant
    spans including the closing ``im_end``."""
    rng = np.random.default_rng(seed)
    rows: list[dict] = []
    while len(rows) < num_rows:
        convs = []
        budget = (num_rows - len(rows) + 2) * seq_len
        while budget > 0:
            ids: list[int] = []
            w: list[float] = []
            for turn in range(int(rng.integers(2, 7))):
                n = int(np.clip(rng.lognormal(np.log(median_turn), 0.8), 4, seq_len // 4))
                body = rng.integers(3, min(vocab_size, im_start), size=n).tolist()
                assistant = turn % 2 == 1
                ids += [im_start, 5 if assistant else 4] + body + [im_end]
                w += [0.0, 0.0] + ([1.0] * n + [1.0] if assistant else [0.0] * (n + 1))
            ids, w = ids[:seq_len], w[:seq_len]
            convs.append({"input_ids": ids, "loss_weights": w})
            budget -= len(ids)
        rows.extend(pack_examples(convs, max_length=seq_len, pad_token_id=pad_token_id, packing_batch_size=1000))
    return _rows_to_arrays(rows[:num_rows], with_weights=True)
