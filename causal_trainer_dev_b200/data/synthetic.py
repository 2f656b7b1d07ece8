"""Synthetic corpora of the shapes the benchmarks name (no dataset or network needed).

``pretraining_rows`` draws documents with log-normal lengths, uniform token ids and an EOS
at each document end, then packs them with the production packer into fixed-length rows.
``chat_rows`` builds ChatML-like conversations with assistant-only loss weights,
``long_document_rows`` rows packed from a few long documents, and ``maskgit_rows`` conversations
whose assistant turns carry image-code grids, already passed through the mixed AR + MaskGIT rule
(``data/maskgit.py``) so that no tokenizer is needed.
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


def long_document_rows(num_rows: int, seq_len: int, vocab_size: int, *, docs_per_row: int = 4, min_len: int = 4096,
                       max_len: int = 12288, eos_token_id: int = 2, pad_token_id: int = 0, seed: int = 0
                       ) -> dict[str, np.ndarray]:
    """Rows of exactly ``seq_len`` tokens holding ``docs_per_row`` documents each: lengths uniform in
    ``[min_len, max_len]``, rescaled so that they fill the row, ids uniform, EOS last."""
    rng = np.random.default_rng(seed)
    out = {f: np.zeros((num_rows, seq_len), dtype=np.int32) for f in FIELDS_INT}
    for r in range(num_rows):
        lens = rng.integers(min_len, max_len + 1, size=docs_per_row).astype(np.float64)
        lens = np.maximum(1, np.floor(lens * seq_len / lens.sum())).astype(np.int64)
        lens[-1] += seq_len - lens.sum()
        pos = 0
        for d, n in enumerate(lens):
            ids = rng.integers(3, vocab_size, size=int(n))
            ids[-1] = eos_token_id
            out["input_ids"][r, pos:pos + n] = ids
            out["segment_ids"][r, pos:pos + n] = d + 1
            out["position_ids"][r, pos:pos + n] = np.arange(n)
            pos += int(n)
        out["attention_mask"][r] = 1
    return out


def maskgit_rows(num_rows: int, seq_len: int, *, text_vocab: int, code_base: int, num_codes: int, mask_id: int,
                 im_start: int, im_end: int, newline_id: int, pad_token_id: int, probability: float = 0.5,
                 sides: tuple[int, ...] = (16, 32), seed: int = 0) -> dict[str, np.ndarray]:
    """Packed conversations whose assistant turns hold one or two ``h x w`` grids of image codes
    (one newline token after every grid row), with the mixed objective already applied: each grid
    is MaskGIT with ``probability`` (cosine-sampled mask ratio, at least one code masked,
    ``attention_end`` = last grid index on the grid, same-position targets on the masked codes, no
    next-token edge into, inside or out of the grid); everything else is next-token prediction on
    the assistant spans."""
    rng = np.random.default_rng(seed)
    convs = []
    budget = (num_rows + 2) * seq_len
    while budget > 0:
        ids: list[int] = []
        w: list[float] = []
        grids: list[tuple[int, int, int]] = []          # (first index, side h, side w)
        for turn in range(2):
            assistant = turn == 1
            ids += [im_start, 5 if assistant else 4]
            w += [0.0, 0.0]
            n = int(np.clip(rng.lognormal(np.log(60), 0.6), 4, 400))
            ids += rng.integers(3, text_vocab, size=n).tolist()
            w += [1.0 if assistant else 0.0] * n
            if assistant:
                for _ in range(int(rng.integers(1, 3))):
                    side = int(rng.choice(sides))
                    grids.append((len(ids), side, side))
                    for _row in range(side):
                        ids += (code_base + rng.integers(0, num_codes, size=side)).tolist() + [newline_id]
                        w += [1.0] * (side + 1)
                    m = int(np.clip(rng.lognormal(np.log(30), 0.6), 2, 200))
                    ids += rng.integers(3, text_vocab, size=m).tolist()
                    w += [1.0] * m
            ids.append(im_end)
            w.append(1.0 if assistant else 0.0)
        if len(ids) > seq_len:
            continue
        convs.append({"input_ids": ids, "loss_weights": w, "_grids": grids})
        budget -= len(ids)
    # pack (keeping track of where every conversation lands) with a first-fit over the production order
    rows_ids = np.full((num_rows, seq_len), pad_token_id, dtype=np.int32)
    seg = np.zeros((num_rows, seq_len), dtype=np.int32)
    posi = np.zeros((num_rows, seq_len), dtype=np.int32)
    wts = np.zeros((num_rows, seq_len), dtype=np.float32)
    fill = np.zeros(num_rows, dtype=np.int64)
    count = np.zeros(num_rows, dtype=np.int64)
    placed: list[tuple[int, int, list]] = []
    for c in convs:
        n = len(c["input_ids"])
        fits = np.flatnonzero(fill + n <= seq_len)
        if not len(fits):
            continue
        r = int(fits[0])
        a = int(fill[r])
        rows_ids[r, a:a + n] = c["input_ids"]
        wts[r, a:a + n] = c["loss_weights"]
        count[r] += 1
        seg[r, a:a + n] = count[r]
        posi[r, a:a + n] = np.arange(n)
        placed.append((r, a, c["_grids"]))
        fill[r] += n
    attended = seg != 0
    same = attended[:, :-1] & attended[:, 1:] & (seg[:, :-1] == seg[:, 1:])
    targets = np.concatenate([rows_ids[:, 1:], np.zeros((num_rows, 1), np.int32)], axis=1)
    pred_w = np.concatenate([wts[:, 1:] * same, np.zeros((num_rows, 1), np.float32)], axis=1).astype(np.float32)
    tokens = rows_ids.copy()
    att_end = np.tile(np.arange(seq_len, dtype=np.int32), (num_rows, 1))
    for r, a, grids in placed:
        for first, h, wd in grids:
            if rng.random() >= probability:
                continue
            lo, hi = a + first, a + first + h * (wd + 1) - 1        # the last newline stays outside the grid
            codes = np.asarray([lo + y * (wd + 1) + x for y in range(h) for x in range(wd)])
            k = max(1, int(np.ceil(len(codes) * np.cos(0.5 * np.pi * rng.random()))))
            masked = rng.choice(codes, size=k, replace=False)
            att_end[r, lo:hi] = hi - 1
            pred_w[r, max(lo - 1, 0):hi] = 0.0
            tokens[r, masked] = mask_id
            targets[r, masked] = rows_ids[r, masked]
            pred_w[r, masked] = wts[r, masked]
    return {"input_ids": tokens, "attention_mask": attended.astype(np.int32), "segment_ids": seg, "position_ids": posi,
            "loss_weights": wts, "attention_end": att_end, "prediction_targets": targets, "prediction_weights": pred_w}
