"""Mixed autoregressive + MaskGIT batches for ChatML image responses (host side).

Applied to host batches after all other preprocessing; prepared artifacts are unchanged.
For every complete, supervised assistant image grid (rows of ``<|image_i|>`` code tokens
joined by single newlines) a coin with probability ``p`` decides whether the grid is trained
as MaskGIT this step.  A selected grid gets:

* ``ceil(n * cos(pi/2 * u))`` (at least one) of its ``n`` codes replaced by ``[MASK]``;
* ``attention_end = last index of the grid`` on all its positions, which the attention
  kernels turn into block-local bidirectional attention with a causal prefix;
* same-position reconstruction targets on the masked codes, and every next-token edge into,
  inside and out of the grid removed.

Everything else stays next-token prediction.  All randomness is a pure function of
``(seed, absolute optimizer step)`` and the draw order is fixed (selection, ratio, choice), so
a resumed run sees the same masks (src/causal_trainer/data/maskgit.py:20-135).
"""
from __future__ import annotations

import math
import re
from typing import Iterator, Mapping

import numpy as np

_IMAGE_TOKEN = re.compile(r"<\|image_[0-9]+\|>\Z")
_REQUIRED = ("[MASK]", "<|im_start|>", "<|im_end|>")


class MaskGITBatchTransform:
    def __init__(self, tokenizer, *, probability: float, seed: int):
        if not math.isfinite(probability) or not 0.0 <= probability <= 1.0:
            raise ValueError("maskgit_probability must be between 0 and 1")
        self.probability, self.seed, self.tokenizer = probability, seed, tokenizer
        vocab = tokenizer.get_vocab()
        for tok in _REQUIRED:
            if tok not in vocab or tokenizer(tok)["input_ids"] != [vocab[tok]]:
                raise ValueError(f"MaskGIT requires {tok!r} to encode as one token")
        self.mask_id, self.start_id, self.end_id = (vocab[t] for t in _REQUIRED)
        image_ids = [i for t, i in vocab.items() if _IMAGE_TOKEN.fullmatch(t)]
        if not image_ids:
            raise ValueError("MaskGIT requires <|image_i|> tokens in the tokenizer vocabulary")
        top = max(max(vocab.values()), getattr(tokenizer, "pad_token_id", None) or 0)
        self.is_image = np.zeros(top + 1, dtype=bool)
        self.is_image[image_ids] = True

    # ------------------------------------------------------------------ grid discovery
    def _grids_in_message(self, tokens: np.ndarray, start: int, end: int) -> Iterator[np.ndarray]:
        """Index arrays of the rectangular code grids between ``start`` and ``end`` (one assistant turn)."""
        codes = start + 1 + np.flatnonzero(self.is_image[tokens[start + 1:end]])
        if not len(codes):
            return
        cuts, row_breaks = [0], []
        for g in np.flatnonzero(np.diff(codes) > 1):
            between = tokens[codes[g] + 1:codes[g + 1]]
            text = self.tokenizer.decode(between[:8].tolist()) if len(between) <= 8 else None
            (row_breaks if text in ("\n", "\r\n") else cuts).append(int(g) + 1)
        cuts.append(len(codes))
        for first, last in zip(cuts[:-1], cuts[1:]):
            edges = [first, *(r for r in row_breaks if first < r < last), last]
            widths = np.diff(edges)
            if np.any(widths != widths[0]):
                raise ValueError("assistant image grid has unequal row widths")
            yield codes[first:last]

    def _blocks(self, tokens: np.ndarray, valid: np.ndarray, segments: np.ndarray):
        if not self.is_image[np.clip(tokens, 0, len(self.is_image) - 1)].any():
            return
        change = (segments[1:] != segments[:-1]) | (valid[1:] != valid[:-1])
        bounds = np.flatnonzero(np.r_[True, change, True])
        for left, right in zip(bounds[:-1], bounds[1:]):
            if not valid[left]:
                continue
            starts = left + np.flatnonzero(tokens[left:right] == self.start_id)
            ends = left + np.flatnonzero(tokens[left:right] == self.end_id)
            for n, s in enumerate(starts):
                limit = starts[n + 1] if n + 1 < len(starts) else right
                e = np.searchsorted(ends, s)
                if e == len(ends) or ends[e] >= limit:
                    continue  # unclosed (e.g. truncated) turn stays autoregressive
                end = int(ends[e])
                header = self.tokenizer.decode(tokens[s + 1:min(end, s + 33)].tolist())
                if not header.startswith(("assistant\n", "assistant\r\n")):
                    continue
                for grid in self._grids_in_message(tokens, int(s), end):
                    yield int(grid[0]), int(grid[-1]) + 1, grid

    # ------------------------------------------------------------------ transform
    def __call__(self, batch: Mapping[str, np.ndarray], *, step: int) -> dict[str, np.ndarray]:
        if self.probability == 0.0:
            return dict(batch)
        original = np.asarray(batch["input_ids"], dtype=np.int32)
        valid = np.asarray(batch["attention_mask"]) != 0
        segments = np.asarray(batch["segment_ids"])
        weights = np.asarray(batch["loss_weights"], dtype=np.float32)
        tokens = original.copy()
        targets = np.zeros_like(original)
        pw = np.zeros_like(weights)
        targets[:, :-1] = original[:, 1:]
        pw[:, :-1] = weights[:, 1:] * (valid[:, :-1] & valid[:, 1:] & (segments[:, :-1] == segments[:, 1:]))
        attention_end = np.broadcast_to(np.arange(original.shape[1], dtype=np.int32), original.shape).copy()
        rng = np.random.default_rng(np.random.SeedSequence([self.seed, step]))
        for row in range(len(original)):
            for start, end, grid in self._blocks(original[row], valid[row], segments[row]):
                if not np.any(weights[row, grid] > 0) or rng.random() >= self.probability:
                    continue
                count = max(1, math.ceil(len(grid) * math.cos(math.pi * 0.5 * rng.random())))
                masked = rng.choice(grid, size=count, replace=False)
                tokens[row, masked] = self.mask_id
                attention_end[row, start:end] = end - 1
                pw[row, max(0, start - 1):end] = 0.0
                targets[row, masked] = original[row, masked]
                pw[row, masked] = weights[row, masked]
        return {**batch, "input_ids": tokens, "attention_end": attention_end, "prediction_targets": targets,
                "prediction_weights": pw}

    def batches(self, batches, *, start_step: int) -> Iterator:
        for step, batch in enumerate(batches, start=start_step):
            if isinstance(batch, Mapping):
                yield self(batch, step=step)
            else:
                yield batch.with_data(self(batch.data, step=step))
