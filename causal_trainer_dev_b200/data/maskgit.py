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

The work is split in two: :class:`GridFinder` turns a token row into a list of
:class:`Grid` spans (a scan over *runs* of code tokens, no randomness), and
:class:`MaskGITBatchTransform` draws the masks for those spans and edits the batch arrays.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass
from typing import Iterator, Mapping

import numpy as np

_CODE_NAME = re.compile(r"<\|image_[0-9]+\|>\Z")
_MARKERS = ("[MASK]", "<|im_start|>", "<|im_end|>")
_NEWLINES = ("\n", "\r\n")
_HEADER_TOKENS = 32          # how far into a turn the role header is looked for
_SEPARATOR_TOKENS = 8        # a row separator longer than this many tokens is not a newline


@dataclass(frozen=True)
class Grid:
    """One rectangular block of image codes inside an assistant turn."""
    positions: np.ndarray      # indices of the code tokens, ascending

    @property
    def first(self) -> int:
        return int(self.positions[0])

    @property
    def stop(self) -> int:
        return int(self.positions[-1]) + 1


class GridFinder:
    """Locates image grids in one token row.  Text decisions (is this gap a newline? does this
    turn belong to the assistant?) go through the tokenizer's decoder and are memoised by token
    ids, so a batch of similar rows decodes each distinct piece once."""

    def __init__(self, tokenizer, code_table: np.ndarray, start_id: int, end_id: int):
        self.tokenizer = tokenizer
        self.code_table = code_table
        self.start_id, self.end_id = start_id, end_id
        self._text: dict[bytes, str] = {}

    def _decoded(self, ids: np.ndarray) -> str:
        key = ids.tobytes()                      # the ids' bytes: one C call instead of a tuple of Python ints
        text = self._text.get(key)
        if text is None:
            text = self._text[key] = self.tokenizer.decode([int(i) for i in ids])
        return text

    def is_code(self, tokens: np.ndarray) -> np.ndarray:
        return self.code_table[np.clip(tokens, 0, len(self.code_table) - 1)] & (tokens >= 0) & (
            tokens < len(self.code_table))

    def _documents(self, valid: np.ndarray, segments: np.ndarray) -> Iterator[tuple[int, int]]:
        """Maximal spans of attended tokens with one segment id."""
        edge = np.empty(len(valid) + 1, dtype=bool)
        edge[0] = edge[-1] = True
        edge[1:-1] = (segments[1:] != segments[:-1]) | (valid[1:] != valid[:-1])
        cut = np.flatnonzero(edge)
        for a, b in zip(cut[:-1], cut[1:]):
            if valid[a]:
                yield int(a), int(b)

    def _assistant_turns(self, tokens: np.ndarray, a: int, b: int) -> Iterator[tuple[int, int]]:
        """``(index of <|im_start|>, index of its <|im_end|>)`` for closed assistant turns of a document."""
        opens = a + np.flatnonzero(tokens[a:b] == self.start_id)
        closes = a + np.flatnonzero(tokens[a:b] == self.end_id)
        if not len(opens) or not len(closes):
            return
        # the first close after each open must come before the next open (else the turn was cut off)
        nxt = np.append(opens[1:], b)
        which = np.searchsorted(closes, opens)
        for o, limit, w in zip(opens, nxt, which):
            if w < len(closes) and closes[w] < limit:
                close = int(closes[w])
                header = self._decoded(tokens[o + 1:min(close, o + 1 + _HEADER_TOKENS)])
                if header.startswith(tuple("assistant" + nl for nl in _NEWLINES)):
                    yield int(o), close

    def _grids_of_turn(self, tokens: np.ndarray, code: np.ndarray, o: int, close: int) -> Iterator[Grid]:
        inside = o + 1 + np.flatnonzero(code[o + 1:close])
        if not len(inside):
            return
        # runs of adjacent codes = grid rows; a run boundary is a newline (same grid) or anything else (new grid)
        breaks = np.flatnonzero(np.diff(inside) != 1) + 1
        run_first = np.concatenate(([0], breaks))
        run_stop = np.concatenate((breaks, [len(inside)]))
        rows: list[tuple[int, int]] = []

        def close_grid() -> Grid:
            widths = {stop - first for first, stop in rows}
            if len(widths) != 1:
                raise ValueError("assistant image grid has unequal row widths")
            return Grid(inside[rows[0][0]:rows[-1][1]])

        for r, (first, stop) in enumerate(zip(run_first, run_stop)):
            if rows:
                gap = tokens[inside[rows[-1][1] - 1] + 1:inside[first]]
                if len(gap) > _SEPARATOR_TOKENS or self._decoded(gap) not in _NEWLINES:
                    yield close_grid()
                    rows = []
            rows.append((int(first), int(stop)))
        yield close_grid()

    def grids(self, tokens: np.ndarray, valid: np.ndarray, segments: np.ndarray) -> list[Grid]:
        code = self.is_code(tokens)
        if not code.any():
            return []
        found: list[Grid] = []
        for a, b in self._documents(valid, segments):
            for o, close in self._assistant_turns(tokens, a, b):
                found.extend(self._grids_of_turn(tokens, code, o, close))
        return found


class MaskGITBatchTransform:
    def __init__(self, tokenizer, *, probability: float, seed: int):
        if not math.isfinite(probability) or not 0.0 <= probability <= 1.0:
            raise ValueError("maskgit_probability must be between 0 and 1")
        self.probability, self.seed, self.tokenizer = probability, seed, tokenizer
        vocab = tokenizer.get_vocab()
        ids = []
        for marker in _MARKERS:
            if marker not in vocab or tokenizer(marker)["input_ids"] != [vocab[marker]]:
                raise ValueError(f"MaskGIT requires {marker!r} to encode as one token")
            ids.append(vocab[marker])
        self.mask_id, self.start_id, self.end_id = ids
        codes = np.fromiter((i for name, i in vocab.items() if _CODE_NAME.fullmatch(name)), dtype=np.int64)
        if not len(codes):
            raise ValueError("MaskGIT requires <|image_i|> tokens in the tokenizer vocabulary")
        size = max(max(vocab.values()), getattr(tokenizer, "pad_token_id", None) or 0) + 1
        self.is_image = np.zeros(size, dtype=bool)
        self.is_image[codes] = True
        self.finder = GridFinder(tokenizer, self.is_image, self.start_id, self.end_id)

    def _draw(self, rng: np.random.Generator, grid: Grid) -> np.ndarray | None:
        """The masked positions of ``grid`` for this step, or None when the coin says autoregressive.
        Draw order (a resume contract): selection, then ratio, then the choice of positions."""
        if rng.random() >= self.probability:
            return None
        n = len(grid.positions)
        count = max(1, math.ceil(n * math.cos(0.5 * math.pi * rng.random())))
        return rng.choice(grid.positions, size=count, replace=False)

    def __call__(self, batch: Mapping[str, np.ndarray], *, step: int) -> dict[str, np.ndarray]:
        if self.probability == 0.0:
            return dict(batch)
        source = np.asarray(batch["input_ids"], dtype=np.int32)
        attended = np.asarray(batch["attention_mask"]) != 0
        segments = np.asarray(batch["segment_ids"])
        weights = np.asarray(batch["loss_weights"], dtype=np.float32)
        rows, length = source.shape

        # next-token defaults: position i predicts token i + 1 inside one attended document
        same_doc = attended[:, :-1] & attended[:, 1:] & (segments[:, :-1] == segments[:, 1:])
        targets = np.concatenate([source[:, 1:], np.zeros((rows, 1), source.dtype)], axis=1)
        pred_w = np.concatenate([weights[:, 1:] * same_doc, np.zeros((rows, 1), np.float32)], axis=1).astype(np.float32)
        tokens = source.copy()
        attention_end = np.tile(np.arange(length, dtype=np.int32), (rows, 1))

        rng = np.random.default_rng(np.random.SeedSequence([self.seed, step]))
        for r in range(rows):
            for grid in self.finder.grids(source[r], attended[r], segments[r]):
                if not (weights[r, grid.positions] > 0).any():
                    continue                      # unsupervised grid: no draw at all
                masked = self._draw(rng, grid)
                if masked is None:
                    continue
                a, b = grid.first, grid.stop
                attention_end[r, a:b] = b - 1                    # block-local bidirectional attention
                pred_w[r, max(a - 1, 0):b] = 0.0                 # no next-token edge into, inside or out of the block
                tokens[r, masked] = self.mask_id
                targets[r, masked] = source[r, masked]           # same-position reconstruction
                pred_w[r, masked] = weights[r, masked]
        out = dict(batch)
        out.update(input_ids=tokens, attention_end=attention_end, prediction_targets=targets, prediction_weights=pred_w)
        return out

    def batches(self, batches, *, start_step: int) -> Iterator:
        """Applies the transform to a stream of host batches (plain mappings or envelopes with
        ``data`` / ``with_data``), numbering them from the absolute optimizer step ``start_step``."""
        step = start_step
        for item in batches:
            yield self(item, step=step) if isinstance(item, Mapping) else item.with_data(self(item.data, step=step))
            step += 1
