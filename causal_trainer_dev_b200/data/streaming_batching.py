"""Fixed-size global optimizer batches out of streaming packing windows, with exact resume.

Windows (``StreamingBatchEnvelope``) arrive with a variable number of packed rows.  The
:class:`BatchGrouper` cuts them into batches of ``micro_batch * accumulation`` rows, keeps the
last full batch of an epoch back until it knows whether the epoch is over (so the batch that
closes an epoch carries ``is_epoch_end``), and pads the epoch tail with zero-loss copies of
the last real row.  Source rows that were filtered out are charged to a trained row, so
``source_examples_seen`` always equals the number of raw rows consumed when a batch is
committed.  :class:`StreamCursor` chains a SHA-256 over every batch; a resumed run replays the
stream from the start, discards the first ``start_step`` batches and must arrive at the
recorded row count and digest, also exactly at end of stream
(src/causal_trainer/data/streaming_batching.py:21-470).
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import dataclass, replace
from typing import Any, Iterable, Iterator, Mapping, Sequence

import numpy as np

from .batching import MODEL_FIELDS

UNKNOWN_TOTAL_STEPS = 2**31 - 1
_DOMAIN = b"causal-trainer-stream-v1\0"


@dataclass(frozen=True)
class StreamingBatchPlan:
    """``total_steps`` is exact only with ``max_steps``; otherwise a large sentinel, because
    metadata row counts are estimates and must never cap training."""

    source_examples_per_epoch: int | None
    global_micro_batch_size: int
    accumulation_steps: int
    epochs: int | None
    max_steps: int
    steps_per_epoch: int | None
    total_steps: int

    @classmethod
    def create(cls, source_examples_per_epoch: int | None, global_micro_batch_size: int, accumulation_steps: int,
               epochs: int, max_steps: int) -> "StreamingBatchPlan":
        if source_examples_per_epoch is not None and source_examples_per_epoch < 0:
            raise ValueError("streaming source example count cannot be negative")
        if global_micro_batch_size <= 0 or accumulation_steps <= 0:
            raise ValueError("streaming batch sizes must be positive")
        if max_steps <= 0 and epochs <= 0:
            raise ValueError("streaming epochs must be positive unless max_steps is set")
        effective = global_micro_batch_size * accumulation_steps
        per_epoch = math.ceil(source_examples_per_epoch / effective) if source_examples_per_epoch is not None else None
        if max_steps > 0:
            return cls(source_examples_per_epoch, global_micro_batch_size, accumulation_steps, None, max_steps,
                       per_epoch, max_steps)
        return cls(source_examples_per_epoch, global_micro_batch_size, accumulation_steps, epochs, max_steps,
                   per_epoch, UNKNOWN_TOTAL_STEPS)

    @property
    def effective_batch_size(self) -> int:
        return self.global_micro_batch_size * self.accumulation_steps

    @property
    def total_source_examples(self) -> int | None:
        if self.source_examples_per_epoch is None or self.epochs is None:
            return None
        return self.source_examples_per_epoch * self.epochs

    @property
    def has_exact_step_limit(self) -> bool:
        return self.max_steps > 0


@dataclass(frozen=True)
class StreamingGlobalBatch:
    data: Mapping[str, Any]
    source_examples: int
    source_examples_before: int
    source_examples_seen: int
    epoch_source_examples_before: int
    epoch_source_examples_seen: int
    epoch: int
    is_epoch_end: bool
    stream_digest_before: str
    stream_digest: str

    def with_data(self, data: Mapping[str, Any]) -> "StreamingGlobalBatch":
        return replace(self, data=data)


def _batch_digest(batch: StreamingGlobalBatch, include_stream_state: bool) -> bytes:
    h = hashlib.sha256()

    def put(raw) -> None:
        h.update(len(raw).to_bytes(8, "big"))
        h.update(raw)

    meta: dict[str, Any] = {
        "epoch": batch.epoch, "is_epoch_end": batch.is_epoch_end, "source_examples": batch.source_examples,
        "source_examples_before": batch.source_examples_before, "source_examples_seen": batch.source_examples_seen,
        "epoch_source_examples_before": batch.epoch_source_examples_before,
        "epoch_source_examples_seen": batch.epoch_source_examples_seen,
    }
    if include_stream_state:
        meta["stream_digest_before"] = batch.stream_digest_before
        meta["stream_digest"] = batch.stream_digest
    put(json.dumps(meta, separators=(",", ":"), sort_keys=True).encode("utf-8"))
    for name in sorted(batch.data):
        arr = np.ascontiguousarray(batch.data[name])
        put(name.encode("utf-8"))
        put(arr.dtype.str.encode("ascii"))
        put(json.dumps(arr.shape, separators=(",", ":")).encode("ascii"))
        put(memoryview(arr).cast("B"))
    return h.digest()


def streaming_global_batch_digest(batch: StreamingGlobalBatch) -> bytes:
    """Digest every rank compares before a step (status byte + this digest is the per-batch vote)."""
    return _batch_digest(batch, include_stream_state=True)


# ----------------------------------------------------------------------------------------- rows as typed arrays
_INT_FIELDS = MODEL_FIELDS
_BATCH_FIELDS = (*MODEL_FIELDS, "loss_weights")


def encode_row(record: Mapping[str, Sequence], *, assistant_only_loss: bool) -> dict[str, np.ndarray]:
    """One packed record as typed 1-D arrays (``int32`` model fields, ``float32`` ``loss_weights``),
    validated: aligned fields, finite non-negative weights (explicit > assistant mask > attention
    mask), and at least one positive-weight target whose predecessor is an attended token of the
    same segment (a row without one can never contribute a loss term)."""
    absent = [f for f in _INT_FIELDS if f not in record]
    if absent:
        raise ValueError(f"streaming packed record is missing model fields: {absent}")
    row = {f: np.asarray(record[f], dtype=np.int64).astype(np.int32) for f in _INT_FIELDS}
    width = row["input_ids"].shape[0]
    if any(v.ndim != 1 or v.shape[0] != width for v in row.values()):
        raise ValueError("streaming packed model fields are not aligned")
    mask = record.get("assistant_masks")
    if mask is not None:
        mask = np.asarray(mask, dtype=np.int64).astype(np.int32)
        if mask.shape != (width,):
            raise ValueError("streaming assistant mask is not aligned with input_ids")
    elif assistant_only_loss:
        raise ValueError("assistant-masked streaming record is missing assistant_masks")
    if "loss_weights" in record:
        weights = np.asarray(record["loss_weights"], dtype=np.float64)
    else:
        weights = (mask if assistant_only_loss else row["attention_mask"]).astype(np.float64)
    if weights.shape != (width,):
        raise ValueError("streaming loss_weights are not aligned with input_ids")
    weights = weights.astype(np.float32)
    if not np.isfinite(weights).all() or (weights < 0).any():
        raise ValueError("streaming loss_weights must be finite and non-negative")
    row["loss_weights"] = weights
    attended, segment = row["attention_mask"] != 0, row["segment_ids"]
    edge = attended[:-1] & attended[1:] & (segment[:-1] != 0) & (segment[:-1] == segment[1:]) & (weights[1:] > 0)
    if not edge.any():
        raise ValueError("a streaming packed row has no positive-weight causal target with a valid same-segment "
                         "predecessor")
    return row


class RowQueue:
    """FIFO of encoded rows kept as 2-D arrays (one per field) plus the number of raw source rows
    charged to each.  ``pop`` hands out the oldest ``n`` rows as a batch without touching Python
    lists of token ids; the arrays grow by doubling."""

    def __init__(self) -> None:
        self.fields: dict[str, np.ndarray] | None = None
        self.charge = np.zeros(0, dtype=np.int64)
        self.head = 0
        self.tail = 0

    def __len__(self) -> int:
        return self.tail - self.head

    def _reserve(self, width: int, extra: int) -> None:
        if self.fields is None:
            cap = max(16, extra)
            self.fields = {f: np.zeros((cap, width), dtype=np.float32 if f == "loss_weights" else np.int32)
                           for f in _BATCH_FIELDS}
            self.charge = np.zeros(cap, dtype=np.int64)
            return
        have = self.charge.shape[0]
        if self.tail + extra <= have:
            return
        live = len(self)
        cap = max(2 * have, live + extra)
        for f, old in self.fields.items():
            grown = np.zeros((cap, old.shape[1]), dtype=old.dtype)
            grown[:live] = old[self.head:self.tail]
            self.fields[f] = grown
        charge = np.zeros(cap, dtype=np.int64)
        charge[:live] = self.charge[self.head:self.tail]
        self.charge, self.head, self.tail = charge, 0, live

    def push(self, row: dict[str, np.ndarray], charge: int) -> None:
        width = row["input_ids"].shape[0]
        if self.fields is not None and self.fields["input_ids"].shape[1] != width:
            raise ValueError("streaming packed rows have different lengths")
        self._reserve(width, 1)
        for f in _BATCH_FIELDS:
            self.fields[f][self.tail] = row[f]
        self.charge[self.tail] = charge
        self.tail += 1

    def pop(self, n: int, pad_to: int | None = None) -> tuple[dict[str, np.ndarray], int]:
        """Oldest ``n`` rows as fresh arrays and their summed charge.  With ``pad_to`` the batch is
        filled up with copies of its last row that carry zero loss weight."""
        a, b = self.head, self.head + n
        size = n if pad_to is None else pad_to
        out = {}
        for f, store in self.fields.items():
            block = np.empty((size, store.shape[1]), dtype=store.dtype)
            block[:n] = store[a:b]
            if size > n:
                block[n:] = 0.0 if f == "loss_weights" else store[b - 1]
            out[f] = block
        charged = int(self.charge[a:b].sum())
        self.head = b
        if self.head == self.tail:
            self.head = self.tail = 0
        return out, charged


@dataclass(frozen=True)
class _Pending:
    data: dict[str, np.ndarray]
    source_examples: int
    epoch: int
    is_epoch_end: bool = False


def _charges(envelope: Any, rows: int) -> np.ndarray:
    """Raw source rows charged to each packed row of a window (all to the last row unless the
    window says otherwise)."""
    if rows == 0:                      # a fully filtered window: its source rows are charged later
        return np.zeros(0, dtype=np.int64)
    total = int(envelope.source_examples)
    explicit = getattr(envelope, "record_source_examples", None)
    if explicit is None:
        out = np.zeros(rows, dtype=np.int64)
        out[-1] = total
        return out
    out = np.asarray([int(v) for v in explicit], dtype=np.int64)
    if out.shape[0] != rows:
        raise ValueError("record_source_examples must align with streaming records")
    if (out < 0).any():
        raise ValueError("record_source_examples must be non-negative")
    if int(out.sum()) != total:
        raise ValueError("record_source_examples must sum to source_examples")
    return out


class BatchGrouper:
    """Windows in, fixed-size batches out.  The newest complete batch is always held back one
    turn: only when the next batch (or the end of the epoch) arrives is it known whether it closes
    the epoch.  Source rows of windows that produced no packed row wait in ``orphans`` and are
    charged to the next row that does arrive (or to the closing batch)."""

    def __init__(self, size: int, assistant_only_loss: bool):
        if size <= 0:
            raise ValueError("effective_batch_size must be positive")
        self.size, self.masked = size, assistant_only_loss
        self.queue = RowQueue()
        self.held: _Pending | None = None
        self.orphans = 0
        self.epoch: int | None = None

    def _hold(self, pending: _Pending) -> Iterator[_Pending]:
        if self.held is not None:
            yield self.held
        self.held = pending

    def feed(self, envelope: Any) -> Iterator[_Pending]:
        epoch = int(envelope.epoch)
        if self.epoch is None:
            self.epoch = epoch
        elif epoch != self.epoch:
            raise ValueError("streaming epoch changed without an epoch-end envelope")
        records = tuple(envelope.records)
        charges = _charges(envelope, len(records))
        if records:
            charges[0] += self.orphans
            self.orphans = 0
            for record, charge in zip(records, charges):
                self.queue.push(encode_row(record, assistant_only_loss=self.masked), int(charge))
        else:
            self.orphans += int(envelope.source_examples)
        while len(self.queue) >= self.size:
            data, charged = self.queue.pop(self.size)
            yield from self._hold(_Pending(data, charged, epoch))
        if not bool(envelope.is_epoch_end):
            return
        leftover = len(self.queue)
        if leftover:
            data, charged = self.queue.pop(leftover, pad_to=self.size)
            yield from self._hold(_Pending(data, charged + self.orphans, epoch))
        elif self.held is not None and self.orphans:
            self.held = replace(self.held, source_examples=self.held.source_examples + self.orphans)
        self.orphans = 0
        if self.held is None:
            raise ValueError(f"streaming epoch {epoch} produced no trainable records after preprocessing")
        closing, self.held, self.epoch = self.held, None, None
        yield replace(closing, is_epoch_end=True)

    def finish(self) -> None:
        if self.epoch is not None or len(self.queue) or self.held is not None or self.orphans:
            raise ValueError("streaming source ended without an epoch-end envelope")


class StreamCursor:
    """Progress counters and the chained SHA-256 over every committed batch."""

    def __init__(self) -> None:
        self.seen = 0
        self.epoch_seen = 0
        self.epoch: int | None = None
        self.digest = hashlib.sha256(_DOMAIN)

    def advance(self, pending: _Pending) -> StreamingGlobalBatch:
        if self.epoch is None:
            self.epoch, self.epoch_seen = pending.epoch, 0
        elif pending.epoch != self.epoch:
            raise RuntimeError("streaming global batches changed epoch without completing the prior epoch")
        n = pending.source_examples
        before = self.digest.hexdigest()
        draft = StreamingGlobalBatch(
            data=pending.data, source_examples=n, source_examples_before=self.seen, source_examples_seen=self.seen + n,
            epoch_source_examples_before=self.epoch_seen, epoch_source_examples_seen=self.epoch_seen + n,
            epoch=pending.epoch, is_epoch_end=pending.is_epoch_end, stream_digest_before=before, stream_digest="")
        self.digest.update(_batch_digest(draft, include_stream_state=False))
        self.seen += n
        self.epoch_seen = 0 if pending.is_epoch_end else self.epoch_seen + n
        if pending.is_epoch_end:
            self.epoch = None
        return replace(draft, stream_digest=self.digest.hexdigest())


class _ResumePoint:
    """What a checkpoint recorded about the stream before its step; checked once, exactly when the
    replay stands at that step."""

    def __init__(self, source_examples: int | None, digest: str | None):
        if source_examples is not None and (type(source_examples) is not int or source_examples < 0):
            raise ValueError("expected_source_examples_before must be a non-negative integer or None")
        if digest is not None and (len(digest) != 64 or set(digest) - set("0123456789abcdef")):
            raise ValueError("expected_stream_digest_before must be a lowercase SHA-256 digest or None")
        self.source_examples, self.digest = source_examples, digest
        self.done = False

    def check(self, cursor: StreamCursor) -> None:
        if self.done:
            return
        self.done = True
        if self.source_examples is not None and cursor.seen != self.source_examples:
            raise RuntimeError(f"streaming resume replay reached source example {cursor.seen}, but checkpoint "
                               f"progress records {self.source_examples}")
        if self.digest is not None and cursor.digest.hexdigest() != self.digest:
            raise RuntimeError("streaming resume replay produced different training batches before the checkpoint; "
                               "pin dataset_revision to the original immutable dataset commit")


def iter_streaming_global_batches(envelopes: Iterable[Any], plan: StreamingBatchPlan, *, assistant_only_loss: bool,
                                  start_step: int = 0, expected_source_examples_before: int | None = None,
                                  expected_stream_digest_before: str | None = None) -> Iterator[StreamingGlobalBatch]:
    """Replays the stream from its start: the first ``start_step`` batches only feed the cursor,
    the checkpoint's record is verified when the replay reaches ``start_step`` (also when that is
    the end of the stream), and everything after is yielded."""
    if start_step < 0 or start_step > plan.total_steps:
        raise ValueError(f"start_step must be in [0, {plan.total_steps}], got {start_step}")
    resume = _ResumePoint(expected_source_examples_before, expected_stream_digest_before)
    cursor = StreamCursor()
    grouper = BatchGrouper(plan.effective_batch_size, assistant_only_loss)
    limit = plan.max_steps if plan.max_steps > 0 else None
    step = 0
    for envelope in envelopes:
        for pending in grouper.feed(envelope):
            if step == start_step:
                resume.check(cursor)
            batch = cursor.advance(pending)
            step += 1
            if step > start_step:
                yield batch
            if limit is not None and step >= limit:
                if step == start_step:
                    resume.check(cursor)
                return
    grouper.finish()
    if step < start_step:
        raise RuntimeError(f"streaming resume requested optimizer step {start_step}, but the reconstructed source "
                           f"produced only {step} batches")
    if step == start_step:
        resume.check(cursor)
