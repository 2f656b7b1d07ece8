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
from .packing import PackedExample

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


# ----------------------------------------------------------------------------------------- grouping
def canonical_record(record: Mapping[str, Sequence], *, assistant_only_loss: bool) -> PackedExample:
    missing = [f for f in MODEL_FIELDS if f not in record]
    if missing:
        raise ValueError(f"streaming packed record is missing model fields: {missing}")
    out: PackedExample = {f: [int(v) for v in record[f]] for f in MODEL_FIELDS}
    n = len(out["input_ids"])
    if any(len(out[f]) != n for f in MODEL_FIELDS):
        raise ValueError("streaming packed model fields are not aligned")
    if "assistant_masks" in record:
        am = [int(v) for v in record["assistant_masks"]]
        if len(am) != n:
            raise ValueError("streaming assistant mask is not aligned with input_ids")
        out["assistant_masks"] = am
    elif assistant_only_loss:
        raise ValueError("assistant-masked streaming record is missing assistant_masks")
    if "loss_weights" in record:
        w = [float(v) for v in record["loss_weights"]]
    else:
        w = [float(v) for v in out["assistant_masks" if assistant_only_loss else "attention_mask"]]
    if len(w) != n:
        raise ValueError("streaming loss_weights are not aligned with input_ids")
    wa = np.asarray(w, dtype=np.float32)
    if not np.isfinite(wa).all() or (wa < 0).any():
        raise ValueError("streaming loss_weights must be finite and non-negative")
    out["loss_weights"] = w
    a = np.asarray(out["attention_mask"], dtype=np.int32)
    s = np.asarray(out["segment_ids"], dtype=np.int32)
    if not np.any((a[:-1] != 0) & (a[1:] != 0) & (s[:-1] != 0) & (s[:-1] == s[1:]) & (wa[1:] > 0)):
        raise ValueError("a streaming packed row has no positive-weight causal target with a valid same-segment "
                         "predecessor")
    return out


def _zero_loss_copy(record: PackedExample) -> PackedExample:
    out = {k: list(v) for k, v in record.items()}
    out["loss_weights"] = [0.0] * len(record["input_ids"])
    if "assistant_masks" in out:
        out["assistant_masks"] = [0] * len(record["input_ids"])
    return out


def _stack(records: Sequence[PackedExample]) -> dict[str, np.ndarray]:
    return {f: np.asarray([r[f] for r in records], dtype=np.float32 if f == "loss_weights" else np.int32)
            for f in (*MODEL_FIELDS, "loss_weights")}


@dataclass(frozen=True)
class _Grouped:
    data: dict[str, np.ndarray]
    source_examples: int
    epoch: int
    is_epoch_end: bool = False


def _row_counts(envelope: Any) -> list[int]:
    records = tuple(envelope.records)
    if not records:
        return []
    explicit = getattr(envelope, "record_source_examples", None)
    if explicit is None:
        counts = [0] * len(records)
        counts[-1] = int(envelope.source_examples)
        return counts
    counts = [int(v) for v in explicit]
    if len(counts) != len(records):
        raise ValueError("record_source_examples must align with streaming records")
    if any(v < 0 for v in counts):
        raise ValueError("record_source_examples must be non-negative")
    if sum(counts) != int(envelope.source_examples):
        raise ValueError("record_source_examples must sum to source_examples")
    return counts


class BatchGrouper:
    """State machine: envelopes in, fixed-size grouped batches out (one batch is held back)."""

    def __init__(self, size: int, assistant_only_loss: bool):
        if size <= 0:
            raise ValueError("effective_batch_size must be positive")
        self.size, self.masked = size, assistant_only_loss
        self.rows: list[tuple[PackedExample, int]] = []
        self.held: _Grouped | None = None
        self.unassigned = 0          # source rows of fully filtered windows, waiting for a row to charge
        self.epoch: int | None = None

    def feed(self, envelope: Any) -> Iterator[_Grouped]:
        epoch = int(envelope.epoch)
        if self.epoch is None:
            self.epoch = epoch
        elif epoch != self.epoch:
            raise ValueError("streaming epoch changed without an epoch-end envelope")
        records, counts = tuple(envelope.records), _row_counts(envelope)
        if records:
            counts[0] += self.unassigned
            self.unassigned = 0
            self.rows.extend((canonical_record(r, assistant_only_loss=self.masked), c)
                             for r, c in zip(records, counts, strict=True))
        else:
            self.unassigned += int(envelope.source_examples)
        while len(self.rows) >= self.size:
            take, self.rows = self.rows[:self.size], self.rows[self.size:]
            if self.held is not None:
                yield self.held
            self.held = _Grouped(_stack([r for r, _ in take]), sum(c for _, c in take), epoch)
        if not bool(envelope.is_epoch_end):
            return
        if self.rows:
            if self.held is not None:
                yield self.held
            real = [r for r, _ in self.rows]
            src = sum(c for _, c in self.rows) + self.unassigned
            self.unassigned = 0
            padded = real + [_zero_loss_copy(real[-1]) for _ in range(self.size - len(real))]
            self.held = _Grouped(_stack(padded), src, epoch)
            self.rows = []
        elif self.held is not None and self.unassigned:
            self.held = replace(self.held, source_examples=self.held.source_examples + self.unassigned)
            self.unassigned = 0
        if self.held is None:
            raise ValueError(f"streaming epoch {epoch} produced no trainable records after preprocessing")
        yield replace(self.held, is_epoch_end=True)
        self.held, self.epoch = None, None

    def finish(self) -> None:
        if self.epoch is not None or self.rows or self.held is not None or self.unassigned:
            raise ValueError("streaming source ended without an epoch-end envelope")


class StreamCursor:
    """Running progress and digest over committed batches."""

    def __init__(self) -> None:
        self.seen = 0
        self.epoch_seen = 0
        self.epoch: int | None = None
        self.digest = hashlib.sha256(_DOMAIN)

    def advance(self, g: _Grouped) -> StreamingGlobalBatch:
        if self.epoch is None:
            self.epoch, self.epoch_seen = g.epoch, 0
        elif g.epoch != self.epoch:
            raise RuntimeError("streaming global batches changed epoch without completing the prior epoch")
        batch = StreamingGlobalBatch(
            data=g.data, source_examples=g.source_examples, source_examples_before=self.seen,
            source_examples_seen=self.seen + g.source_examples, epoch_source_examples_before=self.epoch_seen,
            epoch_source_examples_seen=self.epoch_seen + g.source_examples, epoch=g.epoch,
            is_epoch_end=g.is_epoch_end, stream_digest_before=self.digest.hexdigest(), stream_digest="",
        )
        self.seen += g.source_examples
        self.epoch_seen += g.source_examples
        self.digest.update(_batch_digest(batch, include_stream_state=False))
        if g.is_epoch_end:
            self.epoch, self.epoch_seen = None, 0
        return replace(batch, stream_digest=self.digest.hexdigest())


def iter_streaming_global_batches(envelopes: Iterable[Any], plan: StreamingBatchPlan, *, assistant_only_loss: bool,
                                  start_step: int = 0, expected_source_examples_before: int | None = None,
                                  expected_stream_digest_before: str | None = None) -> Iterator[StreamingGlobalBatch]:
    if start_step < 0 or start_step > plan.total_steps:
        raise ValueError(f"start_step must be in [0, {plan.total_steps}], got {start_step}")
    if expected_source_examples_before is not None and (
            type(expected_source_examples_before) is not int or expected_source_examples_before < 0):
        raise ValueError("expected_source_examples_before must be a non-negative integer or None")
    if expected_stream_digest_before is not None and (
            len(expected_stream_digest_before) != 64
            or any(c not in "0123456789abcdef" for c in expected_stream_digest_before)):
        raise ValueError("expected_stream_digest_before must be a lowercase SHA-256 digest or None")
    cursor = StreamCursor()
    grouper = BatchGrouper(plan.effective_batch_size, assistant_only_loss)
    step = 0
    checked = False

    def check_resume_point() -> None:
        nonlocal checked
        if expected_source_examples_before is not None and cursor.seen != expected_source_examples_before:
            raise RuntimeError(f"streaming resume replay reached source example {cursor.seen}, but checkpoint "
                               f"progress records {expected_source_examples_before}")
        if expected_stream_digest_before is not None and cursor.digest.hexdigest() != expected_stream_digest_before:
            raise RuntimeError("streaming resume replay produced different training batches before the checkpoint; "
                               "pin dataset_revision to the original immutable dataset commit")
        checked = True

    for envelope in envelopes:
        for grouped in grouper.feed(envelope):
            if step == start_step and not checked:
                check_resume_point()
            batch = cursor.advance(grouped)
            if step >= start_step:
                yield batch
            step += 1
            if plan.max_steps > 0 and step >= plan.max_steps:
                if step == start_step and not checked:
                    check_resume_point()
                return
    grouper.finish()
    if step < start_step:
        raise RuntimeError(f"streaming resume requested optimizer step {start_step}, but the reconstructed source "
                           f"produced only {step} batches")
    if step == start_step and not checked:
        check_resume_point()
