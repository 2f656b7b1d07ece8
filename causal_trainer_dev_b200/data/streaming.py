"""Bounded-memory streaming with online tokenisation and packing.

Every rank iterates the *same* deterministic source and builds the same records; nothing is
sharded by process, so the global batch is identical everywhere
(src/causal_trainer/data/streaming.py:376-479).  The pieces:

* :class:`ReplayingReader` — yields one epoch of a source and survives network failures
  forever: on a transient error it reopens the epoch, skips exactly the rows already
  delivered while re-hashing them, and refuses to continue if that prefix changed
  (``:170-295``);
* :func:`iter_streaming_batches` — windows of at most ``packing_batch_size`` source rows are
  tokenised, packed (or padded) and wrapped in a :class:`StreamingBatchEnvelope` that also says
  how many *source* rows each prepared row accounts for (filtered rows are charged to the last
  prepared row of the window); an explicit empty marker ends each epoch (``:473-479``).
"""
from __future__ import annotations

import hashlib
import itertools
import json
from dataclasses import dataclass
from itertools import islice
from typing import Any, Callable, Iterable, Iterator, Mapping, Sequence

from ..hf_retry import is_retryable_hf_error, retry_hf_call
from .packing import PackedExample, _check_same_fields, _join_row, best_fit_decreasing, normalize_example, pad_examples
from .preprocessing import EndPromptSettings, Preprocessor

SourceRecord = Mapping[str, Any]
StreamingSourceFactory = Callable[[int], Iterable[SourceRecord]]


@dataclass(frozen=True)
class StreamingDatasetMetadata:
    num_examples: int | None

    def __post_init__(self) -> None:
        if self.num_examples is not None and (type(self.num_examples) is not int or self.num_examples < 0):
            raise ValueError("num_examples must be a non-negative integer or None")

    @property
    def is_known(self) -> bool:
        return self.num_examples is not None

    def total_examples(self, num_epochs: int | None) -> int | None:
        if self.num_examples is None or num_epochs is None:
            return None
        if type(num_epochs) is not int or num_epochs < 0:
            raise ValueError("num_epochs must be a non-negative integer or None")
        return self.num_examples * num_epochs


def streaming_dataset_metadata(dataset: Any, split: str | None = None) -> StreamingDatasetMetadata:
    """Row-count estimate from a dataset's split metadata; anything missing or odd is ``None``."""
    splits = getattr(getattr(dataset, "info", None), "splits", None)
    if splits is None:
        return StreamingDatasetMetadata(None)
    name = split if split is not None else (str(dataset.split) if getattr(dataset, "split", None) is not None else None)
    if name is None:
        return StreamingDatasetMetadata(None)
    try:
        info = splits.get(name) if hasattr(splits, "get") else splits[name]
    except (KeyError, TypeError):
        return StreamingDatasetMetadata(None)
    value = info.get("num_examples") if isinstance(info, Mapping) else getattr(info, "num_examples", None)
    return StreamingDatasetMetadata(value if type(value) is int and value >= 0 else None)


@dataclass(frozen=True)
class StreamingBatchEnvelope:
    records: tuple[PackedExample, ...]
    source_examples: int
    record_source_examples: tuple[int, ...]
    epoch: int
    is_epoch_end: bool = False

    def __post_init__(self) -> None:
        if type(self.source_examples) is not int or self.source_examples < 0:
            raise ValueError("source_examples must be a non-negative integer")
        if type(self.epoch) is not int or self.epoch < 0:
            raise ValueError("epoch must be a non-negative integer")
        if len(self.record_source_examples) != len(self.records):
            raise ValueError("record_source_examples must align with records")
        if any(type(v) is not int or v < 0 for v in self.record_source_examples):
            raise ValueError("record_source_examples must contain non-negative integers")
        if self.records and sum(self.record_source_examples) != self.source_examples:
            raise ValueError("per-record source counts must sum to source_examples")
        if self.is_epoch_end and (self.records or self.source_examples or self.record_source_examples):
            raise ValueError("an epoch-end marker cannot contain records or source examples")


# ----------------------------------------------------------------------------------------- retrying reader
class PrefixLedger:
    """How many source rows were handed on, and a running SHA-256 over them (optionally over a subset
    of their fields).  A reopened source must reproduce the ledger before it may continue."""

    def __init__(self, fields: tuple[str, ...] | None):
        self.fields = fields
        self.count = 0
        self._hash = hashlib.sha256()

    @staticmethod
    def _absorb(h, record: SourceRecord, fields: tuple[str, ...] | None) -> None:
        view = record if fields is None else {f: record[f] for f in fields if f in record}
        raw = json.dumps(view, ensure_ascii=False, separators=(",", ":"), sort_keys=True, default=str).encode("utf-8")
        h.update(len(raw).to_bytes(8, "big"))
        h.update(raw)

    def record(self, row: SourceRecord) -> None:
        self._absorb(self._hash, row, self.fields)
        self.count += 1

    def skip_known_prefix(self, rows: Iterator[SourceRecord]) -> None:
        """Consumes ``count`` rows from a freshly opened source and checks that they are the rows
        already handed on."""
        check = hashlib.sha256()
        for seen in range(self.count):
            try:
                row = next(rows)
            except StopIteration as exc:
                raise _ShortReplay(f"the reconstructed streaming source ended after {seen} rows while {self.count} "
                                   "previously yielded rows had to be skipped; reopening the same epoch") from exc
            self._absorb(check, row, self.fields)
        if check.digest() != self._hash.digest():
            raise RuntimeError(
                "the reconstructed streaming source prefix changed during retry; pin dataset_revision to an immutable "
                "Hugging Face commit and ensure all hosts use the same deterministic source")


class _ShortReplay(ConnectionError):
    """The reopened source ended before the already-delivered prefix: treated as transient."""


_EXHAUSTED = object()


class ReplayingReader:
    """One epoch of ``source_factory(epoch)``, surviving transient failures for as long as they last.

    State: a :class:`PrefixLedger` of what was delivered.  Opening (or reopening) the source is one
    retried operation -- open, skip the known prefix while re-hashing it, fetch the next row -- so the
    back-off policy of ``hf_retry`` covers connection errors at any of the three.  A transient error
    while reading on is parked and re-raised *inside* the next open attempt, which makes it count
    against the same back-off clock instead of restarting it."""

    def __init__(self, source_factory: StreamingSourceFactory, epoch: int, *, initial_delay: float = 1.0,
                 max_delay: float = 60.0, operation: str = "streaming Hugging Face dataset",
                 digest_fields: Sequence[str] | None = None):
        if not callable(source_factory):
            raise TypeError("source_factory must be callable")
        if type(epoch) is not int or epoch < 0:
            raise ValueError("epoch must be a non-negative integer")
        fields = tuple(str(f) for f in digest_fields) if digest_fields is not None else None
        if fields is not None and not fields:
            raise ValueError("digest_fields cannot be empty")
        self.factory, self.epoch = source_factory, epoch
        self.retry = dict(initial_delay=initial_delay, max_delay=max_delay, operation=f"{operation} epoch {epoch}")
        self.ledger = PrefixLedger(fields)
        self._parked: Exception | None = None

    @property
    def delivered(self) -> int:
        return self.ledger.count

    def _open(self):
        if self._parked is not None:
            error, self._parked = self._parked, None
            raise error
        rows = iter(self.factory(self.epoch))
        self.ledger.skip_known_prefix(rows)
        return rows, next(rows, _EXHAUSTED)

    def __iter__(self) -> Iterator[SourceRecord]:
        rows, row = retry_hf_call(self._open, **self.retry)
        while row is not _EXHAUSTED:
            self.ledger.record(row)
            yield row
            try:
                row = next(rows, _EXHAUSTED)
            except Exception as exc:  # noqa: BLE001
                if not is_retryable_hf_error(exc):
                    raise
                self._parked = exc
            if self._parked is not None:
                # reopened outside the handler above: an error of the reopen (a changed prefix, say) must
                # not inherit the transient error as its context and be mistaken for one
                rows, row = retry_hf_call(self._open, **self.retry)


def iter_retrying_records(source_factory: StreamingSourceFactory, epoch: int, *, initial_delay: float = 1.0,
                          max_delay: float = 60.0, operation: str = "streaming Hugging Face dataset",
                          digest_fields: Sequence[str] | None = None) -> Iterator[SourceRecord]:
    return iter(ReplayingReader(source_factory, epoch, initial_delay=initial_delay, max_delay=max_delay,
                                operation=operation, digest_fields=digest_fields))


# ----------------------------------------------------------------------------------------- windows
def pack_window(examples: Sequence[Mapping[str, Any]], *, max_length: int, pad_token_id: int
                ) -> tuple[list[PackedExample], list[int]]:
    """Packs one window; also returns how many examples went into each row."""
    if not examples:
        return [], []
    normalized = [normalize_example(ex, max_length) for ex in examples]
    fields = tuple(f for f in _check_same_fields(normalized) if f != "segment_ids")
    rows = best_fit_decreasing(normalized, max_length=max_length)
    return [_join_row(r, fields, max_length, pad_token_id, "left") for r in rows], [len(r) for r in rows]


def ensure_loss_weights(record: PackedExample, *, assistant_only_loss: bool) -> PackedExample:
    """A copy of ``record`` that states its loss weights (explicit > assistant mask > attention mask)."""
    out = {k: list(v) for k, v in record.items()}
    basis = "loss_weights" if "loss_weights" in out else ("assistant_masks" if assistant_only_loss else "attention_mask")
    if basis not in out:
        raise ValueError(f"prepared streaming record is missing {basis!r}")
    weights = [float(v) for v in out[basis]]
    if len(weights) != len(out["input_ids"]):
        raise ValueError("prepared streaming loss_weights are not aligned with input_ids")
    if min(weights, default=0.0) < 0:
        raise ValueError("prepared streaming loss_weights must be non-negative")
    out["loss_weights"] = weights
    return out


def assign_source_counts(per_row: Sequence[int], *, source_examples: int, trainable_examples: int) -> tuple[int, ...]:
    """Source rows charged to each prepared row of a window: the examples packed into it, plus, on
    the last row, the window's rows that preprocessing dropped."""
    if not per_row:
        return ()
    counts = [int(v) for v in per_row]
    dropped = source_examples - trainable_examples
    if dropped < 0 or sum(counts) != trainable_examples:
        raise RuntimeError("streaming source provenance is inconsistent with prepared records")
    counts[-1] += dropped
    return tuple(counts)


class WindowAssembler:
    """Turns windows of raw source rows into envelopes of prepared rows (tokenise, then pack or pad)."""

    def __init__(self, preprocessor: Preprocessor, *, max_sequence_length: int, pad_token_id: int, packing: bool,
                 state_weights_from_mask: bool):
        self.pre = preprocessor
        self.length, self.pad, self.packing = max_sequence_length, pad_token_id, packing
        self.masked = state_weights_from_mask

    def envelope(self, window: list[SourceRecord], *, epoch: int, first_index: int) -> StreamingBatchEnvelope:
        tokenized = self.pre.run(window, example_index_offset=first_index, allow_empty=True)
        if self.packing:
            rows, per_row = pack_window(tokenized, max_length=self.length, pad_token_id=self.pad)
        else:
            rows = pad_examples(tokenized, max_length=self.length, pad_token_id=self.pad)
            per_row = [1] * len(rows)
        return StreamingBatchEnvelope(
            records=tuple(ensure_loss_weights(r, assistant_only_loss=self.masked) for r in rows),
            source_examples=len(window),
            record_source_examples=assign_source_counts(per_row, source_examples=len(window),
                                                        trainable_examples=len(tokenized)),
            epoch=epoch)


def iter_streaming_batches(source_factory: StreamingSourceFactory, tokenizer: Any, *, num_epochs: int | None,
                           dataset_text_field: str, max_sequence_length: int, pad_token_id: int,
                           assistant_only_loss: bool = False, last_assistant_only_loss: bool = False,
                           endprompt: EndPromptSettings | None = None, packing: bool = False,
                           packing_batch_size: int = 1000, retry_initial_delay: float = 1.0,
                           retry_max_delay: float = 60.0) -> Iterator[StreamingBatchEnvelope]:
    if not callable(source_factory):
        raise TypeError("source_factory must be callable")
    if max_sequence_length <= 0:
        raise ValueError("max_sequence_length must be positive")
    if packing_batch_size <= 0:
        raise ValueError("packing_batch_size must be positive")
    if num_epochs is not None and (type(num_epochs) is not int or num_epochs <= 0):
        raise ValueError("num_epochs must be a positive integer or None")
    assembler = WindowAssembler(
        Preprocessor(tokenizer, dataset_text_field, max_sequence_length, assistant_only_loss, last_assistant_only_loss,
                     endprompt),
        max_sequence_length=max_sequence_length, pad_token_id=pad_token_id, packing=packing,
        state_weights_from_mask=assistant_only_loss or last_assistant_only_loss)
    epochs = itertools.count() if num_epochs is None else range(num_epochs)
    for epoch in epochs:
        rows = iter(ReplayingReader(source_factory, epoch, initial_delay=retry_initial_delay, max_delay=retry_max_delay,
                                    digest_fields=(dataset_text_field, "tools", "chat_template_kwargs")))
        consumed = 0
        while True:
            window = list(islice(rows, packing_batch_size))
            if not window:
                break
            yield assembler.envelope(window, epoch=epoch, first_index=consumed)
            consumed += len(window)
        yield StreamingBatchEnvelope((), 0, (), epoch, is_epoch_end=True)       # explicit end-of-epoch marker
