"""Step plan and deterministic global batches over a materialised packed dataset.

Every rank builds the identical global batch and keeps its rows, so input semantics do not
depend on the mesh (src/causal_trainer/data/batching.py:18-143).  An epoch's order is
``np.random.default_rng(seed + epoch).shuffle`` of the row indices; resuming at optimizer step
``k`` recomputes ``(epoch, offset)`` from ``k`` alone.  Loss-weight precedence inside a batch:
explicit ``loss_weights`` > ``assistant_masks`` (when an assistant-only mode is on) >
``attention_mask``; weighted and unweighted rows cannot be mixed.
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass
from typing import Any, Callable, Iterable, Iterator, TypeVar

import numpy as np

MODEL_FIELDS = ("input_ids", "attention_mask", "position_ids", "segment_ids")
S = TypeVar("S")
T = TypeVar("T")


@dataclass(frozen=True)
class BatchPlan:
    examples: int
    global_micro_batch_size: int
    accumulation_steps: int
    steps_per_epoch: int
    total_steps: int

    @classmethod
    def create(cls, examples: int, global_micro_batch_size: int, accumulation_steps: int, epochs: float,
               max_steps: int) -> "BatchPlan":
        rows_per_step = global_micro_batch_size * accumulation_steps
        if examples < 1:
            raise ValueError("a batch plan needs at least one dataset row")
        whole_steps, leftover = divmod(examples, rows_per_step)
        if leftover:
            raise ValueError(f"{examples} dataset rows are not divisible by the {rows_per_step} rows one optimizer step "
                             f"consumes; pad with zero-loss rows first (pad_packed_arrays_to_batch_multiple)")
        steps = max_steps if max_steps > 0 else max(1, math.floor(whole_steps * epochs))
        return cls(examples, global_micro_batch_size, accumulation_steps, whole_steps, steps)

    @property
    def effective_batch_size(self) -> int:
        return self.global_micro_batch_size * self.accumulation_steps


def collate(dataset, indices: np.ndarray, assistant_only_loss: bool) -> dict[str, np.ndarray]:
    rows = [dataset[int(i)] for i in indices]
    for n, row in enumerate(rows):
        missing = [f for f in MODEL_FIELDS if f not in row]
        if missing:
            raise ValueError(f"dataset record {n} is missing model fields: {missing}")
    batch = {f: np.asarray([r[f] for r in rows], dtype=np.int32) for f in MODEL_FIELDS}
    if assistant_only_loss:
        absent = [n for n, r in enumerate(rows) if "assistant_masks" not in r]
        if absent:
            raise ValueError(f"assistant-masked loss dataset is missing assistant_masks for records {absent}")
        for n, r in enumerate(rows):
            if len(r["assistant_masks"]) != len(r["input_ids"]):
                raise ValueError(f"dataset record {n} has an assistant mask that is not aligned with input_ids")
    weighted = [n for n, r in enumerate(rows) if "loss_weights" in r]
    if weighted and len(weighted) != len(rows):
        raise ValueError("a batch cannot mix weighted and unweighted training records")
    if weighted:
        for n, r in enumerate(rows):
            if len(r["loss_weights"]) != len(r["input_ids"]):
                raise ValueError(f"dataset record {n} has loss_weights that are not aligned with input_ids")
        batch["loss_weights"] = np.asarray([r["loss_weights"] for r in rows], dtype=np.float32)
    elif assistant_only_loss:
        batch["loss_weights"] = np.asarray([r["assistant_masks"] for r in rows], dtype=np.float32)
    else:
        batch["loss_weights"] = batch["attention_mask"].astype(np.float32)
    if not np.isfinite(batch["loss_weights"]).all() or (batch["loss_weights"] < 0).any():
        raise ValueError("loss_weights must be finite and non-negative")
    for extra in ("attention_end", "prediction_targets", "prediction_weights"):
        if all(extra in r for r in rows):
            dt = np.float32 if extra == "prediction_weights" else np.int32
            batch[extra] = np.asarray([r[extra] for r in rows], dtype=dt)
    return batch


def iter_global_batches(dataset, plan: BatchPlan, *, assistant_only_loss: bool, shuffle: bool, seed: int,
                        start_step: int = 0) -> Iterator[dict[str, np.ndarray]]:
    if not 0 <= start_step <= plan.total_steps:
        raise ValueError(f"start_step must be in [0, {plan.total_steps}], got {start_step}")
    step = start_step
    epoch, within = divmod(start_step, plan.steps_per_epoch)
    size = plan.effective_batch_size
    while step < plan.total_steps:
        order = np.arange(plan.examples, dtype=np.int64)
        if shuffle:
            np.random.default_rng(seed + epoch).shuffle(order)
        for offset in range(within * size, plan.steps_per_epoch * size, size):
            if step >= plan.total_steps:
                return
            yield collate(dataset, order[offset:offset + size], assistant_only_loss)
            step += 1
        epoch += 1
        within = 0


def split_accumulation(batch: dict[str, Any], accumulation_steps: int) -> dict[str, Any]:
    """Reshapes ``[G*mb, ...]`` fields to ``[G, mb, ...]``."""
    out = {}
    for key, value in batch.items():
        if value.shape[0] % accumulation_steps:
            raise ValueError(f"batch field {key} cannot be split into {accumulation_steps} micro-batches")
        out[key] = value.reshape((accumulation_steps, -1, *value.shape[1:]))
    return out


def prefetch_map(values: Iterable[S], transform: Callable[[S], T], *, prefetch_batches: int) -> Iterator[T]:
    """Applies ``transform`` at most ``prefetch_batches`` items ahead of the consumer (synchronously).

    With 1, the active item plus one converted item are alive; with 0 conversion is just in
    time.  When ``transform`` starts asynchronous host-to-device copies from pinned memory the
    copy overlaps the consumer's work without a producer thread or an unbounded queue.
    """
    if prefetch_batches < 0:
        raise ValueError("prefetch_batches cannot be negative")
    source = iter(values)
    ready: deque[T] = deque()
    for _ in range(prefetch_batches + 1):
        try:
            ready.append(transform(next(source)))
        except StopIteration:
            break
    while ready:
        yield ready.popleft()
        try:
            ready.append(transform(next(source)))
        except StopIteration:
            pass
