"""Step plan and deterministic global batches over a materialised packed dataset.

Every rank builds the identical global batch and keeps its rows, so input semantics do not
depend on the mesh (src/causal_trainer/data/batching.py:18-143).  An epoch's order is
``np.random.default_rng(seed + epoch).shuffle`` of the row indices; resuming at optimizer step
``k`` recomputes ``(epoch, offset)`` from ``k`` alone.  Loss-weight precedence inside a batch:
explicit ``loss_weights`` > ``assistant_masks`` (when an assistant-only mode is on) >
``attention_mask``; weighted and unweighted rows cannot be mixed.

Layout of this module: :class:`BatchPlan` is the arithmetic, :class:`StepSchedule` turns an
optimizer step into row indices, :func:`collate` turns row indices into typed arrays (column
gather when the dataset offers ``take``, row stacking otherwise), and :class:`Lookahead` is the
bounded prefetcher behind :func:`prefetch_map`.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Callable, Iterable, Iterator, Mapping, Sequence, TypeVar

import numpy as np

MODEL_FIELDS = ("input_ids", "attention_mask", "position_ids", "segment_ids")
# optional per-token fields a dataset may carry through to the step, with their array types
_PASS_THROUGH = {"attention_end": np.int32, "prediction_targets": np.int32, "prediction_weights": np.float32}
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


class StepSchedule:
    """Which dataset rows optimizer step ``k`` consumes: a pure function of ``(plan, seed, k)``.

    The permutation of an epoch is cached while consecutive steps stay inside it, so walking the
    steps in order shuffles once per epoch, and jumping to any step (a resume) costs one shuffle.
    """

    def __init__(self, plan: BatchPlan, *, shuffle: bool, seed: int):
        self.plan, self.shuffle, self.seed = plan, shuffle, seed
        self._epoch = -1
        self._order: np.ndarray | None = None

    def epoch_order(self, epoch: int) -> np.ndarray:
        if epoch != self._epoch:
            order = np.arange(self.plan.examples, dtype=np.int64)
            if self.shuffle:
                np.random.default_rng(self.seed + epoch).shuffle(order)
            self._epoch, self._order = epoch, order
        return self._order

    def rows(self, step: int) -> np.ndarray:
        epoch, within = divmod(step, self.plan.steps_per_epoch)
        size = self.plan.effective_batch_size
        return self.epoch_order(epoch)[within * size:(within + 1) * size]


def _stack(rows: Sequence[Mapping[str, Any]], field: str, dtype) -> np.ndarray:
    return np.asarray([r[field] for r in rows], dtype=dtype)


def _gather_rows(dataset, indices: np.ndarray) -> tuple[dict[str, np.ndarray], set[str] | None]:
    """Columns of the selected rows.  Returns ``(columns, None)`` for a column store, or the stacked
    rows of a row store together with the set of fields that only *some* rows carried."""
    take = getattr(dataset, "take", None)
    if take is not None:
        return dict(take(np.asarray(indices, dtype=np.int64))), None
    rows = [dataset[int(i)] for i in indices]
    for n, row in enumerate(rows):
        missing = [f for f in MODEL_FIELDS if f not in row]
        if missing:
            raise ValueError(f"dataset record {n} is missing model fields: {missing}")
    everywhere = set(rows[0]).intersection(*map(set, rows[1:])) if rows else set()
    somewhere = set().union(*map(set, rows)) if rows else set()
    width = {n: len(r["input_ids"]) for n, r in enumerate(rows)}
    for field, what in (("assistant_masks", "an assistant mask that is"), ("loss_weights", "loss_weights that are")):
        for n, r in enumerate(rows):
            if field in r and len(r[field]) != width[n]:
                raise ValueError(f"dataset record {n} has {what} not aligned with input_ids")
    columns: dict[str, np.ndarray] = {}
    for field in everywhere:
        if field in MODEL_FIELDS:
            columns[field] = _stack(rows, field, np.int32)
        elif field in ("loss_weights", "assistant_masks"):
            columns[field] = _stack(rows, field, np.float32)
        elif field in _PASS_THROUGH:
            columns[field] = _stack(rows, field, _PASS_THROUGH[field])
    return columns, somewhere - everywhere


def collate(dataset, indices: np.ndarray, assistant_only_loss: bool) -> dict[str, np.ndarray]:
    """The typed arrays of one global batch (``int32`` model fields, ``float32`` weights)."""
    columns, partial = _gather_rows(dataset, indices)
    absent = [f for f in MODEL_FIELDS if f not in columns]
    if absent:
        raise ValueError(f"dataset is missing model fields: {absent}")
    batch = {f: np.asarray(columns[f], dtype=np.int32) for f in MODEL_FIELDS}
    if partial and "loss_weights" in partial:
        raise ValueError("a batch cannot mix weighted and unweighted training records")
    if assistant_only_loss and "assistant_masks" not in columns:
        who = "" if partial is None else " for records " + str(
            [n for n, i in enumerate(indices) if "assistant_masks" not in dataset[int(i)]])
        raise ValueError("assistant-masked loss dataset is missing assistant_masks" + who)
    if "loss_weights" in columns:
        weights = columns["loss_weights"]
    elif assistant_only_loss:
        weights = columns["assistant_masks"]
    else:
        weights = batch["attention_mask"]
    weights = np.asarray(weights, dtype=np.float32)
    if weights.shape != batch["input_ids"].shape:
        raise ValueError("loss weights are not aligned with input_ids")
    if not np.isfinite(weights).all() or (weights < 0).any():
        raise ValueError("loss_weights must be finite and non-negative")
    batch["loss_weights"] = weights
    for field, dtype in _PASS_THROUGH.items():
        if field in columns:
            batch[field] = np.asarray(columns[field], dtype=dtype)
    return batch


def iter_global_batches(dataset, plan: BatchPlan, *, assistant_only_loss: bool, shuffle: bool, seed: int,
                        start_step: int = 0) -> Iterator[dict[str, np.ndarray]]:
    if not 0 <= start_step <= plan.total_steps:
        raise ValueError(f"start_step must be in [0, {plan.total_steps}], got {start_step}")
    schedule = StepSchedule(plan, shuffle=shuffle, seed=seed)
    for step in range(start_step, plan.total_steps):
        yield collate(dataset, schedule.rows(step), assistant_only_loss)


def attention_cost_per_row(segment_ids: np.ndarray, attention_end: np.ndarray | None = None) -> np.ndarray:
    """Visible (query, key) pairs of every row under segment-isolated causal attention (with the
    optional inclusive visibility end of MaskGIT blocks): what the row costs in the attention
    kernels.  Rows of equal length can differ several-fold: one long document against many short ones."""
    seg = np.asarray(segment_ids)
    rows, s = seg.shape
    idx = np.arange(s)[None, :]
    first = np.ones((rows, s), dtype=bool)
    first[:, 1:] = seg[:, 1:] != seg[:, :-1]
    start = np.maximum.accumulate(np.where(first, idx, 0), axis=1)
    lim = idx if attention_end is None else np.maximum(idx, np.asarray(attention_end))
    return np.where(seg != 0, lim - start + 1, 0).sum(axis=1).astype(np.float64)


def longest_document(segment_ids: np.ndarray) -> int:
    """Tokens of the longest run of one non-zero segment id in any row: the longest document the
    rows hold.  A block-sparse attention whose every document has no more blocks than a query may
    select is exactly dense attention, which the engine then runs without the routing passes."""
    seg = np.asarray(segment_ids)
    if seg.size == 0:
        return 0
    rows, s = seg.shape
    idx = np.arange(s)[None, :]
    first = np.ones((rows, s), dtype=bool)
    first[:, 1:] = seg[:, 1:] != seg[:, :-1]
    start = np.maximum.accumulate(np.where(first, idx, 0), axis=1)
    return int(np.where(seg != 0, idx - start + 1, 0).max())


def balanced_row_assignment(costs: np.ndarray, ranks: int) -> np.ndarray:
    """``[ranks, rows / ranks]`` row indices: every rank gets the same number of rows and, as nearly
    as a greedy pass can make it, the same total cost (largest rows first, each to the least loaded
    rank that still has room).  The global batch and therefore the gradient are unchanged; only the
    time the slowest rank needs for its share goes down.  Deterministic: ties go to the lower rank
    and the lower row index, and rows keep their batch order inside a rank."""
    costs = np.asarray(costs, dtype=np.float64)
    n = costs.shape[0]
    if ranks < 1 or n % ranks:
        raise ValueError(f"{n} rows cannot be split evenly over {ranks} ranks")
    per = n // ranks
    load = np.zeros(ranks)
    taken: list[list[int]] = [[] for _ in range(ranks)]
    for row in np.argsort(-costs, kind="stable"):
        open_ranks = [r for r in range(ranks) if len(taken[r]) < per]
        r = min(open_ranks, key=lambda x: (load[x], x))
        taken[r].append(int(row))
        load[r] += costs[row]
    return np.asarray([sorted(t) for t in taken], dtype=np.int64).reshape(ranks, per)


def split_accumulation(batch: dict[str, Any], accumulation_steps: int) -> dict[str, Any]:
    """Reshapes ``[G*mb, ...]`` fields to ``[G, mb, ...]``."""
    bad = [k for k, v in batch.items() if v.shape[0] % accumulation_steps]
    if bad:
        raise ValueError(f"batch field {bad[0]} cannot be split into {accumulation_steps} micro-batches")
    return {k: v.reshape(accumulation_steps, v.shape[0] // accumulation_steps, *v.shape[1:]) for k, v in batch.items()}


class Lookahead(Iterator[T]):
    """Iterator that keeps ``depth`` already-transformed items queued behind the one it hands out.

    Nothing runs concurrently here: ``transform`` is called on the consumer's thread, once per
    request for the next item (and ``depth + 1`` times up front).  It pays off when ``transform`` only
    *starts* work, e.g. asynchronous host-to-device copies from pinned memory, which then overlap
    the consumer's step without a producer thread or an unbounded queue.
    """

    def __init__(self, source: Iterable[S], transform: Callable[[S], T], depth: int):
        self._source = iter(source)
        self._transform = transform
        self._queue: list[T] = []
        self._primed = False
        self._depth = depth

    def _pull(self) -> None:
        try:
            self._queue.append(self._transform(next(self._source)))
        except StopIteration:
            pass

    def __next__(self) -> T:
        if self._primed:
            self._pull()                      # refill the place of the item handed out last time
        else:
            if self._depth < 0:               # reported where a generator would report it: on first use
                raise ValueError("prefetch_batches cannot be negative")
            self._primed = True
            for _ in range(self._depth + 1):
                self._pull()
        if not self._queue:
            raise StopIteration
        return self._queue.pop(0)


def prefetch_map(values: Iterable[S], transform: Callable[[S], T], *, prefetch_batches: int) -> Iterator[T]:
    """Applies ``transform`` at most ``prefetch_batches`` items ahead of the consumer (synchronously):
    with 1, the active item plus one converted item are alive; with 0 conversion is just in time."""
    return Lookahead(values, transform, prefetch_batches)
