"""Segment-isolated fixed-length packing (deterministic best-fit decreasing).

Behaviour kept from the reference (src/causal_trainer/data/packing.py:105-395):

* examples are packed in independent windows of ``packing_batch_size``; inside a window they
  are taken longest first (ties by arrival order) and each goes to the open row that it
  fills most tightly (ties by row age);
* nothing is inserted between documents; isolation comes from regenerated one-based
  ``segment_ids`` (a masked token inside an example starts a new segment) and positions
  restart per segment unless the example carries explicit ``position_ids``;
* rows are padded on the left by default: ``input_ids`` with the pad id, ``loss_weights``
  with 0.0, every other per-token field with 0;
* all examples of a window must carry the same per-token fields.

The implementation keeps the open rows in a sorted free-space index, so a window of n
examples packs in O(n log n) instead of scanning every row for every example.
"""
from __future__ import annotations

import bisect
import math
from itertools import islice
from typing import Any, Iterable, Iterator, Mapping, Sequence

Scalar = int | float
PackedExample = dict[str, list[Scalar]]

_FLOAT_FIELDS = frozenset({"loss_weights"})
_STRICT_FIELDS = frozenset({"attention_mask", "position_ids", "segment_ids", "loss_weights", "labels"})
_ASSISTANT_FIELDS = ("assistant_masks", "assistant_mask", "assistant_tokens_mask")


def _to_list(value: Any, name: str) -> list:
    if hasattr(value, "tolist"):
        value = value.tolist()
    if isinstance(value, tuple):
        value = list(value)
    if not isinstance(value, list) or (value and isinstance(value[0], (list, tuple))):
        raise ValueError(f"Per-token field {name!r} must be a one-dimensional sequence.")
    return value


def _column(value: Any, name: str) -> list[Scalar]:
    raw = _to_list(value, name)
    if name in _FLOAT_FIELDS:
        try:
            out = list(map(float, raw))
        except (TypeError, ValueError) as exc:
            raise ValueError(f"Per-token field {name!r} must contain numbers.") from exc
        if not all(map(math.isfinite, out)):
            raise ValueError(f"Per-token field {name!r} must contain only finite numbers.")
        return out
    try:
        return list(map(int, raw))
    except (TypeError, ValueError) as exc:
        raise ValueError(f"Per-token field {name!r} must contain integers.") from exc


def _binary(values: list) -> bool:
    return set(values) <= {0, 1}


def normalize_example(example: Mapping[str, Any], max_length: int) -> PackedExample:
    """Validates one example and truncates every per-token field to ``max_length`` together."""
    if "input_ids" not in example:
        raise ValueError("Every example must contain input_ids.")
    full = _column(example["input_ids"], "input_ids")
    if not full[:max_length]:
        raise ValueError("Cannot pack an empty input_ids sequence.")
    out: PackedExample = {"input_ids": full[:max_length]}
    for key, value in example.items():
        if key == "input_ids" or isinstance(value, (str, bytes, Mapping)):
            continue
        try:
            col = _column(value, key)
        except ValueError:
            if key in _STRICT_FIELDS or key.endswith(("_mask", "_masks")):
                raise
            continue  # not a per-token field (metadata): dropped
        if len(col) != len(full):
            raise ValueError(f"Per-token field {key!r} has length {len(col)}, expected {len(full)}.")
        out[key] = col[:max_length]
    out.setdefault("attention_mask", [1] * len(out["input_ids"]))
    if not _binary(out["attention_mask"]):
        raise ValueError("attention_mask must contain only binary 0/1 values.")
    for name in _ASSISTANT_FIELDS:
        if name in out and not _binary(out[name]):
            raise ValueError(f"{name} must contain only binary 0/1 values.")
    if "position_ids" in out and min(out["position_ids"]) < 0:
        raise ValueError("position_ids must be non-negative.")
    if "loss_weights" in out and min(out["loss_weights"]) < 0.0:
        raise ValueError("loss_weights must be non-negative.")
    return out


def _check_same_fields(examples: Sequence[PackedExample]) -> tuple[str, ...]:
    fields = tuple(examples[0])
    want = set(fields)
    for i, ex in enumerate(examples[1:], start=1):
        if set(ex) != want:
            raise ValueError(
                "All examples in a packing batch must have the same per-token fields; "
                f"example {i} is missing {sorted(want - set(ex))} and adds {sorted(set(ex) - want)}."
            )
    return fields


def best_fit_decreasing(examples: Sequence[PackedExample], *, max_length: int) -> list[list[PackedExample]]:
    """Rows of examples; order inside a row is placement order."""
    if max_length <= 0:
        raise ValueError("max_length must be positive.")
    order = sorted(range(len(examples)), key=lambda i: (-len(examples[i]["input_ids"]), i))
    rows: list[list[PackedExample]] = []
    free: list[tuple[int, int]] = []  # sorted (free space, row index)
    for i in order:
        n = len(examples[i]["input_ids"])
        if n > max_length:
            raise ValueError(f"Sequence length {n} exceeds packing max_length {max_length}.")
        at = bisect.bisect_left(free, (n, -1))
        if at == len(free):
            rows.append([examples[i]])
            bisect.insort(free, (max_length - n, len(rows) - 1))
        else:
            space, row = free.pop(at)
            rows[row].append(examples[i])
            bisect.insort(free, (space - n, row))
    return rows


def run_metadata(attention_mask: Sequence[int], first_segment: int = 0) -> tuple[list[int], list[int], int]:
    """Positions and one-based segment ids of the contiguous valid runs of one example."""
    n = len(attention_mask)
    if n and type(attention_mask) is list and attention_mask.count(1) == n:
        return list(range(n)), [first_segment + 1] * n, first_segment + 1     # one unbroken run
    positions, segments = [], []
    seg, cur, pos = first_segment, 0, 0
    for m in attention_mask:
        if int(m) == 1:
            if cur == 0:
                seg += 1
                cur, pos = seg, 0
            positions.append(pos)
            segments.append(cur)
            pos += 1
        else:
            positions.append(0)
            segments.append(0)
            cur, pos = 0, 0
    return positions, segments, seg


def _pad_value(field: str, pad_token_id: int) -> Scalar:
    if field == "input_ids":
        return int(pad_token_id)
    return 0.0 if field in _FLOAT_FIELDS else 0


def pad_example(example: Mapping[str, Sequence[Scalar]], *, max_length: int, pad_token_id: int,
                padding_side: str = "left") -> PackedExample:
    if max_length <= 0:
        raise ValueError("max_length must be positive.")
    if padding_side not in ("left", "right"):
        raise ValueError("padding_side must be either 'left' or 'right'.")
    if "input_ids" not in example:
        raise ValueError("example must contain input_ids.")
    return _pad_columns({k: _column(v, k) for k, v in example.items()}, max_length, pad_token_id, padding_side)


def _pad_columns(cols: Mapping[str, list], max_length: int, pad_token_id: int, padding_side: str) -> PackedExample:
    """``pad_example`` on columns that are already typed lists."""
    n = len(cols["input_ids"])
    if n > max_length:
        raise ValueError(f"Packed sequence length {n} exceeds max_length {max_length}.")
    out: PackedExample = {}
    for k, col in cols.items():
        if len(col) != n:
            raise ValueError(f"Packed field {k!r} is not aligned with input_ids.")
        fill = [_pad_value(k, pad_token_id)] * (max_length - n)
        out[k] = fill + col if padding_side == "left" else col + fill
    return out


def _join_row(row: Sequence[PackedExample], fields: Sequence[str], max_length: int, pad_token_id: int,
              padding_side: str) -> PackedExample:
    joined: PackedExample = {f: [] for f in fields}
    keep_positions = "position_ids" in fields
    positions: list[int] = []
    segments: list[int] = []
    last = 0
    for ex in row:
        for f in fields:
            joined[f].extend(ex[f])
        pos, seg, last = run_metadata(ex["attention_mask"], last)
        segments.extend(seg)
        if not keep_positions:
            positions.extend(pos)
    if not keep_positions:
        joined["position_ids"] = positions
    joined["segment_ids"] = segments
    if padding_side not in ("left", "right"):
        raise ValueError("padding_side must be either 'left' or 'right'.")
    return _pad_columns(joined, max_length, pad_token_id, padding_side)


def _windows(items: Iterable[Any], size: int) -> Iterator[list[Any]]:
    it = iter(items)
    while chunk := list(islice(it, size)):
        yield chunk


def pack_examples(examples: Iterable[Mapping[str, Any]], *, max_length: int, pad_token_id: int,
                  packing_batch_size: int = 1000, padding_side: str = "left") -> list[PackedExample]:
    if max_length <= 0:
        raise ValueError("max_length must be positive.")
    if packing_batch_size <= 0:
        raise ValueError("packing_batch_size must be positive.")
    out: list[PackedExample] = []
    for window in _windows(examples, packing_batch_size):
        normalized = [normalize_example(ex, max_length) for ex in window]
        fields = tuple(f for f in _check_same_fields(normalized) if f != "segment_ids")
        for row in best_fit_decreasing(normalized, max_length=max_length):
            out.append(_join_row(row, fields, max_length, pad_token_id, padding_side))
    return out


def pad_examples(examples: Iterable[Mapping[str, Any]], *, max_length: int, pad_token_id: int,
                 padding_side: str = "left") -> list[PackedExample]:
    """Truncates and pads each example on its own (``--packing False``)."""
    out: list[PackedExample] = []
    for ex in examples:
        norm = normalize_example(ex, max_length)
        pos, seg, _ = run_metadata(norm["attention_mask"])
        norm.setdefault("position_ids", pos)
        norm["segment_ids"] = seg
        out.append(pad_example(norm, max_length=max_length, pad_token_id=pad_token_id, padding_side=padding_side))
    return out


def pack_dataset(dataset: Any, *, max_length: int, pad_token_id: int, packing_batch_size: int = 1000,
                 padding_side: str = "left", num_proc: int | None = None) -> Any:
    """Packs a ``datasets.Dataset``-like object one map batch at a time, or any iterable."""
    mapper = getattr(dataset, "map", None)
    kw = dict(max_length=max_length, pad_token_id=pad_token_id, packing_batch_size=packing_batch_size,
              padding_side=padding_side)
    if not callable(mapper):
        return pack_examples(dataset, **kw)

    def on_batch(batch: Mapping[str, Sequence[Any]]) -> dict[str, list[list[Scalar]]]:
        if "input_ids" not in batch:
            raise ValueError("Dataset batch must contain input_ids.")
        rows = [{k: v[i] for k, v in batch.items()} for i in range(len(batch["input_ids"]))]
        packed = pack_examples(rows, **kw)
        return {k: [r[k] for r in packed] for k in packed[0]} if packed else {}

    map_kw: dict[str, Any] = {"batched": True, "batch_size": packing_batch_size}
    if getattr(dataset, "column_names", None) is not None:
        map_kw["remove_columns"] = list(dataset.column_names)
    if num_proc is not None:
        map_kw["num_proc"] = num_proc
    return mapper(on_batch, **map_kw)
