"""Materialised data pipeline: process shards, typed columns, tail padding
(contracts of the reference's tests/data/test_pipeline.py)."""
from itertools import pairwise

import numpy as np
import pytest

from causal_trainer_dev_b200.data.pipeline import (
    PackedArrayDataset,
    RecordList,
    contiguous_shard_bounds,
    packed_dataset_to_arrays,
    pad_packed_arrays_to_batch_multiple,
    select_process_shard,
)


def _canonical_columns(rows: int = 3, s: int = 4) -> dict[str, np.ndarray]:
    ids = np.arange(rows * s, dtype=np.int32).reshape(rows, s)
    return {
        "input_ids": ids, "attention_mask": np.ones_like(ids),
        "position_ids": np.broadcast_to(np.arange(s, dtype=np.int32), ids.shape).copy(),
        "segment_ids": np.ones_like(ids), "assistant_masks": np.ones_like(ids),
        "loss_weights": np.ones(ids.shape, dtype=np.float32),
    }


@pytest.mark.parametrize("size", [0, 1, 2, 7, 10])
@pytest.mark.parametrize("process_count", [1, 2, 3, 4, 12])
def test_contiguous_shards_cover_every_source_row_once(size, process_count):
    intervals = [contiguous_shard_bounds(size, p, process_count) for p in range(process_count)]
    assert [i for a, b in intervals for i in range(a, b)] == list(range(size))
    assert all(left[1] == right[0] for left, right in pairwise(intervals))
    sizes = [b - a for a, b in intervals]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        contiguous_shard_bounds(size, process_count, process_count)


def test_empty_process_shard_keeps_the_schema():
    source = RecordList([{"text": t} for t in "abc"], fingerprint="f")
    shard, start = select_process_shard(source, process_index=7, process_count=8)
    assert start == len(source) and len(shard) == 0 and shard.column_names == source.column_names
    shard, start = select_process_shard(source, process_index=1, process_count=2)
    assert start == 2 and [r["text"] for r in shard] == ["c"]
    same, start = select_process_shard(source, process_index=0, process_count=1)
    assert same is source and start == 0


def test_typed_columns_and_fixed_shapes_of_an_empty_shard():
    rows = [{"input_ids": [1, 2, 3], "attention_mask": [0, 1, 1], "position_ids": [0, 0, 1], "segment_ids": [0, 1, 1]}]
    cols = packed_dataset_to_arrays(rows, max_sequence_length=3)
    assert set(cols) == {"input_ids", "attention_mask", "position_ids", "segment_ids", "loss_weights"}
    assert all(v.shape == (1, 3) for v in cols.values())
    assert all(v.dtype == np.int32 for k, v in cols.items() if k != "loss_weights")
    np.testing.assert_array_equal(cols["loss_weights"], [[0.0, 1.0, 1.0]])      # normal loss: the attention mask
    masked = packed_dataset_to_arrays([{**rows[0], "assistant_masks": [0, 0, 1]}], max_sequence_length=3,
                                      last_assistant_only_loss=True)
    np.testing.assert_array_equal(masked["loss_weights"], [[0.0, 0.0, 1.0]])    # assistant modes: the assistant mask
    empty = packed_dataset_to_arrays([], max_sequence_length=5, assistant_only_loss=True, has_explicit_loss_weights=True)
    assert set(empty) == {"input_ids", "attention_mask", "position_ids", "segment_ids", "assistant_masks", "loss_weights"}
    assert all(v.shape == (0, 5) for v in empty.values()) and empty["loss_weights"].dtype == np.float32
    with pytest.raises(ValueError, match="has length 3, expected 4"):
        packed_dataset_to_arrays(rows, max_sequence_length=4)
    with pytest.raises(ValueError, match="missing field"):
        packed_dataset_to_arrays([{"input_ids": [1]}], max_sequence_length=1)


def test_tail_padding_keeps_every_real_row_and_adds_zero_loss_context():
    columns = _canonical_columns()
    dataset, dummy_rows = pad_packed_arrays_to_batch_multiple(columns, batch_multiple=4)
    assert dummy_rows == 1 and len(dataset) == 4 and dataset.real_rows == 3 and dataset.dummy_rows == 1
    for name, original in columns.items():
        assert dataset.columns[name] is original                 # no copy of the real rows
    dummy = dataset[-1]
    np.testing.assert_array_equal(dummy["attention_mask"], columns["attention_mask"][-1])
    np.testing.assert_array_equal(dummy["loss_weights"], np.zeros_like(dummy["loss_weights"]))
    np.testing.assert_array_equal(dummy["assistant_masks"], np.zeros_like(dummy["assistant_masks"]))
    exact, none = pad_packed_arrays_to_batch_multiple(columns, batch_multiple=3)
    assert none == 0 and len(exact) == 3


def test_real_rows_state_their_weights_once_dummies_exist():
    columns = {k: v for k, v in _canonical_columns().items() if k not in ("loss_weights", "assistant_masks")}
    columns["attention_mask"][0, 0] = 0
    dataset = PackedArrayDataset(columns, dummy_rows=1)
    np.testing.assert_array_equal(dataset[0]["loss_weights"], [0.0, 1.0, 1.0, 1.0])
    with pytest.raises(IndexError):
        dataset[4]


def test_datasets_without_a_trainable_target_are_rejected_not_dropped():
    empty = {name: value[:0] for name, value in _canonical_columns(rows=1).items()}
    with pytest.raises(ValueError, match="no trainable packed rows"):
        pad_packed_arrays_to_batch_multiple(empty, batch_multiple=8)
    columns = _canonical_columns(rows=2, s=4)
    columns["attention_mask"][0] = [0, 0, 0, 1]
    columns["segment_ids"][0] = [0, 0, 0, 1]
    columns["loss_weights"][0] = columns["attention_mask"][0]
    with pytest.raises(ValueError, match="row 0 has no positive-weight causal target.*will not silently drop it"):
        pad_packed_arrays_to_batch_multiple(columns, batch_multiple=2)


def test_rows_answer_column_questions_like_a_dataset():
    from causal_trainer_dev_b200.data.pipeline import RecordList
    from causal_trainer_dev_b200.data.preprocessing import RowTable

    rows = RowTable([{"input_ids": [1, 2]}, {"input_ids": [3]}])
    assert rows["input_ids"] == [[1, 2], [3]] and rows[1] == {"input_ids": [3]}
    assert rows.column_names == ["input_ids"] and rows.cache_files == [] and isinstance(rows[:1], RowTable)
    assert RowTable().column_names == [] and rows.features == {"input_ids": "int64"}
    assert RowTable([], ["input_ids", "loss_weights"]).features == {"input_ids": "int64", "loss_weights": "float32"}
    records = RecordList([{"text": "a"}, {"text": "b"}], "fp")
    assert records["text"] == ["a", "b"] and records.cache_files == []
