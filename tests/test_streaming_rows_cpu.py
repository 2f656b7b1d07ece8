"""Row encoding and the row queue of the streaming batcher: validation rules and FIFO behaviour
under growth, against a plain-list model."""
import numpy as np
import pytest

from causal_trainer_dev_b200.data.streaming_batching import RowQueue, encode_row

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402


def _record(n=6, **over):
    rec = {"input_ids": list(range(5, 5 + n)), "attention_mask": [1] * n, "segment_ids": [1] * n,
           "position_ids": list(range(n))}
    rec.update(over)
    return rec


def test_weights_come_from_the_explicit_column_then_the_assistant_mask_then_attention():
    plain = encode_row(_record(), assistant_only_loss=False)
    assert plain["loss_weights"].dtype == np.float32 and plain["loss_weights"].tolist() == [1.0] * 6
    assert all(plain[f].dtype == np.int32 for f in ("input_ids", "attention_mask", "segment_ids", "position_ids"))
    masked = encode_row(_record(assistant_masks=[0, 0, 1, 1, 0, 1]), assistant_only_loss=True)
    assert masked["loss_weights"].tolist() == [0, 0, 1, 1, 0, 1]
    explicit = encode_row(_record(assistant_masks=[0, 0, 1, 1, 0, 1], loss_weights=[0, 0, 0.5, 0, 0, 2.0]),
                          assistant_only_loss=True)
    assert explicit["loss_weights"].tolist() == [0, 0, 0.5, 0, 0, 2.0]
    ignored_mask = encode_row(_record(assistant_masks=[0, 0, 1, 1, 0, 1]), assistant_only_loss=False)
    assert ignored_mask["loss_weights"].tolist() == [1.0] * 6


@pytest.mark.parametrize("record,assistant,fragment", [
    ({k: v for k, v in _record().items() if k != "segment_ids"}, False, "missing model fields"),
    (_record(position_ids=[0, 1, 2]), False, "not aligned"),
    (_record(), True, "missing assistant_masks"),
    (_record(assistant_masks=[1, 1]), True, "assistant mask is not aligned"),
    (_record(loss_weights=[1.0] * 5), False, "loss_weights are not aligned"),
    (_record(loss_weights=[1, 1, float("nan"), 1, 1, 1]), False, "finite and non-negative"),
    (_record(loss_weights=[1, 1, -0.5, 1, 1, 1]), False, "finite and non-negative"),
])
def test_malformed_records_are_refused_with_the_reason(record, assistant, fragment):
    with pytest.raises(ValueError, match=fragment):
        encode_row(record, assistant_only_loss=assistant)


def test_a_row_needs_one_target_with_an_attended_predecessor_in_its_own_segment():
    # weight only on the first token of each document: a first token has no predecessor in its segment
    with pytest.raises(ValueError, match="no positive-weight causal target"):
        encode_row(_record(segment_ids=[1, 1, 1, 2, 2, 2], loss_weights=[1, 0, 0, 1, 0, 0]), assistant_only_loss=False)
    # the predecessor is padding
    with pytest.raises(ValueError, match="no positive-weight causal target"):
        encode_row(_record(attention_mask=[0, 1, 0, 0, 0, 0], segment_ids=[0, 1, 0, 0, 0, 0], loss_weights=[0, 1, 0, 0, 0, 0]),
                   assistant_only_loss=False)
    ok = encode_row(_record(segment_ids=[1, 1, 1, 2, 2, 2], loss_weights=[0, 0, 0, 0, 0, 1]), assistant_only_loss=False)
    assert ok["loss_weights"][-1] == 1


@settings(max_examples=60, deadline=None)
@given(ops=st.lists(st.one_of(st.tuples(st.just("push"), st.integers(0, 9)), st.tuples(st.just("pop"), st.integers(1, 5))),
                    min_size=1, max_size=80))
def test_row_queue_is_a_fifo_through_growth_and_compaction(ops):
    queue, model, serial = RowQueue(), [], 0
    for kind, arg in ops:
        if kind == "push":
            serial += 1
            row = encode_row(_record(4, input_ids=[serial] * 4), assistant_only_loss=False)
            queue.push(row, arg)
            model.append((serial, arg))
        else:
            n = min(arg, len(model))
            if n == 0:
                continue
            batch, charged = queue.pop(n)
            want, model = model[:n], model[n:]
            assert batch["input_ids"][:, 0].tolist() == [s for s, _ in want]
            assert charged == sum(c for _, c in want)
            assert batch["loss_weights"].dtype == np.float32 and batch["input_ids"].dtype == np.int32
        assert len(queue) == len(model)


def test_padding_a_short_batch_repeats_the_last_row_without_weight():
    queue = RowQueue()
    for s in (7, 8):
        queue.push(encode_row(_record(4, input_ids=[s] * 4), assistant_only_loss=False), 1)
    batch, charged = queue.pop(2, pad_to=4)
    assert charged == 2 and batch["input_ids"][:, 0].tolist() == [7, 8, 8, 8]
    assert batch["loss_weights"][:2].sum() == 8 and batch["loss_weights"][2:].sum() == 0
    assert (batch["attention_mask"][2:] == batch["attention_mask"][1]).all()
    with pytest.raises(ValueError, match="different lengths"):
        queue.push(encode_row(_record(4), assistant_only_loss=False), 1)
        queue.push(encode_row(_record(5), assistant_only_loss=False), 1)
