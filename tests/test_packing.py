import pytest

from causal_trainer_dev_b200.data.packing import best_fit_decreasing, pack_examples, pad_examples


def ex(n, tok, **extra):
    return {"input_ids": [tok] * n, **extra}


def test_best_fit_rows_and_metadata():
    rows = pack_examples([ex(6, 1), ex(4, 2), ex(4, 3), ex(2, 4)], max_length=8, pad_token_id=99)
    assert [r["input_ids"] for r in rows] == [[1] * 6 + [4] * 2, [2] * 4 + [3] * 4]
    assert rows[0]["position_ids"] == [0, 1, 2, 3, 4, 5, 0, 1]
    assert rows[0]["segment_ids"] == [1] * 6 + [2] * 2
    assert rows[1]["segment_ids"] == [1] * 4 + [2] * 4


def test_windows_are_independent():
    rows = pack_examples([ex(6, 1), ex(6, 2), ex(2, 3), ex(2, 4)], max_length=8, pad_token_id=0, packing_batch_size=2)
    assert len(rows) == 3


def test_left_padding_keeps_fields_aligned():
    rows = pack_examples([ex(3, 5, assistant_masks=[0, 1, 1]), ex(2, 6, assistant_masks=[0, 1])], max_length=8,
                         pad_token_id=99)
    r = rows[0]
    assert r["input_ids"] == [99, 99, 99, 5, 5, 5, 6, 6]
    assert r["attention_mask"] == [0, 0, 0, 1, 1, 1, 1, 1]
    assert r["assistant_masks"] == [0, 0, 0, 0, 1, 1, 0, 1]
    assert r["position_ids"] == [0, 0, 0, 0, 1, 2, 0, 1]
    assert r["segment_ids"] == [0, 0, 0, 1, 1, 1, 2, 2]


def test_internal_mask_zero_starts_new_segment_and_truncation_is_joint():
    r = pad_examples([{"input_ids": [1, 2, 3, 4], "attention_mask": [1, 1, 0, 1]}], max_length=4, pad_token_id=0)[0]
    assert r["segment_ids"] == [1, 1, 0, 2] and r["position_ids"] == [0, 1, 0, 0]
    r = pack_examples([{"input_ids": list(range(10)), "labels": list(range(10, 20))}], max_length=4, pad_token_id=0)[0]
    assert r["input_ids"] == [0, 1, 2, 3] and r["labels"] == [10, 11, 12, 13]


def test_explicit_positions_and_weights_survive():
    rows = pack_examples([{"input_ids": [7, 8], "position_ids": [100, 101], "loss_weights": [1.0, 0.5]}],
                         max_length=4, pad_token_id=0)
    assert rows[0]["position_ids"] == [0, 0, 100, 101] and rows[0]["loss_weights"] == [0.0, 0.0, 1.0, 0.5]


def test_mixed_fields_and_oversize_are_errors():
    with pytest.raises(ValueError, match="same per-token fields"):
        pack_examples([ex(2, 1, labels=[1, 1]), ex(2, 2)], max_length=8, pad_token_id=0)
    with pytest.raises(ValueError, match="exceeds"):
        best_fit_decreasing([ex(9, 1)], max_length=8)


def test_bfd_matches_linear_scan_oracle():
    import random

    rng = random.Random(0)
    items = [ex(rng.randint(1, 60), i) for i in range(300)]
    fast = best_fit_decreasing(items, max_length=64)
    # quadratic statement of the same rule
    order = sorted(range(len(items)), key=lambda i: (-len(items[i]["input_ids"]), i))
    bins, used = [], []
    for i in order:
        n = len(items[i]["input_ids"])
        best, rem = None, None
        for b, u in enumerate(used):
            r = 64 - u - n
            if r >= 0 and (rem is None or r < rem):
                best, rem = b, r
        if best is None:
            bins.append([items[i]])
            used.append(n)
        else:
            bins[best].append(items[i])
            used[best] += n
    assert [[e["input_ids"][0] for e in b] for b in fast] == [[e["input_ids"][0] for e in b] for b in bins]
