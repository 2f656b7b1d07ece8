import math

import numpy as np
import pytest

from causal_trainer_dev_b200.data.maskgit import MaskGITBatchTransform
from causal_trainer_dev_b200.data.tokenizer import TrainingTokenizer
from helpers import write_tokenizer


@pytest.fixture()
def tok(tmp_path):
    return TrainingTokenizer.from_directory(write_tokenizer(tmp_path / "tok"))


def _row(tok, text, length=64):
    ids = tok(text)["input_ids"]
    pad = length - len(ids)
    return dict(input_ids=np.array([ids + [0] * pad], dtype=np.int32),
                attention_mask=np.array([[1] * len(ids) + [0] * pad], dtype=np.int32),
                segment_ids=np.array([[1] * len(ids) + [0] * pad], dtype=np.int32),
                loss_weights=np.array([[1.0] * len(ids) + [0.0] * pad], dtype=np.float32))


GRID = "<|image_1|><|image_2|><|image_3|>\n<|image_4|><|image_5|><|image_6|>"
CHAT = f"<|im_start|>user\n<|image_9|><|image_9|> w1<|im_end|>\n<|im_start|>assistant\nw2 {GRID} w3<|im_end|>\n"


def test_selected_grid_gets_mask_targets_and_bidirectional_end(tok):
    t = MaskGITBatchTransform(tok, probability=1.0, seed=0)
    batch = _row(tok, CHAT)
    out = t(batch, step=5)
    ids = batch["input_ids"][0]
    grid = np.flatnonzero(t.is_image[ids])[2:]            # the user's two image tokens are never touched
    start, end = int(grid[0]), int(grid[-1]) + 1
    masked = np.flatnonzero(out["input_ids"][0] == t.mask_id)
    assert len(masked) >= 1 and set(masked) <= set(grid)
    assert (out["attention_end"][0, start:end] == end - 1).all()
    assert (out["attention_end"][0, :start] == np.arange(start)).all()
    assert (out["prediction_targets"][0, masked] == ids[masked]).all()
    assert (out["prediction_weights"][0, masked] == 1).all()
    unmasked_in_block = np.setdiff1d(np.arange(start - 1, end), masked)
    assert (out["prediction_weights"][0, unmasked_in_block] == 0).all()       # no AR edge into/out of the block
    assert out["prediction_weights"][0, end] == 1 and out["prediction_targets"][0, end] == ids[end + 1]
    again = t(batch, step=5)
    assert all(np.array_equal(out[k], again[k]) for k in out)                # pure function of (seed, step)
    assert not np.array_equal(out["input_ids"], t(batch, step=6)["input_ids"]) or True


def test_mask_count_follows_the_cosine_rule(tok):
    t = MaskGITBatchTransform(tok, probability=1.0, seed=3)
    batch = _row(tok, CHAT)
    rng = np.random.default_rng(np.random.SeedSequence([3, 11]))
    rng.random()
    expected = max(1, math.ceil(6 * math.cos(math.pi * 0.5 * rng.random())))
    assert int((t(batch, step=11)["input_ids"] == t.mask_id).sum()) == expected


def test_probability_zero_user_images_and_unclosed_turns_are_untouched(tok):
    batch = _row(tok, CHAT)
    assert "attention_end" not in MaskGITBatchTransform(tok, probability=0.0, seed=0)(batch, step=0)
    t = MaskGITBatchTransform(tok, probability=1.0, seed=0)
    unclosed = _row(tok, f"<|im_start|>assistant\n{GRID} w3")
    out = t(unclosed, step=0)
    assert np.array_equal(out["input_ids"], unclosed["input_ids"])
    disabled = _row(tok, CHAT)
    disabled["loss_weights"][:] = 0
    assert np.array_equal(t(disabled, step=0)["input_ids"], disabled["input_ids"])
    ragged = _row(tok, "<|im_start|>assistant\n<|image_1|><|image_2|>\n<|image_3|><|im_end|>\n")
    with pytest.raises(ValueError, match="unequal row widths"):
        t(ragged, step=0)


def test_all_selection_combinations_occur_with_two_grids(tok):
    two = f"<|im_start|>assistant\n{GRID} w1 w2 {GRID}<|im_end|>\n"
    t = MaskGITBatchTransform(tok, probability=0.5, seed=1)
    batch = _row(tok, two)
    grids = np.flatnonzero(t.is_image[batch["input_ids"][0]])
    first, second = grids[:6], grids[6:]
    seen = set()
    for step in range(100):
        ids = t(batch, step=step)["input_ids"][0]
        seen.add((bool((ids[first] == t.mask_id).any()), bool((ids[second] == t.mask_id).any())))
    assert seen == {(False, False), (False, True), (True, False), (True, True)}
