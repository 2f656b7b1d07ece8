import numpy as np
import pytest

from causal_trainer_dev_b200.data.batching import BatchPlan, collate, iter_global_batches, prefetch_map


def test_plan_arithmetic():
    p = BatchPlan.create(128, 16, 2, 1.0, -1)
    assert p.effective_batch_size == 32 and p.steps_per_epoch == 4 and p.total_steps == 4
    assert BatchPlan.create(128, 16, 2, 1.0, 9).total_steps == 9
    with pytest.raises(ValueError, match="divisible"):
        BatchPlan.create(100, 16, 2, 1.0, -1)


def _dataset(n, s=4):
    return [dict(input_ids=[i] * s, attention_mask=[1] * s, position_ids=list(range(s)), segment_ids=[1] * s)
            for i in range(n)]


def test_resume_reproduces_the_tail():
    ds = _dataset(16)
    plan = BatchPlan.create(16, 2, 1, 2.0, -1)
    kw = dict(assistant_only_loss=False, shuffle=True, seed=3)
    full = [b["input_ids"][:, 0].tolist() for b in iter_global_batches(ds, plan, **kw)]
    tail = [b["input_ids"][:, 0].tolist() for b in iter_global_batches(ds, plan, start_step=7, **kw)]
    assert len(full) == 16 and tail == full[7:]
    assert sorted(sum(full[:8], [])) == list(range(16))  # one epoch covers every row once


def test_loss_weight_precedence():
    base = dict(input_ids=[1, 2], attention_mask=[1, 1], position_ids=[0, 1], segment_ids=[1, 1])
    plain = collate([base], np.array([0]), False)
    assert plain["loss_weights"].tolist() == [[1.0, 1.0]]
    masked = collate([dict(base, assistant_masks=[0, 1])], np.array([0]), True)
    assert masked["loss_weights"].tolist() == [[0.0, 1.0]]
    explicit = collate([dict(base, assistant_masks=[0, 1], loss_weights=[0.5, 0.25])], np.array([0]), True)
    assert explicit["loss_weights"].tolist() == [[0.5, 0.25]]
    with pytest.raises(ValueError, match="mix weighted"):
        collate([dict(base, loss_weights=[1.0, 1.0]), base], np.array([0, 1]), False)
    with pytest.raises(ValueError, match="missing assistant_masks"):
        collate([base], np.array([0]), True)


def test_prefetch_converts_exactly_one_ahead():
    seen = []

    def f(x):
        seen.append(x)
        return x * 10

    it = prefetch_map(range(4), f, prefetch_batches=1)
    assert next(it) == 0 and seen == [0, 1]
    assert next(it) == 10 and seen == [0, 1, 2]
    assert list(it) == [20, 30] and seen == [0, 1, 2, 3]


def test_rows_are_dealt_to_ranks_by_attention_cost():
    from causal_trainer_dev_b200.data.batching import attention_cost_per_row, balanced_row_assignment
    from causal_trainer_dev_b200.data.synthetic import pretraining_rows

    data = pretraining_rows(32, 1024, 5000, eos_token_id=2, pad_token_id=0, median_len=150.0, sigma=1.0, min_len=8, seed=4)
    cost = attention_cost_per_row(data["segment_ids"])
    # one document of n tokens costs n (n + 1) / 2 pairs; padding costs nothing
    seg = np.array([[1, 1, 1, 2, 2, 0, 0, 0]])
    assert attention_cost_per_row(seg).tolist() == [6 + 3]
    end = np.array([[0, 1, 2, 4, 4, 5, 6, 7]])               # the second document is bidirectional
    assert attention_cost_per_row(seg, end).tolist() == [6 + 4]
    for ranks in (2, 4, 8):
        rows = balanced_row_assignment(cost, ranks)
        assert rows.shape == (ranks, 32 // ranks) and sorted(rows.reshape(-1).tolist()) == list(range(32))
        assert (np.diff(rows, axis=1) > 0).all()                                  # batch order kept inside a rank
        contiguous = cost.reshape(ranks, -1).sum(1)
        dealt = cost[rows].sum(1)
        assert dealt.max() / dealt.mean() < 1.06 <= contiguous.max() / contiguous.mean()
        assert np.array_equal(rows, balanced_row_assignment(cost, ranks))         # deterministic
    with pytest.raises(ValueError, match="evenly"):
        balanced_row_assignment(cost[:30], 4)


def test_longest_document_and_the_dense_shortcut_of_block_sparse_layers():
    from causal_trainer_dev_b200.data.batching import longest_document
    from causal_trainer_dev_b200.models.config import ModelConfig
    from causal_trainer_dev_b200.models.moba import AttentionOptions
    from causal_trainer_dev_b200.training.engine import EngineOptions, LayerwiseEngine

    seg = np.array([[1, 1, 1, 2, 2, 0, 0, 0],
                    [1, 2, 2, 2, 2, 2, 1, 0]], dtype=np.int32)
    assert longest_document(seg) == 5
    assert longest_document(np.zeros((2, 8), dtype=np.int32)) == 0
    assert longest_document(np.zeros((0, 8), dtype=np.int32)) == 0

    cfg = ModelConfig(vocab_size=64, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=1,
                      num_key_value_heads=1, head_dim=64)
    ao = AttentionOptions(method="moba", moba_block_size=128, moba_top_k=2)
    engine = LayerwiseEngine.__new__(LayerwiseEngine)        # only the dispatch rule is exercised
    engine.cfg, engine.options = cfg, EngineOptions(attention_options=ao)
    assert engine._uses_moba(0, 1024)                        # 8 blocks, a query keeps 2
    assert engine._uses_moba(0, 1024, longest=257)           # a document of 3 blocks
    assert not engine._uses_moba(0, 1024, longest=256)       # 2 blocks: nothing can be dropped
    assert not engine._uses_moba(0, 256)
    engine.options = EngineOptions(attention_options=ao, moba_dense_shortcut=False)
    assert engine._uses_moba(0, 1024, longest=256)
