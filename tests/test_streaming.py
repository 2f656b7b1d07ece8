import pytest

from causal_trainer_dev_b200.data import streaming as S
from causal_trainer_dev_b200.data import streaming_batching as SB
from causal_trainer_dev_b200.data.tokenizer import TrainingTokenizer
from helpers import write_tokenizer


class Flaky:
    """Source that raises a connection error once after ``fail_after`` rows."""

    def __init__(self, rows, fail_after, changed_prefix=False):
        self.rows, self.fail_after, self.opened, self.changed = rows, fail_after, 0, changed_prefix

    def __call__(self, epoch):
        self.opened += 1
        first = self.opened == 1

        def gen():
            for i, r in enumerate(self.rows):
                if first and i == self.fail_after:
                    raise ConnectionError("boom")
                yield ({"text": "w39"} if (self.changed and not first and i == 0) else r)
        return gen()


def test_reconnect_replays_prefix_without_duplicates(monkeypatch):
    monkeypatch.setattr("time.sleep", lambda s: None)
    rows = [{"text": f"w{i}"} for i in range(6)]
    src = Flaky(rows, 3)
    assert list(S.iter_retrying_records(src, 0, digest_fields=("text",))) == rows and src.opened == 2


def test_changed_prefix_is_rejected(monkeypatch):
    monkeypatch.setattr("time.sleep", lambda s: None)
    rows = [{"text": f"w{i}"} for i in range(6)]
    with pytest.raises(RuntimeError, match="prefix changed"):
        list(S.iter_retrying_records(Flaky(rows, 3, changed_prefix=True), 0, digest_fields=("text",)))


def test_non_network_errors_fail_fast():
    def factory(epoch):
        def gen():
            yield {"text": "w1"}
            raise KeyError("bad row")
        return gen()
    with pytest.raises(KeyError):
        list(S.iter_retrying_records(factory, 0))


def _envelopes(tmp_path, n_rows=10, epochs=1, window=4):
    tok = TrainingTokenizer.from_directory(write_tokenizer(tmp_path / "tok"))
    rows = [{"text": " ".join(f"w{(i + j) % 40}" for j in range(3 + i % 4))} for i in range(n_rows)]
    return list(S.iter_streaming_batches(lambda e: iter(rows), tok, num_epochs=epochs, dataset_text_field="text",
                                         max_sequence_length=8, pad_token_id=0, packing=True, packing_batch_size=window))


def test_envelopes_account_for_every_source_row(tmp_path):
    env = _envelopes(tmp_path)
    assert env[-1].is_epoch_end and not env[-1].records
    assert sum(e.source_examples for e in env) == 10
    for e in env[:-1]:
        assert sum(e.record_source_examples) == e.source_examples and len(e.records) <= 4
        assert all("loss_weights" in r for r in e.records)


def test_grouping_pads_epoch_tail_and_resume_verifies_digest(tmp_path):
    env = _envelopes(tmp_path, epochs=2)
    plan = SB.StreamingBatchPlan.create(10, 2, 1, 2, -1)
    batches = list(SB.iter_streaming_global_batches(env, plan, assistant_only_loss=False))
    assert sum(b.is_epoch_end for b in batches) == 2
    assert batches[-1].source_examples_seen == 20
    for b in batches:
        assert b.data["input_ids"].shape == (2, 8)
    tail = [b for b in batches if b.is_epoch_end][0]
    if (tail.data["loss_weights"][-1] == 0).all():      # padded with a zero-loss copy of the last real row
        assert (tail.data["input_ids"][-1] == tail.data["input_ids"][-2]).all()
    k = 3
    resumed = list(SB.iter_streaming_global_batches(
        env, plan, assistant_only_loss=False, start_step=k,
        expected_source_examples_before=batches[k - 1].source_examples_seen,
        expected_stream_digest_before=batches[k - 1].stream_digest))
    assert [b.stream_digest for b in resumed] == [b.stream_digest for b in batches[k:]]
    with pytest.raises(RuntimeError, match="different training batches"):
        list(SB.iter_streaming_global_batches(env, plan, assistant_only_loss=False, start_step=k,
                                              expected_stream_digest_before="0" * 64))
    # resume exactly at end of stream is still verified
    end = list(SB.iter_streaming_global_batches(
        env, plan, assistant_only_loss=False, start_step=len(batches),
        expected_source_examples_before=20, expected_stream_digest_before=batches[-1].stream_digest))
    assert end == []


def test_missing_epoch_marker_and_empty_epoch_are_errors(tmp_path):
    env = _envelopes(tmp_path)
    plan = SB.StreamingBatchPlan.create(None, 2, 1, 1, -1)
    with pytest.raises(ValueError, match="without an epoch-end"):
        list(SB.iter_streaming_global_batches(env[:-1], plan, assistant_only_loss=False))
    empty = [S.StreamingBatchEnvelope((), 3, (), 0), S.StreamingBatchEnvelope((), 0, (), 0, is_epoch_end=True)]
    with pytest.raises(ValueError, match="no trainable records"):
        list(SB.iter_streaming_global_batches(empty, plan, assistant_only_loss=False))


def test_plan_semantics():
    p = SB.StreamingBatchPlan.create(100, 4, 2, 3, -1)
    assert p.steps_per_epoch == 13 and p.total_steps == SB.UNKNOWN_TOTAL_STEPS and not p.has_exact_step_limit
    q = SB.StreamingBatchPlan.create(None, 4, 2, 0, 50)
    assert q.total_steps == 50 and q.epochs is None and q.has_exact_step_limit
