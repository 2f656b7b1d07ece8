"""The replaying reader of streamed sources: what it hands on across repeated transient failures,
what it refuses, and the ledger it keeps.  ``time.sleep`` is patched out: only the order of events
is under test."""
import pytest

from causal_trainer_dev_b200.data import streaming as S

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402


class Source:
    """``factory(epoch)`` over fixed rows; the k-th opening fails (ConnectionError) before yielding
    row ``fail_at[k]`` when that entry is not None.  ``short[k]`` truncates the k-th opening."""

    def __init__(self, rows, fail_at=(), short=()):
        self.rows, self.fail_at, self.short, self.opened = rows, list(fail_at), dict(short), 0

    def __call__(self, epoch):
        k = self.opened
        self.opened += 1
        stop = self.fail_at[k] if k < len(self.fail_at) else None
        rows = self.rows[: self.short[k]] if k in self.short else self.rows

        def gen():
            for i, r in enumerate(rows):
                if stop is not None and i == stop:
                    raise ConnectionError(f"opening {k} lost at row {i}")
                yield r
        return gen()


@pytest.fixture(autouse=True)
def no_sleep(monkeypatch):
    monkeypatch.setattr("time.sleep", lambda s: None)


@settings(max_examples=50, deadline=None)
@given(n=st.integers(1, 12), fails=st.lists(st.integers(0, 11), max_size=5))
def test_every_row_is_handed_on_once_and_in_order_whatever_fails(n, fails):
    rows = [{"text": f"r{i}", "extra": i} for i in range(n)]
    src = Source(rows, fail_at=[f % n for f in fails])
    reader = S.ReplayingReader(src, 0, digest_fields=("text",))
    assert list(reader) == rows
    assert reader.delivered == n and src.opened <= len(fails) + 1


def test_a_reopened_source_that_ends_inside_the_known_prefix_is_reopened_again():
    rows = [{"text": f"r{i}"} for i in range(6)]
    src = Source(rows, fail_at=[4], short={1: 2})            # second opening has 2 rows where 4 were delivered
    assert list(S.iter_retrying_records(src, 0)) == rows and src.opened == 3


def test_digest_fields_limit_what_must_replay_identically():
    rows = [{"text": f"r{i}", "served_by": "a"} for i in range(5)]

    class Relabelled(Source):
        def __call__(self, epoch):
            first = self.opened == 0
            inner = super().__call__(epoch)
            return inner if first else ({**r, "served_by": "b"} for r in inner)

    got = list(S.iter_retrying_records(Relabelled(rows, fail_at=[3]), 0, digest_fields=("text",)))
    assert [r["text"] for r in got] == [r["text"] for r in rows]
    with pytest.raises(RuntimeError, match="prefix changed"):
        list(S.iter_retrying_records(Relabelled(rows, fail_at=[3]), 0))         # whole rows are compared


def test_argument_checks():
    with pytest.raises(TypeError):
        S.ReplayingReader([{"text": "x"}], 0)
    with pytest.raises(ValueError):
        S.ReplayingReader(lambda e: iter(()), -1)
    with pytest.raises(ValueError):
        S.ReplayingReader(lambda e: iter(()), True)
    with pytest.raises(ValueError):
        S.ReplayingReader(lambda e: iter(()), 0, digest_fields=())
    assert list(S.ReplayingReader(lambda e: iter(()), 3)) == []


def test_ledger_counts_and_hashes_length_prefixed_rows():
    a, b = S.PrefixLedger(None), S.PrefixLedger(None)
    a.record({"text": "ab"}), a.record({"text": "c"})
    b.record({"text": "a"}), b.record({"text": "bc"})
    assert a.count == b.count == 2
    a.skip_known_prefix(iter([{"text": "ab"}, {"text": "c"}, {"text": "more"}]))
    with pytest.raises(RuntimeError, match="prefix changed"):
        b.skip_known_prefix(iter([{"text": "ab"}, {"text": "c"}]))            # same bytes, different row bounds


def test_source_rows_dropped_by_preprocessing_are_charged_to_the_last_prepared_row():
    assert S.assign_source_counts([2, 1, 3], source_examples=9, trainable_examples=6) == (2, 1, 6)
    assert S.assign_source_counts([], source_examples=4, trainable_examples=0) == ()
    with pytest.raises(RuntimeError, match="provenance"):
        S.assign_source_counts([2, 2], source_examples=3, trainable_examples=4)
    with pytest.raises(RuntimeError, match="provenance"):
        S.assign_source_counts([2, 2], source_examples=9, trainable_examples=5)
