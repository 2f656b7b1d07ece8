"""Property tests (hypothesis) of host-side pieces whose contracts are easy to state and easy to
break at the edges: packing, the per-row attention cost and the dealing of rows to ranks, the
safetensors writer / reader pair, the learning-rate schedule."""
import math

import numpy as np
import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402

FAST = settings(max_examples=60, deadline=None)


# ------------------------------------------------------------------ packing
@FAST
@given(lengths=st.lists(st.integers(1, 64), min_size=1, max_size=40), max_length=st.integers(64, 96),
       side=st.sampled_from(["left", "right"]))
def test_packing_keeps_every_token_once_and_documents_apart(lengths, max_length, side):
    from causal_trainer_dev_b200.data.packing import pack_examples

    examples = []
    token = 10
    for n in lengths:                                   # distinct token ids: every token is traceable
        examples.append({"input_ids": list(range(token, token + n)), "attention_mask": [1] * n})
        token += n
    rows = pack_examples(examples, max_length=max_length, pad_token_id=0, padding_side=side)
    seen = []
    for row in rows:
        ids, mask, seg, pos = (np.asarray(row[k]) for k in ("input_ids", "attention_mask", "segment_ids", "position_ids"))
        assert len(ids) == max_length
        assert ((mask == 0) == (seg == 0)).all() and (ids[mask == 0] == 0).all()
        real = ids[mask == 1]
        seen.extend(real.tolist())
        # a document is one run of its segment id, its tokens consecutive and its positions 0..n-1
        for s in set(seg[seg != 0].tolist()):
            where = np.flatnonzero(seg == s)
            assert (np.diff(where) == 1).all()
            assert (np.diff(ids[where]) == 1).all()
            assert pos[where].tolist() == list(range(len(where)))
        pad = np.flatnonzero(mask == 0)                 # padding sits on one side only
        if len(pad):
            assert (pad == np.arange(len(pad))).all() if side == "left" else (pad == np.arange(max_length - len(pad), max_length)).all()
    assert sorted(seen) == list(range(10, token))
    # best-fit decreasing never needs more rows than one document per row, nor fewer than the volume bound
    assert math.ceil(sum(lengths) / max_length) <= len(rows) <= len(lengths)


# ------------------------------------------------------------------ attention cost, dealing rows
def _segments(draw_lengths, seq):
    seg = np.zeros(seq, dtype=np.int32)
    at = 0
    for i, n in enumerate(draw_lengths):
        n = min(n, seq - at)
        if n <= 0:
            break
        seg[at:at + n] = i + 1
        at += n
    return seg


@FAST
@given(rows=st.lists(st.lists(st.integers(1, 24), min_size=0, max_size=6), min_size=1, max_size=6))
def test_attention_cost_and_longest_document_match_a_loop(rows):
    from causal_trainer_dev_b200.data.batching import attention_cost_per_row, longest_document

    seq = 48
    seg = np.stack([_segments(r, seq) for r in rows])
    cost = attention_cost_per_row(seg)
    want_cost, want_longest = [], 0
    for r in seg:
        total, run, prev = 0, 0, 0
        for s in r.tolist():
            run = run + 1 if (s != 0 and s == prev) else (1 if s != 0 else 0)
            prev = s
            total += run                                # a token sees its own document up to itself
            want_longest = max(want_longest, run)
        want_cost.append(total)
    assert cost.tolist() == want_cost
    assert longest_document(seg) == want_longest


@FAST
@given(costs=st.lists(st.floats(0, 1e6, allow_nan=False), min_size=1, max_size=12), ranks=st.integers(1, 4),
       per=st.integers(1, 4))
def test_balanced_assignment_is_a_partition_and_never_worse_than_slices(costs, ranks, per):
    from causal_trainer_dev_b200.data.batching import balanced_row_assignment

    costs = np.asarray((costs * (ranks * per))[: ranks * per])
    rows = balanced_row_assignment(costs, ranks)
    assert rows.shape == (ranks, per)
    assert sorted(rows.reshape(-1).tolist()) == list(range(ranks * per))
    assert all(r.tolist() == sorted(r.tolist()) for r in rows)              # batch order kept inside a rank
    loads = costs[rows].sum(axis=1)
    # the greedy deal keeps every rank within one row's cost of the mean
    assert loads.max() <= costs.sum() / ranks + costs.max() + 1e-6
    assert np.array_equal(rows, balanced_row_assignment(costs, ranks))


# ------------------------------------------------------------------ safetensors
def _raw(t: torch.Tensor) -> bytes:
    return t.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""


DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64, torch.uint8, torch.bool]


@settings(max_examples=25, deadline=None)
@given(specs=st.lists(st.tuples(st.sampled_from(range(len(DTYPES))), st.lists(st.integers(0, 5), min_size=0, max_size=3)),
                      min_size=1, max_size=6),
       meta=st.dictionaries(st.text("abcxyz_", min_size=1, max_size=6), st.text(max_size=12), max_size=3))
def test_safetensors_round_trip_is_bit_exact(tmp_path_factory, specs, meta):
    from causal_trainer_dev_b200.checkpointing import safetensors_io as sio

    gen = torch.Generator().manual_seed(len(specs))
    tensors = {}
    for i, (d, shape) in enumerate(specs):
        dtype = DTYPES[d]
        raw = torch.randint(0, 255, tuple(shape), generator=gen)
        tensors[f"t{i}"] = (raw % 2).bool() if dtype == torch.bool else raw.to(dtype)
    path = tmp_path_factory.mktemp("st") / "x.safetensors"
    sio.save_file(tensors, path, metadata=meta)
    back = sio.load_file(path)
    assert set(back) == set(tensors)
    for k, v in tensors.items():
        assert back[k].dtype == v.dtype and back[k].shape == v.shape
        assert _raw(back[k]) == _raw(v)
    infos, got_meta, _ = sio.read_header(path)
    assert got_meta == dict(meta) and set(infos) == set(tensors)


# ------------------------------------------------------------------ schedule
@FAST
@given(name=st.sampled_from(["cosine", "linear", "constant"]), start=st.floats(1e-6, 1.0), ratio=st.floats(0.0, 1.0),
       total=st.integers(1, 200), warm_frac=st.floats(0.0, 0.9))
def test_schedule_warms_up_linearly_then_decays_monotonically_to_the_end_value(name, start, ratio, total, warm_frac):
    from causal_trainer_dev_b200.training.optimizer import build_learning_rate_schedule

    warm = min(int(total * warm_frac), total - 1)
    end = start * ratio
    lr = build_learning_rate_schedule(name, start, end, total, warm)
    values = [lr(s) for s in range(total + 3)]
    assert all(math.isfinite(v) and v >= 0.0 for v in values)
    for s in range(warm):
        assert values[s] == pytest.approx(start * s / warm)
    tail = values[warm:]
    assert tail[0] == pytest.approx(start)
    if name == "constant":
        assert all(v == pytest.approx(start) for v in tail)
    else:
        assert all(a >= b - 1e-12 for a, b in zip(tail, tail[1:]))
        assert values[total] == pytest.approx(end, abs=1e-12) and values[total + 2] == pytest.approx(end, abs=1e-12)


# ------------------------------------------------------------------ chunked loss
@settings(max_examples=30, deadline=None)
@given(budget=st.integers(1, 40), seed=st.integers(0, 50), use_weights=st.booleans())
def test_chunked_loss_is_independent_of_the_chunk_size_and_matches_full_logits(budget, seed, use_weights):
    """Equivalence of execution modes: any token budget gives the sums (and gradients) of the plain
    full-logits cross-entropy over the shifted, segment-aware targets."""
    import torch.nn.functional as F

    from causal_trainer_dev_b200.training.losses import chunked_causal_lm_loss

    g = torch.Generator().manual_seed(seed)
    b, s, d, vocab = 2, 12, 8, 17
    hidden = torch.randn(b, s, d, generator=g, dtype=torch.float64).requires_grad_()
    head = torch.randn(vocab, d, generator=g, dtype=torch.float64).requires_grad_()
    ids = torch.randint(1, vocab, (b, s), generator=g)
    mask = torch.ones(b, s, dtype=torch.int64)
    mask[1, 9:] = 0
    seg = torch.ones(b, s, dtype=torch.int64)
    seg[0, 5:] = 2
    seg[1, 9:] = 0
    weights = torch.rand(b, s, generator=g, dtype=torch.float64) if use_weights else None
    nll, count = chunked_causal_lm_loss(hidden, head, ids, mask, seg, loss_weights=weights, token_budget=budget)
    # the definition: position i predicts token i + 1 when both are attended tokens of one document
    w = ((seg[:, :-1] == seg[:, 1:]) & (seg[:, 1:] != 0) & (mask[:, :-1] == 1) & (mask[:, 1:] == 1)).double()
    if weights is not None:
        w = w * weights[:, 1:]
    logits = hidden[:, :-1] @ head.t()
    per_token = F.cross_entropy(logits.reshape(-1, vocab), ids[:, 1:].reshape(-1), reduction="none").reshape(b, s - 1)
    want_nll, want_count = (per_token * w).sum(), w.sum()
    # the loss is accumulated in fp32 whatever the inputs are
    assert float(count.detach()) == pytest.approx(float(want_count), rel=1e-5)
    assert float(nll.detach()) == pytest.approx(float(want_nll.detach()), rel=1e-5)
    got = torch.autograd.grad(nll, (hidden, head))
    ref = torch.autograd.grad(want_nll, (hidden, head))
    for a, c in zip(got, ref):
        torch.testing.assert_close(a.double(), c, rtol=1e-4, atol=1e-5)
