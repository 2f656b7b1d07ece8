"""Schedules and the AdamW step of the PyTorch path against hand-computed values
(contracts of the reference's tests/training/test_optimizer.py and test_async_dispatch.py)."""
import math

import numpy as np
import pytest
import torch

from causal_trainer_dev_b200.data.batching import split_accumulation
from causal_trainer_dev_b200.training.optimizer import AdamWConfig, FlatAdamW, ScheduleConfig, learning_rate_at
from causal_trainer_dev_b200.training.runner import MetricWindow


def test_cosine_end_is_an_absolute_learning_rate():
    cfg = ScheduleConfig(2e-5, 5e-6, "cosine", 0, 100)
    assert math.isclose(learning_rate_at(cfg, 0), 2e-5)
    assert math.isclose(learning_rate_at(cfg, 100), 5e-6)
    assert math.isclose(learning_rate_at(cfg, 50), 0.5 * (2e-5 + 5e-6))
    assert math.isclose(learning_rate_at(cfg, 1000), 5e-6)            # held after the end


def test_warmup_is_linear_from_zero_then_decay_spans_the_rest():
    cfg = ScheduleConfig(1e-3, 1e-4, "linear", 10, 110)
    assert learning_rate_at(cfg, 0) == 0.0
    assert math.isclose(learning_rate_at(cfg, 5), 5e-4)
    assert math.isclose(learning_rate_at(cfg, 10), 1e-3)
    assert math.isclose(learning_rate_at(cfg, 60), 1e-3 + (1e-4 - 1e-3) * 0.5)
    assert math.isclose(learning_rate_at(ScheduleConfig(3e-4, 0.0, "constant", 4, 50), 30), 3e-4)
    with pytest.raises(ValueError):
        learning_rate_at(ScheduleConfig(1e-3, 0.0, "exponential", 0, 10), 1)


def test_adamw_step_matches_the_formula_with_clip_and_decay_mask():
    torch.manual_seed(0)
    w = torch.randn(4, 3)
    b = torch.randn(3)
    gw, gb = torch.randn(4, 3) * 3, torch.randn(3) * 3
    cfg = AdamWConfig(weight_decay=0.1, max_grad_norm=1.0, beta1=0.9, beta2=0.99, epsilon=1e-8)
    pw, pb = w.clone(), b.clone()
    opt = FlatAdamW([(pw, True), (pb, False)], cfg)            # decay only on the matrix
    norm = opt.update([gw.clone(), gb.clone()], lr=0.01)
    want_norm = math.sqrt(float(gw.pow(2).sum() + gb.pow(2).sum()))
    assert math.isclose(float(norm), want_norm, rel_tol=1e-6)
    clip = min(1.0, 1.0 / want_norm)

    def step(p, g, decay):
        g = g * clip
        m = 0.1 * g
        v = 0.01 * g * g
        return p - 0.01 * ((m / (1 - 0.9)) / (torch.sqrt(v / (1 - 0.99)) + 1e-8) + decay * p)

    assert torch.allclose(pw, step(w, gw, 0.1), atol=1e-6)
    assert torch.allclose(pb, step(b, gb, 0.0), atol=1e-6)
    assert opt.count == 1 and opt.m[0].dtype == pw.dtype          # moments in the parameter dtype


def test_adamw_without_clipping_and_with_nonfinite_norm():
    p = torch.ones(2, 2)
    opt = FlatAdamW([(p, True)], AdamWConfig(weight_decay=0.0, max_grad_norm=0.0, beta1=0.0, beta2=0.0))
    opt.update([torch.full((2, 2), 4.0)], lr=0.25)               # m = g, v = g^2: update = lr * sign(g)
    assert torch.allclose(p, torch.full((2, 2), 0.75), atol=1e-6)
    q = torch.ones(2)
    opt2 = FlatAdamW([(q, False)], AdamWConfig(max_grad_norm=1.0))
    norm = opt2.update([torch.tensor([float("inf"), 1.0])], lr=0.1)   # a non-finite norm must not turn the clip into NaN
    assert not torch.isfinite(norm)


def test_metric_window_keeps_a_bounded_number_of_steps_in_flight():
    class M:
        def __init__(self, v):
            self.v, self.read = v, False

        def to_floats(self):
            self.read = True
            return {"loss": self.v}

    w = MetricWindow(2)
    ms = [M(float(i)) for i in range(4)]
    for i, m in enumerate(ms):
        w.push(i, m)
    assert [m.read for m in ms] == [True, True, False, False]     # only the two newest are still pending
    assert w.latest == {"loss": 1.0, "step": 1}
    assert w.drain() == {"loss": 3.0, "step": 3} and not w.pending
    assert [m.read for m in ms] == [True, True, False, True]     # only the newest pending step is read back


def test_split_accumulation_reshapes_or_refuses():
    batch = {"input_ids": np.arange(24).reshape(6, 4), "loss_weights": np.ones((6, 4), dtype=np.float32)}
    out = split_accumulation(batch, 3)
    assert out["input_ids"].shape == (3, 2, 4) and np.array_equal(out["input_ids"][1, 0], np.arange(8, 12))
    with pytest.raises(ValueError):
        split_accumulation(batch, 4)
