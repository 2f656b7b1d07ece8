import math

import torch

from causal_trainer_dev_b200.training.losses import (aligned_targets_and_weights, causal_lm_loss,
                                                     shifted_targets_and_weights)


def test_segment_boundaries_and_padding():
    ids = torch.tensor([[0, 10, 11, 20, 21]])
    t, w = shifted_targets_and_weights(ids, torch.tensor([[0, 1, 1, 1, 1]]), torch.tensor([[0, 1, 1, 2, 2]]))
    assert t.tolist() == [[0, 11, 0, 21]] and (w > 0).tolist() == [[False, True, False, True]]


def test_zero_label_is_a_real_segment_and_reuse_is_new():
    ids = torch.arange(6)[None]
    _, w = shifted_targets_and_weights(ids, torch.ones(1, 6, dtype=torch.long), torch.tensor([[0, 0, 7, 7, 0, 0]]))
    assert (w > 0).tolist() == [[True, False, True, False, True]]


def test_weight_is_read_at_the_target_and_needs_a_predecessor():
    ids = torch.arange(5)[None]
    mask = torch.tensor([[0, 1, 1, 1, 1]])
    _, w = shifted_targets_and_weights(ids, mask, None, assistant_mask=torch.tensor([[1, 1, 0, 1, 0]]))
    assert w.tolist() == [[0.0, 0.0, 1.0, 0.0]]
    _, w = shifted_targets_and_weights(ids, mask, None, loss_mask=torch.tensor([[1.0, 1.0, 0.25, 0.5, 2.0]]))
    assert w.tolist() == [[0.0, 0.25, 0.5, 2.0]]


def test_fractional_weights_with_uniform_logits():
    hidden = torch.zeros(1, 5, 4)
    head = torch.zeros(5, 4)
    batch = dict(input_ids=torch.tensor([[1, 2, 3, 4, 0]]), attention_mask=torch.ones(1, 5, dtype=torch.long),
                 loss_weights=torch.tensor([[1.0, 1.0, 1.0, 0.25, 0.5]]))
    nll, wsum = causal_lm_loss(hidden, head, batch, implementation="xla")
    assert abs(float(wsum) - 2.75) < 1e-6 and abs(float(nll) - 2.75 * math.log(5)) < 1e-5


def test_padded_targets_give_exact_zero_gradient_at_the_last_position():
    torch.manual_seed(0)
    hidden = torch.randn(2, 6, 8, requires_grad=True)
    head = torch.randn(11, 8)
    batch = dict(input_ids=torch.randint(0, 11, (2, 6)), attention_mask=torch.ones(2, 6, dtype=torch.long))
    t, w = aligned_targets_and_weights(batch)
    assert t.shape == (2, 6) and torch.all(w[:, -1] == 0)
    nll, _ = causal_lm_loss(hidden, head, batch, implementation="xla")
    nll.backward()
    assert torch.all(hidden.grad[:, -1] == 0) and hidden.grad[:, :-1].abs().sum() > 0
    # equals the unpadded statement
    ref = torch.nn.functional.cross_entropy((hidden[:, :-1] @ head.t()).reshape(-1, 11), batch["input_ids"][:, 1:].reshape(-1),
                                            reduction="sum")
    assert torch.allclose(nll, ref, rtol=1e-5)


def test_single_token_sequence_is_zero():
    batch = dict(input_ids=torch.tensor([[3]]), attention_mask=torch.ones(1, 1, dtype=torch.long))
    nll, wsum = causal_lm_loss(torch.zeros(1, 1, 4), torch.zeros(7, 4), batch, implementation="xla")
    assert float(nll) == 0.0 and float(wsum) == 0.0


def test_prediction_targets_take_over():
    batch = dict(input_ids=torch.tensor([[1, 2, 3]]), attention_mask=torch.ones(1, 3, dtype=torch.long),
                 prediction_targets=torch.tensor([[9, 9, -5]]), prediction_weights=torch.tensor([[0.0, 1.0, 0.0]]))
    t, w = aligned_targets_and_weights(batch)
    assert t.tolist() == [[0, 9, 0]] and w.tolist() == [[0.0, 1.0, 0.0]]
