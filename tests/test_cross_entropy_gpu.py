"""Projection-fused cut cross-entropy against the fp32 logits oracle."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("rows,d,vocab", [(300, 256, 1000), (1024, 512, 32000)])
def test_cut_ce_forward_backward(cuda_lib, rows, d, vocab):
    from causal_trainer_dev_b200.ops import cross_entropy as CE

    torch.manual_seed(0)
    hidden = torch.randn(rows, d, device="cuda").bfloat16()
    head = (0.05 * torch.randn(vocab, d, device="cuda")).bfloat16()
    targets = torch.randint(0, vocab, (rows,), device="cuda")
    weights = (torch.rand(rows, device="cuda") > 0.3).float() * torch.rand(rows, device="cuda")
    hf = hidden.float().requires_grad_()
    wf = head.float().requires_grad_()
    nll_ref, w_ref = CE.reference_cross_entropy(hf, wf, targets, weights)
    nll_ref.backward()
    h = hidden.clone().requires_grad_()
    w = head.clone().requires_grad_()
    nll, wsum = CE.cut_cross_entropy(h, w, targets, weights, chunk_rows=256)
    nll.backward()
    assert abs(nll.item() - nll_ref.item()) / abs(nll_ref.item()) < 2e-3
    assert abs(wsum.item() - w_ref.item()) < 1e-3 * max(1.0, w_ref.item())
    # relative L2 bound of the reference's cut-CE tests (tests/kernels/test_tiled_cut.py:121-125)
    assert _rel(h.grad, hf.grad) < 0.025
    assert _rel(w.grad, wf.grad) < 0.025
    # rows with zero weight get exactly zero hidden gradient
    assert torch.all(h.grad[weights == 0] == 0)
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_logits_slab_ce_matches_reference(cuda_lib):
    """The materialised-logits backend (stats kernel + in-place dlogits) against fp32 PyTorch."""
    from causal_trainer_dev_b200.ops import cross_entropy as ce

    torch.manual_seed(3)
    rows, d, vocab = 700, 256, 3001          # vocabulary not a multiple of 8, rows not a multiple of the chunk
    hidden = (torch.randn(rows, d, device="cuda") * 0.5).bfloat16()
    head = (torch.randn(vocab, d, device="cuda") * 0.1).bfloat16()
    targets = torch.randint(0, vocab, (rows,), device="cuda")
    weights = (torch.rand(rows, device="cuda") > 0.25).float()
    nll, wsum, dh, dw = ce.logits_ce_forward_backward(hidden, head, targets, weights, 0.01, chunk_rows=256)
    hf = hidden.float().requires_grad_(True)
    wf = head.float().requires_grad_(True)
    logits = hf @ wf.t()
    ref = (torch.nn.functional.cross_entropy(logits, targets, reduction="none") * weights).sum()
    (ref * 0.01).backward()
    assert abs(float(nll) - float(ref.detach())) / float(ref.detach()) < 5e-3
    assert float(wsum) == float(weights.sum())
    assert ((dh.float() - hf.grad).norm() / hf.grad.norm()) < 3e-2
    assert ((dw.float() - wf.grad).norm() / wf.grad.norm()) < 3e-2
