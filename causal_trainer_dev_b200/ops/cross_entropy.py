"""Projection-fused ("cut") cross-entropy and its chunked / plain companions.

``cut_cross_entropy`` never materialises the ``[tokens, vocab]`` logits in the forward
pass: the LM-head GEMM runs on tcgen05 with an epilogue that reduces each 256-column
slab of a row to (max, sum-exp, target logit) while the tile is still in TMEM
(``csrc/gemm.cu``, EPI_CE_STATS); a small kernel merges the slabs into the row LSE and
the weighted NLL.  The backward pass recomputes logits chunk by chunk with the
``(softmax - onehot) * coef`` epilogue (EPI_CE_DLOGITS) into a bounded bf16 slab and feeds
two ordinary GEMMs (dHidden, dHead), so memory is O(chunk * vocab), not O(tokens * vocab).

Losses are *sums* (``nll_sum``, ``weight_sum``); the caller normalises globally, as
src/causal_trainer/training/steps.py:172 does.

Reference counterparts: pallas_cut_linear_cross_entropy
(src/causal_trainer/kernels/cut_cross_entropy.py:85-156, 225-278, 349-403, 828-960),
the chunked logits backend (src/causal_trainer/kernels/cross_entropy.py:99-189, 254-322)
and the XLA oracle (src/causal_trainer/kernels/fused_cross_entropy.py:64-109).
"""
from __future__ import annotations

import ctypes

import torch

from . import lib as _lib
from .gemm import gemm

SLAB = 256


def reference_cross_entropy(hidden, head, targets, weights):
    """fp32 oracle: returns (nll_sum, weight_sum).  head is [vocab, hidden]."""
    logits = hidden.float() @ head.float().t()
    lse = torch.logsumexp(logits, dim=-1)
    tgt = logits.gather(-1, targets.long().clamp_min(0)[:, None])[:, 0]
    w = weights.float()
    return ((lse - tgt) * w).sum(), w.sum()


def chunked_cross_entropy(hidden, head, targets, weights, token_budget: int = 4096):
    """Autograd-friendly chunked logits CE (the ``pallas``/``xla`` backends of the CLI).

    Walks row chunks of at most ``token_budget`` rows, skips chunks whose weights are all
    zero, and checkpoints each chunk so only one logits slab is alive at a time.
    """
    from torch.utils.checkpoint import checkpoint

    def one(h, t, w):
        logits = (h @ head.t()).float()
        lse = torch.logsumexp(logits, dim=-1)
        tgt = logits.gather(-1, t.long()[:, None])[:, 0]
        return ((lse - tgt) * w.float()).sum()

    total = hidden.new_zeros((), dtype=torch.float32)
    for start in range(0, hidden.shape[0], token_budget):
        w = weights[start:start + token_budget]
        if not bool((w != 0).any()):
            continue
        h, t = hidden[start:start + token_budget], targets[start:start + token_budget]
        if torch.is_grad_enabled() and (hidden.requires_grad or head.requires_grad):
            total = total + checkpoint(one, h, t, w, use_reentrant=False)
        else:
            total = total + one(h, t, w)
    return total, weights.float().sum()


def cut_ce_forward(hidden, head, targets, weights, grad_scale: float | torch.Tensor = 1.0, exchange=None):
    """Returns (nll_sum, weight_sum, lse, coef); coef = weights * grad_scale for the backward.

    ``grad_scale`` may be a one-element device tensor (the reciprocal of a token count that was
    just all-reduced): it is applied on the device, so the caller never has to read it back.

    With ``exchange`` (vocabulary-parallel head: ``head`` holds this rank's vocabulary rows and
    ``targets`` are already relative to them, -1 elsewhere) the per-row statistics are combined
    across the tensor-parallel ranks inside ``exchange.ce_exchange``.
    """
    rows, d = hidden.shape
    vocab = head.shape[0]
    slabs = (vocab + SLAB - 1) // SLAB
    dev = hidden.device
    scale_on_device = grad_scale if isinstance(grad_scale, torch.Tensor) else None
    if scale_on_device is not None:
        grad_scale = 1.0
    pmax = torch.empty((slabs, rows), dtype=torch.float32, device=dev)
    psum = torch.empty((slabs, rows), dtype=torch.float32, device=dev)
    tlogit = torch.zeros(rows, dtype=torch.float32, device=dev)
    tgt = targets.to(torch.int32).contiguous()
    w = weights.to(torch.float32).contiguous()
    L = _lib.lib()
    from .gemm import _FLAG_SOURCES, _flag_args, _rotations, flag_source_of

    hit = flag_source_of(head) if _FLAG_SOURCES else None
    hit_a = flag_source_of(hidden) if _FLAG_SOURCES else None
    _, m_rotate = _rotations(None, hit_a, hidden, head, False, False, rows, vocab)
    code = L.ctb_ce_stats(_lib.ptr(hidden), _lib.ptr(head), rows, vocab, d, ctypes.c_long(hidden.stride(0)),
                          ctypes.c_long(head.stride(0)), _lib.ptr(tgt), _lib.ptr(pmax), _lib.ptr(psum),
                          _lib.ptr(tlogit), *_flag_args(hit), *_flag_args(hit_a), m_rotate, _lib.stream_ptr())
    _lib.check(code, "ctb_ce_stats")
    if exchange is not None:
        nll, wsum, lse, coef = exchange.ce_exchange(pmax, psum, slabs, tlogit, w, grad_scale)
        if scale_on_device is not None:
            coef.mul_(scale_on_device.reshape(()).to(coef.dtype))
        return nll, wsum, lse, coef
    lse = torch.empty(rows, dtype=torch.float32, device=dev)
    coef = torch.empty(rows, dtype=torch.float32, device=dev)
    nblk = (rows + 255) // 256
    bn = torch.empty(nblk, dtype=torch.float32, device=dev)
    bw = torch.empty(nblk, dtype=torch.float32, device=dev)
    code = L.ctb_ce_combine(_lib.ptr(pmax), _lib.ptr(psum), slabs, _lib.ptr(tlogit), _lib.ptr(w),
                            ctypes.c_float(grad_scale), _lib.ptr(lse), _lib.ptr(coef), _lib.ptr(bn), _lib.ptr(bw),
                            rows, _lib.stream_ptr())
    _lib.check(code, "ctb_ce_combine")
    if scale_on_device is not None:
        coef.mul_(scale_on_device.reshape(()).to(coef.dtype))
    return bn.sum(), bw.sum(), lse, coef


def cut_ce_backward(hidden, head, targets, lse, coef, *, chunk_rows: int = 4096, need_dhead: bool = True,
                    dhead_out: torch.Tensor | None = None, dhead_accumulate: bool = False, push=None):
    """Returns (dhidden [rows,d] bf16, dhead [vocab,d] or None).

    With ``push`` (vocabulary-parallel head) the partial ``dhidden`` tiles are reduce-scattered
    into the owners' receive buffers by the GEMM epilogue and ``dhidden`` is returned as None.
    """
    rows, d = hidden.shape
    vocab = head.shape[0]
    dev = hidden.device
    tgt = targets.to(torch.int32).contiguous()
    dhidden = torch.empty_like(hidden) if push is None else None
    dhead = None
    if need_dhead:
        dhead = dhead_out if dhead_out is not None else torch.empty((vocab, d), dtype=torch.bfloat16, device=dev)
    chunk_rows = min(chunk_rows, rows)
    if push is not None:
        if rows % 128:
            raise ValueError("the push epilogue needs a multiple of 128 rows")
        chunk_rows = max(128, chunk_rows // 128 * 128)
    slab = torch.empty((chunk_rows, vocab), dtype=torch.bfloat16, device=dev)
    L = _lib.lib()
    first = True
    for start in range(0, rows, chunk_rows):
        n = min(chunk_rows, rows - start)
        h = hidden[start:start + n]
        g = slab[:n]
        code = L.ctb_ce_dlogits(_lib.ptr(h), _lib.ptr(head), _lib.ptr(g), n, vocab, d, ctypes.c_long(h.stride(0)),
                                ctypes.c_long(head.stride(0)), ctypes.c_long(g.stride(0)),
                                _lib.ptr(tgt[start:start + n]), _lib.ptr(lse[start:start + n]),
                                _lib.ptr(coef[start:start + n]), _lib.stream_ptr())
        _lib.check(code, "ctb_ce_dlogits")
        if push is None:
            gemm(g, head, b_mn=True, out=dhidden[start:start + n])              # dH = G @ W
        else:
            from .gemm import gemm_push

            gemm_push(g, head, push, b_mn=True, row_offset=start,
                      tiles_per_dest=(push.rows_per_rank // 128) * (-(-d // 256)))
        if need_dhead:
            gemm(g, h, a_mn=True, b_mn=True, out=dhead, accumulate=(dhead_accumulate or not first))  # dW += G^T H
        first = False
    return dhidden, dhead


def logits_ce_forward_backward(hidden, head, targets, weights, grad_scale: float = 1.0, *, chunk_rows: int = 4096,
                               need_dhead: bool = True, dhead_out: torch.Tensor | None = None,
                               dhead_accumulate: bool = False):
    """Cross-entropy through a materialised bf16 logits slab per row chunk (the ``pallas`` loss
    backend of the reference, src/causal_trainer/kernels/cross_entropy.py:216-251, 358-397):
    logits GEMM -> row statistics kernel -> dlogits written in place over the logits -> dH, dW.

    Returns ``(nll_sum, weight_sum, dhidden, dhead)``.  Rows with zero weight are skipped chunk-wise.
    """
    rows, d = hidden.shape
    vocab = head.shape[0]
    dev = hidden.device
    tgt = targets.to(torch.int32).contiguous()
    w = weights.to(torch.float32).contiguous()
    coef = w * grad_scale
    dhidden = torch.zeros_like(hidden)
    dhead = None
    if need_dhead:
        dhead = dhead_out if dhead_out is not None else torch.empty((vocab, d), dtype=torch.bfloat16, device=dev)
    chunk_rows = min(chunk_rows, rows)
    ldl = (vocab + 7) // 8 * 8
    slab = torch.empty((chunk_rows, ldl), dtype=torch.bfloat16, device=dev)
    lse = torch.empty(rows, dtype=torch.float32, device=dev)
    tl = torch.empty(rows, dtype=torch.float32, device=dev)
    L = _lib.lib()
    first = True
    for start in range(0, rows, chunk_rows):
        n = min(chunk_rows, rows - start)
        h = hidden[start:start + n]
        g = slab[:n, :vocab]
        gemm(h, head, out=g)
        code = L.ctb_logits_ce_stats(_lib.ptr(g), ctypes.c_long(ldl), n, vocab, _lib.ptr(tgt[start:start + n]),
                                     _lib.ptr(lse[start:start + n]), _lib.ptr(tl[start:start + n]), _lib.stream_ptr())
        _lib.check(code, "ctb_logits_ce_stats")
        code = L.ctb_logits_ce_backward(_lib.ptr(g), ctypes.c_long(ldl), n, vocab, _lib.ptr(tgt[start:start + n]),
                                        _lib.ptr(lse[start:start + n]), _lib.ptr(coef[start:start + n]),
                                        _lib.stream_ptr())
        _lib.check(code, "ctb_logits_ce_backward")
        gemm(g, head, b_mn=True, out=dhidden[start:start + n])
        if need_dhead:
            gemm(g, h, a_mn=True, b_mn=True, out=dhead, accumulate=(dhead_accumulate or not first))
        first = False
    nll = torch.where(w != 0, (lse - tl) * w, torch.zeros_like(lse))
    return nll.sum(), w.sum(), dhidden, dhead


class _CutCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, head, targets, weights, chunk_rows):
        nll, wsum, lse, coef = cut_ce_forward(hidden, head, targets, weights, 1.0)
        ctx.save_for_backward(hidden, head, targets, lse, coef)
        ctx.chunk_rows = chunk_rows
        return nll, wsum

    @staticmethod
    def backward(ctx, dnll, dw):
        hidden, head, targets, lse, coef = ctx.saved_tensors
        coef = coef * dnll.float()
        dh, dhead = cut_ce_backward(hidden, head, targets, lse, coef, chunk_rows=ctx.chunk_rows,
                                    need_dhead=ctx.needs_input_grad[1])
        return dh, dhead, None, None, None


def cut_cross_entropy(hidden, head, targets, weights, chunk_rows: int = 4096):
    """Differentiable projection-fused CE on the sm_100a kernels: (nll_sum, weight_sum)."""
    return _CutCE.apply(hidden, head, targets, weights, chunk_rows)
