"""Learning-rate schedules and the AdamW state of the PyTorch (oracle / CPU) path.

Schedules: linear warm-up from 0 to ``learning_rate`` over ``warmup_steps``, then cosine,
linear or constant decay to the *absolute* end value ``learning_rate_end`` over the
remaining steps (src/causal_trainer/training/optimizer.py:9-39).  AdamW: gradients are
clipped by global norm, weight decay applies to tensors with more than one dimension, and
both moments are stored in the parameter dtype (optimizer.py:42-75).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..ops import elementwise as ew


@dataclass(frozen=True)
class ScheduleConfig:
    learning_rate: float
    learning_rate_end: float = 0.0
    scheduler: str = "cosine"
    warmup_steps: int = 0
    total_steps: int = 1


def learning_rate_at(cfg: ScheduleConfig, step: int) -> float:
    """Learning rate used for the update made at zero-based optimizer step ``step``."""
    if cfg.scheduler not in ("cosine", "linear", "constant"):
        raise ValueError(f"unknown scheduler {cfg.scheduler!r}")
    warm = max(cfg.warmup_steps, 0)
    if warm > 0 and step < warm:
        return cfg.learning_rate * step / warm
    if cfg.scheduler == "constant":
        return cfg.learning_rate
    decay_steps = max(cfg.total_steps - warm, 1)
    t = min(max(step - warm, 0), decay_steps) / decay_steps
    if cfg.scheduler == "linear":
        return cfg.learning_rate + (cfg.learning_rate_end - cfg.learning_rate) * t
    alpha = cfg.learning_rate_end / cfg.learning_rate
    cosine = 0.5 * (1.0 + math.cos(math.pi * t))
    return cfg.learning_rate * ((1.0 - alpha) * cosine + alpha)


def build_learning_rate_schedule(name: str, start: float, end: float, total_steps: int, warmup_steps: int = 0):
    """``step -> learning rate`` as a plain function, with the argument checks of
    src/causal_trainer/training/optimizer.py:9-39 (``end`` is an absolute value; a one-step run may
    name one warm-up step, which is then dropped)."""
    if total_steps <= 0:
        raise ValueError("total_steps must be positive")
    if not 0 <= warmup_steps < total_steps:
        if warmup_steps == total_steps == 1:
            warmup_steps = 0
        else:
            raise ValueError("warmup_steps must be in [0, total_steps)")
    if name not in ("cosine", "linear", "constant"):
        raise ValueError(f"unsupported scheduler: {name}")
    cfg = ScheduleConfig(float(start), float(end), name, int(warmup_steps), int(total_steps))
    return lambda step: learning_rate_at(cfg, int(step))


@dataclass(frozen=True)
class AdamWConfig:
    weight_decay: float = 0.0
    max_grad_norm: float = 1.0
    beta1: float = 0.9
    beta2: float = 0.999
    epsilon: float = 1e-8


class FlatAdamW:
    """AdamW over the flat unit buffers of :class:`ModelParams` (or any list of flat tensors).

    ``regions`` are ``(param, decay)`` pairs; the state lives in tensors of the parameter
    dtype.  ``update`` takes gradients already normalised by the global token count and cast
    to the parameter dtype (the clip norm is measured on those, steps.py:173-178).
    """

    def __init__(self, regions: list[tuple[torch.Tensor, bool]], cfg: AdamWConfig):
        self.cfg = cfg
        self.regions = regions
        self.m = [torch.zeros_like(p) for p, _ in regions]
        self.v = [torch.zeros_like(p) for p, _ in regions]
        self.count = 0

    def state_tensors(self) -> list[torch.Tensor]:
        return [t for pair in zip(self.m, self.v) for t in pair]

    @staticmethod
    def global_norm(grads: list[torch.Tensor], round_bf16: bool = False) -> torch.Tensor:
        total = None
        for g in grads:
            if g.is_cuda and g.dtype in (torch.bfloat16, torch.float32):
                sq = ew.sum_of_squares(g, round_bf16=round_bf16)
            else:
                sq = g.float().pow(2).sum()
            total = sq if total is None else total + sq
        return torch.sqrt(total)

    def update(self, grads: list[torch.Tensor], lr: float, grad_norm: torch.Tensor | None = None) -> torch.Tensor:
        c = self.cfg
        # fp32 accumulators feeding bf16 parameters: the cast to the parameter dtype happens
        # inside the kernels (norm and update both see the rounded value).
        rounding = [g.dtype == torch.float32 and p.dtype == torch.bfloat16 for (p, _), g in zip(self.regions, grads)]
        if grad_norm is None:
            grad_norm = self.global_norm(grads, round_bf16=any(rounding))
        clip = torch.ones_like(grad_norm)
        if c.max_grad_norm > 0:
            clip = torch.clamp(c.max_grad_norm / torch.clamp(grad_norm, min=1e-16), max=1.0)
            clip = torch.where(torch.isfinite(grad_norm), clip, torch.ones_like(clip))
        self.count += 1
        for (p, decay), g, m, v in zip(self.regions, grads, self.m, self.v):
            kw = dict(lr=lr, b1=c.beta1, b2=c.beta2, eps=c.epsilon, decay=c.weight_decay if decay else 0.0,
                      step=self.count)
            with torch.no_grad():
                if p.is_cuda and p.dtype == torch.bfloat16:
                    ew.adamw_update(p, g, m, v, clip=clip.float().reshape(1), round_bf16=g.dtype == torch.float32,
                                    **kw)
                else:
                    ew.adamw_reference(p, g, m, v, clip=float(clip), **kw)
        return grad_norm
