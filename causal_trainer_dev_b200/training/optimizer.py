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

    def attach_arenas(self, units: list, frozen: set[tuple[str, str]], region_of: dict[tuple[str, str], int]) -> None:
        """Lets whole units be updated in ONE launch each (``ops.elementwise.adamw_regions``: 16-byte
        accesses over the unit's flat buffer with a region table for decay / no decay / frozen),
        instead of one launch per tensor.  ``units`` are flat bf16 CUDA parameter buffers with
        segments; ``region_of[(unit, segment)]`` is the index of the segment's region.  The moments of
        those regions become views into one flat buffer per unit, so checkpoints keep their layout."""
        self.arenas = []
        for u in units:
            dev = u.data.device
            m_flat, v_flat = torch.zeros_like(u.data), torch.zeros_like(u.data)
            cuts, modes, covered = [0], [], []
            for seg in u.layout.segments:                      # segments are ascending; gaps are alignment padding
                if seg.offset > cuts[-1]:
                    cuts.append(seg.offset)
                    modes.append(-1)
                key = (u.layout.name, seg.name)
                cuts.append(seg.offset + seg.numel)
                modes.append(-1 if key in frozen else (1 if seg.decay else 0))
                if key in region_of:
                    i = region_of[key]
                    sl = slice(seg.offset, seg.offset + seg.numel)
                    self.m[i], self.v[i] = m_flat[sl], v_flat[sl]
                    covered.append(i)
            if cuts[-1] < u.data.numel():
                cuts.append(u.data.numel())
                modes.append(-1)
            self.arenas.append(dict(unit=u, m=m_flat, v=v_flat, regions=covered,
                                    bounds=torch.tensor(cuts, dtype=torch.int64, device=dev),
                                    modes=torch.tensor(modes, dtype=torch.int32, device=dev)))
        self._in_arena = {i for a in self.arenas for i in a["regions"]}

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
        arenas = getattr(self, "arenas", None)
        # whole-unit path: usable when every unit's gradient is one flat buffer of matching size
        by_unit = arenas is not None and all(a["unit"].grad is not None and a["unit"].grad.is_cuda
                                             and a["unit"].grad.numel() == a["unit"].data.numel() for a in arenas)
        skip = self._in_arena if by_unit else set()
        # fp32 accumulators feeding bf16 parameters: the cast to the parameter dtype happens
        # inside the kernels (norm and update both see the rounded value).
        rounding = [g.dtype == torch.float32 and p.dtype == torch.bfloat16 for (p, _), g in zip(self.regions, grads)]
        if grad_norm is None:
            rest = [g for i, g in enumerate(grads) if i not in skip]
            total = self.global_norm(rest, round_bf16=any(rounding)).pow(2) if rest else None
            if by_unit:
                # frozen segments and alignment gaps hold zeros, so a unit's sum is that of its trained tensors
                for a in arenas:
                    g = a["unit"].grad
                    sq = ew.sum_of_squares(g, round_bf16=g.dtype == torch.float32)
                    total = sq if total is None else total + sq
            grad_norm = torch.sqrt(total)
        clip = torch.ones_like(grad_norm)
        if c.max_grad_norm > 0:
            clip = torch.clamp(c.max_grad_norm / torch.clamp(grad_norm, min=1e-16), max=1.0)
            clip = torch.where(torch.isfinite(grad_norm), clip, torch.ones_like(clip))
        self.count += 1
        if by_unit:
            with torch.no_grad():
                for a in arenas:
                    u = a["unit"]
                    ew.adamw_regions(u.data, u.grad, a["m"], a["v"], a["bounds"], a["modes"], lr=lr, b1=c.beta1, b2=c.beta2,
                                     eps=c.epsilon, decay=c.weight_decay, step=self.count, clip=clip.float().reshape(1),
                                     round_bf16=u.grad.dtype == torch.float32)
        for i, ((p, decay), g, m, v) in enumerate(zip(self.regions, grads, self.m, self.v)):
            if i in skip:
                continue
            kw = dict(lr=lr, b1=c.beta1, b2=c.beta2, eps=c.epsilon, decay=c.weight_decay if decay else 0.0,
                      step=self.count)
            with torch.no_grad():
                if p.is_cuda and p.dtype == torch.bfloat16:
                    ew.adamw_update(p, g, m, v, clip=clip.float().reshape(1), round_bf16=g.dtype == torch.float32,
                                    **kw)
                else:
                    ew.adamw_reference(p, g, m, v, clip=float(clip), **kw)
        return grad_norm
