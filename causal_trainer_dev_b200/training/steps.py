"""One optimizer step: micro-batch accumulation, global normalisation, clip, AdamW.

Order of operations (src/causal_trainer/training/steps.py:132-194):

1. every micro-batch contributes ``nll_sum`` gradients; with more than one micro-batch they
   are accumulated in fp32;
2. the sum is divided by the *global* loss-weight total of the whole effective batch
   (all micro-batches, all data-parallel ranks), then cast to the parameter dtype;
3. the global gradient norm is measured on those cast gradients, the clip coefficient and
   the scheduled learning rate are applied by AdamW (decay only on matrices, moments in the
   parameter dtype), and the update is cast to the parameter dtype before the add.

Because the loss-weight total depends only on the batch, it is known *before* any backward
pass, so each micro-batch is differentiated with ``grad_scale = 1/total`` and nothing has
to be rescaled afterwards.  Two gradient producers share this step: the autograd oracle in
this file (any device) and the layerwise sm_100a engine (``training/engine.py``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Protocol

import torch
import torch.distributed as dist

from ..models.decoder import ForwardOptions, decoder_forward
from ..models.params import ModelParams
from . import losses
from .optimizer import AdamWConfig, FlatAdamW, ScheduleConfig, learning_rate_at



class GradientProducer(Protocol):
    def __call__(self, batch: dict[str, torch.Tensor], grad_scale: float, first: bool) -> tuple[torch.Tensor, torch.Tensor]:
        """Adds ``grad_scale * d(nll_sum)/d(param)`` into every unit's ``grad`` buffer."""


@dataclass
class StepMetrics:
    loss: torch.Tensor
    nll_sum: torch.Tensor
    token_count: torch.Tensor
    grad_norm: torch.Tensor
    learning_rate: float

    def to_floats(self) -> dict[str, float]:
        return {
            "loss": float(self.loss), "nll_sum": float(self.nll_sum), "token_count": float(self.token_count),
            "grad_norm": float(self.grad_norm), "learning_rate": float(self.learning_rate),
        }


def loss_weight_total(batches: list[dict[str, torch.Tensor]], group=None) -> torch.Tensor:
    """Global sum of loss weights of an effective batch (all micro-batches, all DP ranks)."""
    total = None
    for b in batches:
        _, w = losses.aligned_targets_and_weights(b)
        s = w.sum(dtype=torch.float32)
        total = s if total is None else total + s
    if group is not None or (dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1):
        total = total.clone()
        dist.all_reduce(total, group=group)
    return total


class AutogradProducer:
    """Gradient producer that differentiates the PyTorch oracle decoder."""

    def __init__(self, params: ModelParams, options: ForwardOptions, loss_implementation: str = "xla",
                 token_budget: int = 4096, cut_chunk_size: int = 0, lora=None):
        self.params = params
        self.options = options
        self.loss_kw = dict(implementation=loss_implementation, token_budget=token_budget,
                            cut_chunk_size=cut_chunk_size)
        self.lora = lora
        for u in params.units.values():
            u.data.requires_grad_(lora is None)

    def __call__(self, batch, grad_scale, first):
        p = self.params
        opts = self.options
        if first and self.lora is not None:
            # adapter leaves accumulate in ``.grad`` over the micro-batches of ONE step only
            for _, t in self.lora.trainable():
                t.grad = None
        hidden = decoder_forward(
            p, batch["input_ids"], batch["attention_mask"], batch.get("segment_ids"), batch.get("position_ids"),
            batch.get("attention_end"), opts,
        )
        head = p.units["final"].view("lm_head")
        if self.lora is not None and self.lora.train_embed_and_lm_head:
            head = self.lora.lm_head
        nll, wsum = losses.causal_lm_loss(hidden, head, batch, **self.loss_kw)
        (nll * grad_scale).backward()
        with torch.no_grad():
            for u in p.units.values():
                if u.data.grad is None:
                    continue
                if u.grad is None:
                    u.grad = torch.zeros_like(u.data, dtype=torch.float32)
                if first:
                    u.grad.copy_(u.data.grad)
                else:
                    u.grad.add_(u.data.grad)
                u.data.grad = None
        return nll.detach(), wsum.detach()


@dataclass
class TrainStep:
    """Drives gradient producers and owns optimizer state for a :class:`ModelParams`."""

    params: ModelParams | None        # None when the base is frozen and lives elsewhere (sharded adapter training)
    producer: Callable
    adamw: AdamWConfig
    schedule: ScheduleConfig
    frozen: tuple[str, ...] = ()
    dp_group: object | None = None
    extra_regions: list[tuple[torch.Tensor, bool, Callable[[], torch.Tensor]]] = field(default_factory=list)
    train_base: bool = True

    def __post_init__(self) -> None:
        self._regions: list[tuple[torch.Tensor, bool]] = []
        self._grad_of: list[Callable[[], torch.Tensor]] = []
        from ..models.freezing import frozen_segments

        frozen_segs = frozen_segments(self.params.config, tuple(self.frozen)) if self.train_base else set()
        region_of: dict[tuple[str, str], int] = {}
        if self.train_base:
            for name, u in self.params.units.items():
                for seg in u.layout.segments:
                    if (name, seg.name) in frozen_segs:
                        continue
                    sl = slice(seg.offset, seg.offset + seg.numel)
                    region_of[(name, seg.name)] = len(self._regions)
                    self._regions.append((u.data.detach()[sl], seg.decay))
                    self._grad_of.append(lambda u=u, sl=sl: u.grad[sl])
        for p, decay, g in self.extra_regions:
            self._regions.append((p, decay))
            self._grad_of.append(g)
        self.optimizer = FlatAdamW(self._regions, self.adamw)
        units = list(self.params.units.values()) if self.train_base else []
        from_engine = hasattr(self.producer, "provider")     # the CUDA engine leaves untrained segments' gradients at zero
        if units and from_engine and self.dp_group is None and all(
                u.data.is_cuda and u.data.dtype == torch.bfloat16 for u in units):
            # single-replica bf16 training on a GPU: one AdamW launch per unit instead of one per tensor
            self.optimizer.attach_arenas(units, frozen_segs, region_of)

    @property
    def optimizer_step(self) -> int:
        return self.optimizer.count

    def run(self, micro_batches: list[dict[str, torch.Tensor]], lr_position: int | None = None) -> StepMetrics:
        total = loss_weight_total(micro_batches, self.dp_group)
        denom = torch.clamp(total, min=1.0)
        scale = 1.0 / denom          # a device scalar on GPU runs: the step never waits for the host to read it
        nll_sum = None
        options = getattr(self.producer, "options", None)
        if options is not None and hasattr(options, "optimizer_step"):
            options.optimizer_step = self.optimizer_step      # MoBA's dense_after_step switch
        for i, batch in enumerate(micro_batches):
            nll, _ = self.producer(batch, scale, i == 0)
            nll_sum = nll if nll_sum is None else nll_sum + nll
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(self.dp_group) > 1
        if distributed:
            nll_sum = nll_sum.clone()
            dist.all_reduce(nll_sum, group=self.dp_group)
        grads = []
        for (p, _), g_of in zip(self._regions, self._grad_of):
            g = g_of()
            if distributed:
                dist.all_reduce(g, group=self.dp_group)
            grads.append(g if (g.is_cuda and p.dtype == torch.bfloat16) else g.to(p.dtype))
        step = self.optimizer.count if lr_position is None else lr_position
        lr = learning_rate_at(self.schedule, step)
        grad_norm = self.optimizer.update(grads, lr)
        return StepMetrics(nll_sum / denom, nll_sum, total, grad_norm, lr)


# ---- step builders as plain functions (src/causal_trainer/training/steps.py:26,213,378) ----------
def make_train_step(params: ModelParams, options: ForwardOptions, *, adamw: AdamWConfig, schedule: ScheduleConfig,
                    loss_implementation: str = "xla", token_budget: int = 4096, cut_chunk_size: int = 0,
                    dp_group=None) -> TrainStep:
    """Full-parameter step on the autograd producer (any device); ``step.run(micro_batches)`` makes
    one optimizer update.  The layerwise CUDA engine is wired the same way by the runner, with
    ``training.engine.LayerwiseEngine`` as the producer."""
    producer = AutogradProducer(params, options, loss_implementation, token_budget, cut_chunk_size)
    return TrainStep(params, producer, adamw, schedule, dp_group=dp_group)


def make_frozen_full_train_step(params: ModelParams, options: ForwardOptions, frozen_parameters, *, adamw: AdamWConfig,
                                schedule: ScheduleConfig, loss_implementation: str = "xla", token_budget: int = 4096,
                                cut_chunk_size: int = 0, dp_group=None) -> TrainStep:
    """Full-parameter step with ``lm_head`` / ``embed`` / ``norm`` components held fixed: they get
    no optimizer region and no optimizer state."""
    frozen = tuple(frozen_parameters)
    if not frozen:
        raise ValueError("frozen components must not be empty")
    producer = AutogradProducer(params, options, loss_implementation, token_budget, cut_chunk_size)
    return TrainStep(params, producer, adamw, schedule, frozen=frozen, dp_group=dp_group)


def make_lora_train_step(params: ModelParams, lora, options: ForwardOptions, *, adamw: AdamWConfig,
                         schedule: ScheduleConfig, loss_implementation: str = "xla", token_budget: int = 4096,
                         cut_chunk_size: int = 0, dp_group=None) -> TrainStep:
    """Adapter step: the base stays fixed (no gradients, no optimizer state for it), the adapter
    leaves of ``lora`` (and its embedding / LM-head copies when it has them) are the regions."""
    options.lora = lora
    producer = AutogradProducer(params, options, loss_implementation, token_budget, cut_chunk_size, lora=lora)
    extra = [(t.detach(), t.dim() > 1, (lambda t=t: t.grad)) for _, t in lora.trainable()]
    return TrainStep(params, producer, adamw, schedule, dp_group=dp_group, extra_regions=extra, train_base=False)
