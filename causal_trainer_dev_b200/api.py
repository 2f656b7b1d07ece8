"""Public training API: the calls a user of the framework makes.

``Trainer`` owns the sharded parameters, the optimizer state and the sm_100a engine of one
rank (one process per GPU).  ``train_step`` takes the rank's rows of one global batch as
*host* tensors (pinned for asynchronous copies), uploads them, runs every micro-batch
through forward / recompute / backward, reduces and applies the update, and returns the
step metrics as Python floats (one device-to-host read).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from .models.config import ModelConfig
from .models.params import ModelParams
from .ops import lib as _lib
from .training.engine import EngineOptions, LayerwiseEngine, LocalProvider
from .training.optimizer import AdamWConfig, ScheduleConfig, learning_rate_at
from .training.steps import TrainStep

BATCH_FIELDS = ("input_ids", "attention_mask", "segment_ids", "position_ids", "loss_weights", "attention_end",
                "prediction_targets", "prediction_weights")


@dataclass
class TrainerConfig:
    micro_batch_rows: int = 4
    adamw: AdamWConfig = AdamWConfig()
    schedule: ScheduleConfig = ScheduleConfig(learning_rate=2e-5, total_steps=1000)
    seed: int = 0
    fsdp: bool = True                  # shard parameters, gradients and optimizer state over all ranks
    fused_collectives: bool = True     # in-kernel NVLink all-gather / reduce-scatter instead of NCCL
    cut_chunk_rows: int = 4096
    init: str = "normal"               # "normal": N(0, initializer_range) on the device; "hf": ModelParams.init_random
    remat: str = "auto"                # "auto": keep activations that fit, recompute the rest; "full"; "none"
    tp: int = 1                        # tensor-parallel degree; ranks are laid out (fsdp, tp) with tp fastest
    sp: int = 1                        # sequence-parallel degree (queries sharded, K/V all-gathered); may be combined with tp
    sp_layout: str = "contiguous"      # "zigzag": rank r computes chunks r and 2 sp - 1 - r of every row (equal causal work)
    force_sharded_runtime: bool = False  # run the FSDP runtime even on one rank (measures its own overhead)
    frozen: tuple[str, ...] = ()       # components held fixed: any of "lm_head", "embed", "norm"
    loss_backend: str = "cut"          # "cut": projection-fused; "logits": bf16 logits slab per row chunk
    attention_options: object | None = None   # models.moba.AttentionOptions for MoBA layers
    moba_dense_shortcut: bool = True   # rows whose documents all fit in top_k blocks run the (identical) dense kernel


class Trainer:
    def __init__(self, model: ModelConfig, cfg: TrainerConfig | None = None, device: torch.device | None = None):
        self.model = model
        self.cfg = cfg or TrainerConfig()
        if device is None and not torch.cuda.is_available():
            raise RuntimeError("Trainer drives the sm_100a layerwise engine and needs a CUDA device; on a CPU use "
                               "training.steps.make_train_step (the PyTorch oracle path)")
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self._bytes_h2d = 0
        self._bytes_d2h = 0
        self.data_rank, self.data_world = self.rank, self.world
        if self.cfg.sp > 1:
            from .parallel.fsdp import FsdpRuntime
            from .parallel.runtime import RankLattice
            from .training.sp_engine import SpLayerwiseEngine, sp_tp_engine

            sp, tp = self.cfg.sp, self.cfg.tp
            if self.world % (sp * tp):
                raise ValueError(f"sp * tp = {sp * tp} must divide the number of ranks ({self.world})")
            fsdp = self.world // (sp * tp)
            self.lattice = RankLattice((1, fsdp, 1, tp, sp), self.rank)
            shard_group = self.lattice.group(("fsdp", "sp"))      # sp ranks are further FSDP ranks
            sp_group = self.lattice.group(("sp",))
            self.data_rank, self.data_world = self.lattice.coords()["fsdp"], fsdp
            if tp > 1:
                # heads over tp, tokens over sp: the tensor-parallel schedule on each rank's token slice
                from .parallel.tp import tp_local_config

                if self.cfg.frozen:
                    raise ValueError("frozen components are not supported together with tensor parallelism")
                tp_group = self.lattice.group(("tp",))
                self.runtime = FsdpRuntime(tp_local_config(model, tp), self.cfg, self.device, group=shard_group,
                                           full_cfg=model, tp_group=tp_group)
                self.engine = sp_tp_engine(model, tp_group, sp_group, self.runtime, self._engine_options(),
                                           fused=self.cfg.fused_collectives, layout=self.cfg.sp_layout)
            else:
                self.runtime = FsdpRuntime(model, self.cfg, self.device, group=shard_group, frozen=self.cfg.frozen)
                self.engine = SpLayerwiseEngine(model, sp_group, self.runtime, self._engine_options(),
                                                fused=self.cfg.fused_collectives, layout=self.cfg.sp_layout)
            self.step_fn = self.runtime.make_step(self.engine)
        elif self.cfg.tp > 1:
            from .parallel.fsdp import FsdpRuntime
            from .parallel.runtime import RankLattice
            from .parallel.tp import tp_local_config
            from .training.tp_engine import TpLayerwiseEngine

            if self.world % self.cfg.tp:
                raise ValueError(f"tp={self.cfg.tp} must divide the number of ranks ({self.world})")
            self.lattice = RankLattice((1, self.world // self.cfg.tp, 1, self.cfg.tp, 1), self.rank)
            fsdp_group = self.lattice.group(("fsdp",))
            tp_group = self.lattice.group(("tp",))
            self.data_rank, self.data_world = self.lattice.coords()["fsdp"], self.world // self.cfg.tp
            local = tp_local_config(model, self.cfg.tp)
            if self.cfg.frozen:
                raise ValueError("frozen components are not supported together with tensor parallelism")
            self.runtime = FsdpRuntime(local, self.cfg, self.device, group=fsdp_group, full_cfg=model, tp_group=tp_group)
            self.engine = TpLayerwiseEngine(model, tp_group, self.runtime, self._engine_options(),
                                            fused=self.cfg.fused_collectives)
            self.step_fn = self.runtime.make_step(self.engine)
        elif (self.world > 1 or self.cfg.force_sharded_runtime) and self.cfg.fsdp:
            from .parallel.fsdp import FsdpRuntime

            self.runtime = FsdpRuntime(model, self.cfg, self.device, frozen=self.cfg.frozen)
            self.engine = LayerwiseEngine(model, self.runtime, self._engine_options())
            self.step_fn = self.runtime.make_step(self.engine)
        else:
            self.params = self._init_params()
            self.provider = LocalProvider(self.params, torch.bfloat16)
            self.engine = LayerwiseEngine(model, self.provider, self._engine_options())
            self.step_fn = TrainStep(self.params, self.engine, self.cfg.adamw, self.cfg.schedule, frozen=self.cfg.frozen)
        self._accum_checked = False

    def _engine_options(self) -> EngineOptions:
        c = self.cfg
        return EngineOptions(cut_chunk_rows=c.cut_chunk_rows, remat=c.remat, train_lm_head="lm_head" not in c.frozen,
                             train_embed="embed" not in c.frozen, train_norm="norm" not in c.frozen,
                             loss_backend=c.loss_backend, attention_options=c.attention_options,
                             moba_dense_shortcut=c.moba_dense_shortcut)

    def _init_params(self) -> ModelParams:
        if self.cfg.init == "hf":
            return ModelParams.init_random(self.model, self.cfg.seed, torch.bfloat16).to(self.device)
        params = ModelParams(self.model, torch.bfloat16, self.device)
        gen = torch.Generator(device=self.device).manual_seed(self.cfg.seed)
        for name, t in params.named_tensors():
            if name.endswith("layernorm.weight") or name == "model.norm.weight":
                t.fill_(1.0)
            elif name.endswith(".bias"):
                t.zero_()
            else:
                t.normal_(0.0, self.model.initializer_range, generator=gen)
        params.tensor("model.embed_tokens.weight")[self.model.pad_token_id].zero_()
        return params

    # ------------------------------------------------------------------ data movement
    def local_rows(self, global_batch: dict) -> dict[str, torch.Tensor]:
        """This rank's rows of a global batch (NumPy arrays or tensors, identical on every rank) as
        pinned host tensors.  Rows are dealt to the data ranks so that each gets the same number of
        rows and nearly the same attention cost (``data.batching.balanced_row_assignment``): packed
        rows of equal length differ several-fold in visible (query, key) pairs, and the step ends
        when the slowest rank does."""
        import numpy as np

        from .data.batching import attention_cost_per_row, balanced_row_assignment

        arrays = {k: (v.numpy() if isinstance(v, torch.Tensor) else np.asarray(v)) for k, v in global_batch.items()}
        costs = attention_cost_per_row(arrays["segment_ids"], arrays.get("attention_end"))
        rows = balanced_row_assignment(costs, self.data_world)[self.data_rank]
        out = {}
        for k, v in arrays.items():
            t = torch.from_numpy(np.ascontiguousarray(v[rows]))
            out[k] = t.pin_memory() if torch.cuda.is_available() else t
        return out

    def upload(self, host_batch: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        out = {}
        for k, v in host_batch.items():
            if k not in BATCH_FIELDS:
                continue
            self._bytes_h2d += v.numel() * v.element_size()
            out[k] = v.to(self.device, non_blocking=True)
        if self.cfg.attention_options is not None and "segment_ids" in host_batch:
            # a host-side fact about the rows (no device read): lets a MoBA layer whose selection
            # cannot leave anything out run as the dense kernel it is equal to
            from .data.batching import longest_document

            out["longest_document"] = longest_document(host_batch["segment_ids"].numpy())
        return out

    def split_micro_batches(self, batch: dict[str, torch.Tensor]) -> list[dict[str, torch.Tensor]]:
        rows = batch["input_ids"].shape[0]
        mb = min(self.cfg.micro_batch_rows, rows)
        if rows % mb:
            raise ValueError(f"{rows} local rows are not a multiple of micro_batch_rows={mb}")
        return [{k: (v[i:i + mb] if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
                for i in range(0, rows, mb)]

    # ------------------------------------------------------------------ steps
    def train_step_device(self, device_batch: dict[str, torch.Tensor]):
        """Step on inputs that already live on the GPU; returns device-resident metrics."""
        micro = self.split_micro_batches(device_batch)
        if len(micro) > 1 and not self._accum_checked:
            self._switch_to_fp32_accumulation()
        return self.step_fn.run(micro)

    def train_step(self, host_batch: dict[str, torch.Tensor]) -> dict[str, float]:
        """Host tensors in, Python floats out (includes the H2D copies and one D2H read)."""
        metrics = self.train_step_device(self.upload(host_batch))
        packed = torch.stack([metrics.loss.float(), metrics.nll_sum.float(), metrics.token_count.float(),
                              metrics.grad_norm.float()]).cpu()
        self._bytes_d2h += packed.numel() * 4
        # a bounded device wait that gave up during this step left a record: a step built on a
        # flag that never arrived is wrong, so it ends here rather than in a later loss curve
        failure = _lib.poll_device_status()
        if failure is not None:
            raise failure
        loss, nll, count, gnorm = packed.tolist()
        return {"loss": loss, "nll_sum": nll, "token_count": count, "grad_norm": gnorm,
                "learning_rate": metrics.learning_rate}

    def _switch_to_fp32_accumulation(self) -> None:
        # Several micro-batches per step accumulate in fp32 (the reference's scan does the same).
        self._accum_checked = True
        if hasattr(self, "provider"):
            self.provider.grad_dtype = torch.float32
        elif hasattr(self, "runtime"):
            self.runtime.set_grad_dtype(torch.float32)

    def transfer_counters(self) -> tuple[int, int]:
        return self._bytes_h2d, self._bytes_d2h

    def launches(self) -> int:
        from .ops import lib

        return lib.launch_count()

    def current_learning_rate(self) -> float:
        return learning_rate_at(self.cfg.schedule, self.step_fn.optimizer_step)
