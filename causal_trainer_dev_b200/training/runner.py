"""``causal-train`` orchestration.

Program lifetime (same stages as src/causal_trainer/training/runner.py:642-2393, written as a
staged :class:`TrainingRun` instead of one function):

 1. parse flags; start ``torch.distributed``; all ranks must present the same flags;
 2. build the rank lattice ``(dp, fsdp, ep, tp, sp)`` and validate it against the model;
 3. resolve the model source, read ``config.json``, load the tokenizer when data is raw;
 4. data, one of four modes: prepared+materialised, prepared+streaming, raw+materialised
    (shard -> tokenise -> pack -> merge), raw+streaming;
 5. training signature -> resume discovery (every rank must find the same checkpoint)
    -> ``start | continue | finalize | complete``;
 6. parameters (HF checkpoint, lazily sharded) -> LoRA / frozen components -> optimizer state;
 7. the step loop: batches are prefetched to pinned memory and copied asynchronously, metrics
    stay on the device for up to ``async_dispatch_steps`` steps, periodic bundles are written
    and pruned;
 8. the final bundle in ``output_dir``.

Every fallible host stage funnels its exception through the collective error bus so that no
rank enters the next collective alone.  Devices: bf16 on CUDA uses the layerwise sm_100a
engine (FSDP over all data ranks when there are several); anything else runs the PyTorch
oracle path with gradient all-reduce.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import logging
import math
import time
from collections import deque
from pathlib import Path
from typing import Any, Iterator

import numpy as np
import torch

from ..checkpointing import bundles
from ..checkpointing import huggingface as hfio
from ..checkpointing import safetensors_io as st
from ..data import batching, maskgit, pipeline, prepared, streaming, streaming_batching
from ..data.preprocessing import EndPromptSettings
from ..data.tokenizer import TrainingTokenizer
from ..models.config import ModelConfig, validate_splash_block_size
from ..models.decoder import ForwardOptions
from ..models.lora import LoraState
from ..models.params import ModelParams
from ..parallel import runtime as rt
from . import logging as tlog
from .arguments import parse_args
from .optimizer import AdamWConfig, ScheduleConfig
from .steps import AutogradProducer, TrainStep

log = logging.getLogger("causal_trainer")

STREAMING_SCHEDULE_POLICY = "buffered-estimate-v1"
_SIGNATURE_ARGUMENTS = (
    "repo_id", "dataset_name", "dataset_format", "dataset_config_name", "dataset_revision", "dataset_split",
    "dataset_streaming", "dataset_text_field", "processor_repo_id", "processor_revision", "revision",
    "max_sequence_length", "packing", "packing_batch_size", "streaming_shuffle_buffer", "assistant_only_loss",
    "last_assistant_only_loss", "endprompt_enable", "endprompt_logical_length", "endprompt_logical_length_min",
    "endprompt_prompts", "endprompt_prompt_loss_weight", "endprompt_context_loss_weight", "preprocessing_mode",
    "attn_mechanism", "block_size_q", "block_size_k", "loss_token_budget", "loss_implementation", "mlp_chunk_size",
    "scan_layers", "total_batch_size", "gradient_accumulation_steps", "learning_rate", "learning_rate_end",
    "scheduler", "warmup_steps", "weight_decay", "max_grad_norm", "adam_beta1", "adam_beta2", "adam_epsilon",
    "num_train_epochs", "max_steps", "shuffle", "seed", "gradient_checkpointing", "lora", "lora_rank",
    "lora_train_embed_and_lm_head", "lora_save_adapter_only", "frozen_parameters", "param_dtype", "dtype",
    "sharding_axis", "sharding_dcn_axis",
)


# --------------------------------------------------------------------------------------- pure helpers
def arguments_digest(args) -> bytes:
    """SHA-256 of every flag except the per-process ones (``process_id``, ``local_device_ids``)."""
    values = {f.name: getattr(args, f.name) for f in dataclasses.fields(args)
              if f.name not in ("process_id", "local_device_ids")}
    return rt.digest_of(values)


def resolve_loss_implementation(args, backend: str = "cuda", *, cut_supported: bool = True) -> str:
    """The loss backend a run uses: ``auto`` is the cut cross-entropy GEMM epilogues (never materialised
    logits) wherever they apply, else the chunked-logits kernels (``pallas``, the flag value kept from
    src/causal_trainer/training/runner.py:331-346); an explicit choice is kept as given.  ``cut_supported``
    is false on the paths that cannot run the fused epilogues (CPU, fp32 compute)."""
    if backend not in ("cuda", "cpu"):
        raise ValueError(f"this trainer runs on CUDA (or on the CPU oracle path), not on {backend!r}")
    chosen = args.loss_implementation
    if chosen == "auto":
        chosen = "cut" if cut_supported else "pallas"
    if getattr(args, "cut_chunk_size", 0) > 0 and (chosen != "cut" or not cut_supported):
        raise ValueError("cut_chunk_size requires the cut loss backend on a path that supports it")
    return chosen


def prepared_streaming_limits(total_rows: int, effective_batch: int, epochs: float, max_steps: int
                              ) -> tuple[int, int | None]:
    """``(total optimizer steps, whole epochs or None)`` for a prepared artifact of known size."""
    if max_steps > 0:
        return max_steps, None
    per_epoch = math.ceil(total_rows / effective_batch)
    return max(1, math.floor(per_epoch * epochs)), max(1, math.ceil(epochs))


def buffered_streaming_schedule_total(estimated_steps: int) -> int:
    """Schedule horizon for a stream of estimated length: 5 % slack, at least one extra step."""
    return estimated_steps + max(1, math.ceil(estimated_steps * 0.05))


def streaming_schedule_position(step_in_epoch: int, epoch: int, estimate_per_epoch: int) -> int:
    """Learning-rate position: capped at the per-epoch estimate inside an epoch."""
    return epoch * estimate_per_epoch + min(step_in_epoch, estimate_per_epoch)


def project_streaming_progress_total(steps_done: int, epochs_done: int, epochs_total: int) -> int:
    """Progress-bar total extrapolated from completed epochs (never below the steps already done)."""
    if epochs_done <= 0:
        return steps_done
    return max(steps_done, math.ceil(steps_done / epochs_done * epochs_total))


def validate_structure(args, cfg: ModelConfig, lattice: rt.RankLattice) -> None:
    """Divisibility and mode rules (the fixed-architecture gate of the reference is not kept)."""
    lattice.validate()
    tp, sp, fsdp, dp = (lattice.size(a) for a in ("tp", "sp", "fsdp", "dp"))
    if cfg.num_attention_heads % tp or cfg.intermediate_size % tp or cfg.vocab_size % tp:
        raise ValueError("tp must divide num_attention_heads, intermediate_size and vocab_size")
    if cfg.num_key_value_heads % tp and tp % cfg.num_key_value_heads:
        raise ValueError("tp must divide, or be a multiple of, num_key_value_heads")
    if args.max_sequence_length % (sp * 128 if sp > 1 else 1):
        raise ValueError("max_sequence_length must be a multiple of 128 * sp under sequence parallelism")
    if args.total_batch_size % (dp * fsdp):
        raise ValueError(f"total_batch_size={args.total_batch_size} must divide by dp*fsdp={dp * fsdp}")
    if args.projection_chunk_size > 0 and (dp != 1 or fsdp != 1):
        raise ValueError("projection_chunk_size requires dp=fsdp=ep=1")
    if args.attention_options is not None:
        args.attention_options.validate_layers(cfg.num_hidden_layers)
    if args.attn_mechanism == "splash":
        validate_splash_block_size(args.max_sequence_length, args.block_size_q, "block_size_q")
        validate_splash_block_size(args.max_sequence_length, args.block_size_k, "block_size_k")


def resume_signature_payload(args, cfg: ModelConfig, plan, dataset_fingerprint, mesh_shape, *, process_count: int,
                             real_rows: int, dummy_rows: int, prepared_revision: str | None = None) -> dict[str, Any]:
    arguments = {n: getattr(args, n) for n in _SIGNATURE_ARGUMENTS}
    arguments["output_dir"] = None
    for name in ("projection_chunk_size", "remat_group_size", "cut_chunk_size"):
        if getattr(args, name) != (1 if name == "remat_group_size" else 0):
            arguments[name] = getattr(args, name)
    if args.attention_options is not None:
        arguments["attention_options"] = dataclasses.asdict(args.attention_options)
    if args.maskgit_probability:
        arguments["maskgit_probability"] = args.maskgit_probability
    payload = {
        "arguments": json.loads(json.dumps(arguments, default=str)),
        "dataset_fingerprint": dataset_fingerprint,
        "preprocessing_process_count": process_count,
        "prepared_real_rows": real_rows, "prepared_dummy_rows": dummy_rows,
        "mesh_shape": dict(zip(rt.AXES, (int(x) for x in mesh_shape))),
        "model_config": cfg.to_dict(), "plan": dataclasses.asdict(plan),
        "streaming_scheduler_policy": STREAMING_SCHEDULE_POLICY if args.uses_raw_streaming and args.max_steps <= 0 else None,
    }
    if args.dataset_format == "prepared":
        payload["prepared_revision"] = prepared_revision
    return payload


def resume_identity(ckpt: bundles.ResumeCheckpoint | None, output_dir: Path, signature: str) -> bytes:
    payload = {
        "checkpoint_id": ckpt.checkpoint_id if ckpt else None, "exists": ckpt is not None,
        "global_step": ckpt.global_step if ckpt else 0, "has_optimizer_state": ckpt.has_optimizer_state if ckpt else False,
        "is_output_root": ckpt is not None and ckpt.path == output_dir,
        "manifest_digest": ckpt.manifest_digest if ckpt else None,
        "source_examples_seen": ckpt.source_examples_seen if ckpt else 0,
        "streaming_data_digest": ckpt.streaming_data_digest if ckpt else None,
        "total_steps": ckpt.total_steps if ckpt else 0, "training_complete": ckpt.training_complete if ckpt else False,
        "training_signature": signature,
    }
    return hashlib.sha256(json.dumps(payload, ensure_ascii=False, separators=(",", ":"), sort_keys=True).encode()).digest()


class MetricWindow:
    """At most ``limit`` finished steps keep their metrics on the device; older ones are read back."""

    def __init__(self, limit: int):
        self.limit = limit
        self.pending: deque = deque()
        self.latest: dict[str, float] | None = None

    def push(self, step: int, metrics) -> None:
        self.pending.append((step, metrics))
        while len(self.pending) > self.limit:
            self._pop()

    def _pop(self) -> None:
        step, m = self.pending.popleft()
        self.latest = dict(m.to_floats(), step=step)

    def drain(self) -> dict[str, float] | None:
        """Reads back the newest pending step only (the device finishes steps in order, so that one
        read synchronises all of them) and drops the references to the older ones."""
        if self.pending:
            step, m = self.pending[-1]
            self.pending.clear()
            self.latest = dict(m.to_floats(), step=step)
        return self.latest


def endprompt_settings(args) -> EndPromptSettings | None:
    if not args.endprompt_enable:
        return None
    return EndPromptSettings(args.effective_endprompt_logical_length_min, args.effective_endprompt_logical_length,
                             args.endprompt_prompt_texts, args.endprompt_prompt_loss_weight,
                             args.endprompt_context_loss_weight)


def _guarded(stage: str):
    """Decorator: run a host stage, then agree with all ranks on whether it failed."""
    def wrap(fn):
        def inner(*a, **k):
            error: BaseException | None = None
            result = None
            try:
                result = fn(*a, **k)
            except Exception as exc:  # noqa: BLE001 - re-raised on every rank by the bus
                error = exc
            rt.raise_if_any_process_error(error, stage)
            return result
        return inner
    return wrap


# --------------------------------------------------------------------------------------- the run
class TrainingRun:
    def __init__(self, args):
        self.args = args
        self.env = rt.initialize_distributed(args.coordinator_address, args.num_processes, args.process_id,
                                             args.local_device_ids, enabled=args.distributed)
        tlog.configure_logging(rt.process_index())
        rt.assert_equal(arguments_digest(args), "command-line arguments")
        self.lattice = rt.RankLattice.create(args.sharding_axis)
        self.cuda = torch.cuda.is_available()
        self.device = torch.device("cuda", self.env.local_rank) if self.cuda else torch.device("cpu")
        self.param_dtype = torch.bfloat16 if args.param_dtype == "bfloat16" else torch.float32
        engine_ok = (self.cuda and self.param_dtype == torch.bfloat16 and args.dtype == "bfloat16"
                     and args.attn_mechanism != "vanilla" and args.loss_implementation != "xla"
                     and (args.attention_options is None or args.attention_options.backend != "reference"))
        self.use_engine = engine_ok and not args.lora
        # adapters on the CUDA engine: every rank holds the frozen base, adapter gradients are all-reduced
        self.use_lora_engine = (engine_ok and args.lora and not args.lora_train_embed_and_lm_head
                                and self.lattice.size("tp") == 1 and self.lattice.size("sp") == 1)
        if self.lattice.size("sp") > 1 and (not self.use_engine or args.attention_options is not None):
            raise ValueError("sequence parallelism (sp > 1) runs on the bf16 CUDA engine with dense attention; "
                             "shard long MoBA rows over tp instead")
        if self.lattice.size("tp") > 1 and not self.use_engine:
            raise ValueError("tensor parallelism (tp > 1) runs on the bf16 CUDA engine only: it needs GPUs, "
                             "--attn_mechanism efficient, a fused loss, no LoRA and dense attention")
        self.prepared_revision: str | None = None
        self.source_examples_seen = 0
        self.stream_digest: str | None = None
        self.training_complete = False

    # ---- stage 3: model source ----
    @_guarded("resolve model source")
    def resolve_model(self) -> None:
        a = self.args
        self.source = hfio.resolve_hf_source(a.repo_id, revision=a.revision, token=a.token)
        self.cfg = ModelConfig.from_dict(hfio.load_hf_config(self.source))
        validate_structure(a, self.cfg, self.lattice)
        self.processor_source = self.source if a.processor_repo_id is None else hfio.resolve_hf_source(
            a.processor_repo_id, revision=a.processor_revision, token=a.token)
        self.tokenizer = None
        if a.dataset_format == "raw" or a.maskgit_probability:
            self.tokenizer = TrainingTokenizer.from_directory(self.processor_source)
            self.tokenizer.validate_model_vocabulary(self.cfg.vocab_size)
        self.has_weights = any(self.source.glob("*.safetensors"))

    # ---- stage 4: data ----
    def _pad_token_id(self) -> int:
        if self.tokenizer is not None and self.tokenizer.pad_token_id is not None:
            return int(self.tokenizer.pad_token_id)
        return int(self.cfg.pad_token_id)

    @_guarded("load dataset")
    def load_data(self) -> None:
        a = self.args
        nproc, pidx = rt.process_count(), rt.process_index()
        effective = a.effective_batch_size
        self.streaming = a.dataset_streaming
        self.dummy_rows = 0
        self.fingerprint: Any = None
        if a.dataset_format == "prepared":
            self.prepared_revision = prepared.resolve_prepared_revision(a.dataset_name, token=a.token,
                                                                        revision=a.dataset_revision)
            self.manifest = prepared.load_prepared_manifest(a.dataset_name, token=a.token, revision=self.prepared_revision)
            if self.manifest.max_sequence_length != a.max_sequence_length:
                raise ValueError("prepared dataset max_sequence_length does not match --max_sequence_length")
            if self.manifest.max_token_id >= self.cfg.vocab_size:
                raise ValueError("prepared dataset contains token ids outside the model vocabulary")
            if a.uses_assistant_loss_mask and not self.manifest.uses_assistant_loss_mask:
                raise ValueError("assistant-only loss needs a prepared dataset built with an assistant mask")
            self.fingerprint = self.manifest.global_digest
            rt.assert_equal(bytes.fromhex(self.manifest.global_digest), "prepared dataset manifest")
            if self.streaming:
                steps, epochs = prepared_streaming_limits(self.manifest.total_rows, effective, a.num_train_epochs,
                                                          a.max_steps)
                self.plan = streaming_batching.StreamingBatchPlan.create(
                    self.manifest.total_rows, a.total_batch_size, a.gradient_accumulation_steps, epochs or 1,
                    a.max_steps if a.max_steps > 0 else steps)
                self.real_rows = self.manifest.total_rows
                return
            local = prepared.load_prepared_dataset(a.dataset_name, self.manifest, token=a.token,
                                                   revision=self.prepared_revision, process_index=pidx,
                                                   process_count=nproc)
            columns = rt.merge_packed_host_arrays(local)
        elif self.streaming:
            dataset = pipeline.load_training_split(a.dataset_name, a.dataset_split, token=a.token,
                                                   config_name=a.dataset_config_name, revision=a.dataset_revision,
                                                   streaming=True)
            meta = streaming.streaming_dataset_metadata(dataset, a.dataset_split)
            self.stream_source = dataset
            self.fingerprint = getattr(dataset, "_fingerprint", None)
            self.plan = streaming_batching.StreamingBatchPlan.create(
                meta.num_examples, a.total_batch_size, a.gradient_accumulation_steps,
                int(a.num_train_epochs) if a.max_steps <= 0 else 1, a.max_steps)
            self.real_rows = 0
            return
        else:
            dataset = pipeline.load_training_split(a.dataset_name, a.dataset_split, token=a.token,
                                                   config_name=a.dataset_config_name, revision=a.dataset_revision)
            rt.assert_equal(pipeline.source_dataset_identity(dataset), "source dataset")
            self.fingerprint = getattr(dataset, "_fingerprint", None)
            sharded = a.preprocessing_mode == "shard_then_merge" and nproc > 1
            shard, offset = (pipeline.select_process_shard(dataset, process_index=pidx, process_count=nproc)
                             if sharded else (dataset, 0))
            rows = pipeline.prepare_training_dataset(
                shard, self.tokenizer, dataset_text_field=a.dataset_text_field,
                max_sequence_length=a.max_sequence_length, packing=a.packing, packing_batch_size=a.packing_batch_size,
                pad_token_id=self._pad_token_id(), assistant_only_loss=a.assistant_only_loss,
                last_assistant_only_loss=a.last_assistant_only_loss, endprompt=endprompt_settings(a),
                num_proc=a.preprocessing_num_workers, example_index_offset=offset, allow_empty=sharded)
            explicit = a.endprompt_enable
            local = pipeline.packed_dataset_to_arrays(rows, max_sequence_length=a.max_sequence_length,
                                                      assistant_only_loss=a.uses_assistant_loss_mask,
                                                      has_explicit_loss_weights=explicit)
            columns = rt.merge_packed_host_arrays(local) if sharded else local
        self.dataset, self.dummy_rows = pipeline.pad_packed_arrays_to_batch_multiple(columns, batch_multiple=effective)
        self.real_rows = self.dataset.real_rows
        self.plan = batching.BatchPlan.create(len(self.dataset), a.total_batch_size, a.gradient_accumulation_steps,
                                              a.num_train_epochs, a.max_steps)

    # ---- stage 5: resume ----
    @_guarded("discover checkpoints")
    def discover_resume(self) -> None:
        a = self.args
        payload = resume_signature_payload(
            a, self.cfg, self.plan, self.fingerprint, self.lattice.shape, process_count=rt.process_count(),
            real_rows=self.real_rows, dummy_rows=self.dummy_rows, prepared_revision=self.prepared_revision)
        self.signature = bundles.training_signature(payload)
        self.artifact_kind = "peft-adapter" if (a.lora and a.lora_save_adapter_only) else "merged"
        layout = hfio.expected_model_layout(self.cfg, self.param_dtype) if self.artifact_kind == "merged" else None
        self.checkpoint = bundles.find_latest_checkpoint(
            a.output_dir, self.signature, expected_model_layout=layout, expected_artifact_kind=self.artifact_kind,
            verify_artifact_digests=rt.process_index() == 0)
        rt.assert_equal(resume_identity(self.checkpoint, Path(a.output_dir), self.signature), "resume checkpoint")
        self.action = bundles.resume_action(self.checkpoint, output_dir=Path(a.output_dir),
                                            total_steps=self.plan.total_steps)
        self.start_step = self.checkpoint.global_step if self.checkpoint is not None else 0

    def engine_options(self, frozen: tuple[str, ...] = ()):
        """How the command line maps onto the CUDA engine, on every branch that builds one.  Flags
        that describe the reference's XLA program and have no counterpart here are named in the log
        instead of being dropped silently."""
        from .engine import EngineOptions

        a = self.args
        remat = {"auto": "auto", "recompute": "full", "keep": "none"}[a.activation_memory]
        if a.gradient_checkpointing == "disabled":
            remat = "none"
        if a.scan_layers:
            log.info("scan_layers: the engine always runs one set of kernels per layer in a host loop; nothing to select")
        if a.projection_chunk_size:
            log.warning("projection_chunk_size=%d: projections are not tiled separately here; token rows are sharded "
                        "over tp and the MLP is tiled by mlp_chunk_size", a.projection_chunk_size)
        if a.attn_mechanism == "splash" or a.block_size_q != a.block_size_k:
            log.info("block_size_q / block_size_k: the tcgen05 attention kernels use fixed 128-row query tiles and "
                     "128-key tiles; the flags are validated and recorded in the resume signature only")
        return EngineOptions(
            cut_chunk_rows=a.cut_chunk_size or 4096, attention_options=a.attention_options, remat=remat,
            remat_group_size=a.remat_group_size, mlp_chunk_rows=a.mlp_chunk_size,
            train_lm_head="lm_head" not in frozen, train_embed="embed" not in frozen, train_norm="norm" not in frozen,
            loss_backend="logits" if a.loss_implementation == "pallas" else "cut")

    # ---- stage 6: parameters, optimizer ----
    @_guarded("load parameters")
    def build_model(self) -> None:
        a = self.args
        adamw = AdamWConfig(a.weight_decay, a.max_grad_norm, a.adam_beta1, a.adam_beta2, a.adam_epsilon)
        total = self.plan.total_steps
        if self.streaming and a.max_steps <= 0 and self.plan.steps_per_epoch is not None:
            total = buffered_streaming_schedule_total(self.plan.steps_per_epoch * max(1, int(a.num_train_epochs)))
        schedule = ScheduleConfig(a.learning_rate, a.learning_rate_end, a.scheduler, a.warmup_steps, total)
        weights_from = self.checkpoint.path if (self.checkpoint is not None and self.artifact_kind == "merged") \
            else (self.source if self.has_weights else None)
        data_ranks = self.lattice.size("dp") * self.lattice.size("fsdp")
        self.lora: LoraState | None = None
        tp, sp = self.lattice.size("tp"), self.lattice.size("sp")
        if self.use_lora_engine and data_ranks > 1:
            # adapters over a frozen base that is sharded like a trained model: the runtime serves
            # the weights (all-gather -> GEMM), adapters are replicated and their gradients all-reduced
            from ..api import TrainerConfig
            from ..parallel.fsdp import FsdpRuntime
            from .lora_engine import LoraLayerwiseEngine

            tcfg = TrainerConfig(micro_batch_rows=a.micro_batch_rows or a.total_batch_size // data_ranks, adamw=adamw,
                                 schedule=schedule, seed=a.seed, fused_collectives=a.fused_collectives,
                                 cut_chunk_rows=a.cut_chunk_size or 4096)
            self.runtime = FsdpRuntime(self.cfg, tcfg, self.device, group=self.lattice.group(("dp", "fsdp")),
                                       trainable=False)
            if weights_from is not None:
                hfio.load_sharded_parameters(weights_from, self.runtime)
            self.params = None
            self.lora = LoraState.init(self.cfg, a.lora_rank, seed=a.seed, dtype=self.param_dtype, device=self.device)
            if self.checkpoint is not None and self.artifact_kind == "peft-adapter":
                self.lora.load_peft_tensors(st.load_file(self.checkpoint.path / "adapter_model.safetensors"))
            producer = LoraLayerwiseEngine(self.cfg, self.runtime, self.lora, self.engine_options())
            self.step_fn = TrainStep(None, producer, adamw, schedule, extra_regions=producer.extra_regions(),
                                     train_base=False)
        elif self.use_engine and (data_ranks > 1 or tp > 1 or sp > 1):
            from ..api import TrainerConfig
            from ..parallel.fsdp import FsdpRuntime
            from .engine import EngineOptions, LayerwiseEngine

            tcfg = TrainerConfig(micro_batch_rows=a.micro_batch_rows or a.total_batch_size // data_ranks, adamw=adamw,
                                 schedule=schedule, seed=a.seed, fused_collectives=a.fused_collectives,
                                 cut_chunk_rows=a.cut_chunk_size or 4096, tp=tp)
            frozen = a.frozen_parameter_components
            options = self.engine_options(frozen)
            if tp > 1 and (frozen or options.loss_backend != "cut"):
                raise ValueError("tensor parallelism runs the vocabulary-parallel cut cross-entropy with every "
                                 "component trainable: --frozen_parameters and --loss_implementation pallas need tp = 1")
            # parameters, gradients and optimizer state are sharded over dp x fsdp (a dp replica
            # would only cost memory); tensor-parallel ranks hold slices of every projection
            data_group = self.lattice.group(("dp", "fsdp", "sp") if sp > 1 else ("dp", "fsdp"))
            if sp > 1 and tp > 1:
                from ..parallel.tp import tp_local_config
                from .sp_engine import sp_tp_engine

                tp_group = self.lattice.group(("tp",))
                self.runtime = FsdpRuntime(tp_local_config(self.cfg, tp), tcfg, self.device, group=data_group,
                                           full_cfg=self.cfg, tp_group=tp_group)
                engine = sp_tp_engine(self.cfg, tp_group, self.lattice.group(("sp",)), self.runtime, options,
                                      fused=a.fused_collectives, layout=a.sp_layout)
            elif sp > 1:
                from .sp_engine import SpLayerwiseEngine

                self.runtime = FsdpRuntime(self.cfg, tcfg, self.device, group=data_group, frozen=frozen)
                engine = SpLayerwiseEngine(self.cfg, self.lattice.group(("sp",)), self.runtime, options,
                                           fused=a.fused_collectives, layout=a.sp_layout)
            elif tp > 1:
                from ..parallel.tp import tp_local_config
                from .tp_engine import TpLayerwiseEngine

                tp_group = self.lattice.group(("tp",))
                self.runtime = FsdpRuntime(tp_local_config(self.cfg, tp), tcfg, self.device, group=data_group,
                                           full_cfg=self.cfg, tp_group=tp_group)
                engine = TpLayerwiseEngine(self.cfg, tp_group, self.runtime, options, fused=a.fused_collectives)
            else:
                self.runtime = FsdpRuntime(self.cfg, tcfg, self.device, group=data_group, frozen=frozen)
                engine = LayerwiseEngine(self.cfg, self.runtime, options)
            if weights_from is not None:
                hfio.load_sharded_parameters(weights_from, self.runtime)
            self.step_fn = self.runtime.make_step(engine)
            self.params = None
        else:
            self.runtime = None
            if weights_from is not None:
                self.params = ModelParams(self.cfg, self.param_dtype, "cpu")
                hfio.load_parameters(weights_from, self.params)
            else:
                log.warning("no *.safetensors in %s: initialising N(0, %g) weights", self.source,
                            self.cfg.initializer_range)
                self.params = ModelParams.init_random(self.cfg, a.seed, self.param_dtype)
            self.params.to(self.device)
            frozen = a.frozen_parameter_components if not a.lora else ()
            if self.use_engine:
                from .engine import EngineOptions, LayerwiseEngine, LocalProvider

                grad_dtype = torch.float32 if a.gradient_accumulation_steps > 1 else torch.bfloat16
                producer = LayerwiseEngine(self.cfg, LocalProvider(self.params, grad_dtype), self.engine_options(frozen))
                self.step_fn = TrainStep(self.params, producer, adamw, schedule, frozen=frozen)
            else:
                opts = ForwardOptions(
                    attn_mechanism="vanilla" if (a.attn_mechanism == "vanilla" or not self.cuda) else "efficient",
                    gradient_checkpointing=a.gradient_checkpointing == "nothing_saveable", mlp_chunk_size=a.mlp_chunk_size,
                    attention_options=a.attention_options,
                    compute_dtype=torch.bfloat16 if a.dtype == "bfloat16" and self.cuda else self.param_dtype)
                extra = []
                if a.lora:
                    self.lora = LoraState.init(self.cfg, a.lora_rank, seed=a.seed, dtype=self.param_dtype,
                                               device=self.device, train_embed_and_lm_head=a.lora_train_embed_and_lm_head,
                                               base=self.params)
                    if self.checkpoint is not None and self.artifact_kind == "peft-adapter":
                        self.lora.load_peft_tensors(st.load_file(self.checkpoint.path / "adapter_model.safetensors"))
                if self.use_lora_engine:
                    from .engine import EngineOptions, LocalProvider
                    from .lora_engine import LoraLayerwiseEngine

                    producer = LoraLayerwiseEngine(self.cfg, LocalProvider(self.params, torch.bfloat16), self.lora,
                                                   self.engine_options())
                    extra = producer.extra_regions()
                else:
                    if a.lora:
                        opts.lora = self.lora
                        extra = [(t.detach(), t.dim() > 1, (lambda t=t: t.grad)) for _, t in self.lora.trainable()]
                    producer = AutogradProducer(self.params, opts, a.loss_implementation, a.loss_token_budget,
                                                a.cut_chunk_size, lora=self.lora)
                dp_group = rt.host_group() if (rt.process_count() > 1 and not self.cuda) else None
                self.step_fn = TrainStep(self.params, producer, adamw, schedule, frozen=frozen, dp_group=dp_group,
                                         extra_regions=extra, train_base=not a.lora)
        if self.checkpoint is not None and self.checkpoint.has_optimizer_state and self.action == "continue":
            self.load_optimizer_state(self.checkpoint.path, self.checkpoint.global_step)

    # ---- optimizer state <-> checkpoint ----
    def _state_entries(self) -> list[tuple[str, str, str, int]]:
        """``(path, kind, unit, tp slice)`` of every moment buffer of the sharded runtime, in file order."""
        r = self.runtime
        out = []
        for kind in ("mu", "nu"):
            for name in r.units:
                if r.tp_world == 1:
                    out.append((f"{kind}/{name}", kind, name, 0))
                else:       # one entry per tensor-parallel slice, in tp rank order
                    out += [(f"{kind}/{name}/tp{t}", kind, name, t) for t in range(r.tp_world)]
        return out

    def _sharded_state(self) -> bool:
        """The optimizer state lives in the sharded runtime (not in a ``FlatAdamW`` of this process)."""
        return self.runtime is not None and self.runtime.trainable

    def optimizer_state_layout(self) -> list[tuple[str, torch.dtype, tuple[int, ...]]]:
        if self._sharded_state():
            r = self.runtime
            return [("count", torch.int64, ())] + [(path, torch.bfloat16, (r.units[name].layout.numel,))
                                                    for path, _, name, _ in self._state_entries()]
        opt = self.step_fn.optimizer
        out: list[tuple[str, torch.dtype, tuple[int, ...]]] = [("count", torch.int64, ())]
        for i, (m, v) in enumerate(zip(opt.m, opt.v)):
            out += [(f"mu/{i:05d}", m.dtype, tuple(m.shape)), (f"nu/{i:05d}", v.dtype, tuple(v.shape))]
        return out

    def _owner_table(self) -> dict[tuple[int, int], int]:
        """Global rank of the process that is shard ``s`` of tensor-parallel slice ``t``."""
        if getattr(self, "_owners", None) is None:
            r = self.runtime
            mine = (r.tp_rank, r.rank, torch.distributed.get_rank())
            everyone = [None] * torch.distributed.get_world_size()
            torch.distributed.all_gather_object(everyone, mine)
            self._owners = {}
            for t, shard, g in everyone:
                self._owners.setdefault((t, shard), g)      # replicas (dp, sp) hold the same shard: the first serves
        return self._owners

    def optimizer_state_pieces(self):
        """Collective generator for ``hfio.export_optimizer_stream``: every moment buffer arrives at
        process 0 shard by shard (one point-to-point transfer per shard), so no process ever holds
        more than one shard of one unit beyond its own state
        (src/causal_trainer/checkpointing/huggingface.py:1517-1646)."""
        if not self._sharded_state():
            opt = self.step_fn.optimizer
            yield "count", iter([torch.tensor([opt.count], dtype=torch.int64)])
            for i, (m, v) in enumerate(zip(opt.m, opt.v)):
                yield f"mu/{i:05d}", iter([m.detach().reshape(-1)])
                yield f"nu/{i:05d}", iter([v.detach().reshape(-1)])
            return
        r = self.runtime
        dist_ = torch.distributed
        me = dist_.get_rank()
        owners = self._owner_table()
        yield "count", iter([torch.tensor([r.count], dtype=torch.int64)])

        def shards(kind: str, name: str, t: int):
            u = r.units[name]
            arena = r.m if kind == "mu" else r.v
            for shard in range(r.world):
                lo = shard * u.shard_elems
                valid = max(0, min(u.shard_elems, u.layout.numel - lo))
                owner = owners[(t, shard)]
                piece = None
                if owner == me:
                    piece = r.shard_view(name, of=arena)
                    if me != 0:
                        dist_.send(piece.contiguous(), dst=0)
                elif me == 0:
                    piece = torch.empty(u.shard_elems, dtype=torch.bfloat16, device=self.device)
                    dist_.recv(piece, src=owner)
                if valid and me == 0:
                    yield piece[:valid]
                elif valid:
                    yield None

        for path, kind, name, t in self._state_entries():
            yield path, shards(kind, name, t)

    def load_optimizer_state(self, path: Path, step: int) -> None:
        names = [p for p, _, _ in self.optimizer_state_layout()]
        with hfio.OptimizerCheckpoint(path, names, global_step=step) as ckpt:
            if self._sharded_state():
                r = self.runtime
                r.count = int(ckpt.tensor("count"))
                for entry, kind, name, t in self._state_entries():
                    if t != r.tp_rank:
                        continue
                    u = r.units[name]
                    lo = r.rank * u.shard_elems
                    piece = ckpt.flat_range(entry, lo, max(lo, min(lo + u.shard_elems, u.layout.numel)))
                    view = r.shard_view(name, of=r.m if kind == "mu" else r.v)
                    view.zero_()
                    view[:piece.numel()].copy_(piece)       # only this rank's bytes were read
                return
            opt = self.step_fn.optimizer
            opt.count = int(ckpt.tensor("count"))
            for i, (m, v) in enumerate(zip(opt.m, opt.v)):
                m.copy_(ckpt.tensor(f"mu/{i:05d}"))
                v.copy_(ckpt.tensor(f"nu/{i:05d}"))

    # ---- checkpoint bundles ----
    def save_bundle(self, destination: Path, step: int) -> None:
        a = self.args

        def export_model(dest: Path, cid: str) -> None:
            if self.artifact_kind == "peft-adapter":
                hfio.export_adapter_checkpoint(dest, self.lora, base_model_name_or_path=a.repo_id, checkpoint_id=cid,
                                               revision=a.revision)
                return
            source = hfio.TensorSource(self.cfg, params=self.params, runtime=self.runtime,
                                       transform=self.lora.export_transform() if self.lora is not None else None)
            hfio.export_hf_checkpoint(dest, source, checkpoint_id=cid, assets_from=self.processor_source)

        export_optimizer = None
        if a.save_optimizer_state:
            def export_optimizer(dest: Path, cid: str) -> None:
                hfio.export_optimizer_stream(dest, self.optimizer_state_layout(), self.optimizer_state_pieces(),
                                             global_step=step, checkpoint_id=cid)
        bundles.save_checkpoint_bundle(
            destination, export_model=export_model, export_optimizer=export_optimizer, artifact_kind=self.artifact_kind,
            global_step=step, total_steps=self.plan.total_steps, signature=self.signature,
            source_examples_seen=self.source_examples_seen, streaming_data_digest=self.stream_digest,
            training_complete=self.training_complete)

    # ---- stage 7: batches ----
    def global_batches(self) -> Iterator[Any]:
        a = self.args
        if not self.streaming:
            it = batching.iter_global_batches(self.dataset, self.plan, assistant_only_loss=a.uses_assistant_loss_mask,
                                              shuffle=a.shuffle, seed=a.seed, start_step=self.start_step)
        else:
            if a.dataset_format == "prepared":
                envelopes = prepared.iter_prepared_streaming_batches(
                    a.dataset_name, self.manifest, num_epochs=self.plan.epochs, window_size=a.packing_batch_size,
                    token=a.token, revision=self.prepared_revision)
            else:
                source = self.stream_source

                def factory(epoch: int):
                    s = source.shuffle(seed=a.seed, buffer_size=a.streaming_shuffle_buffer) if a.shuffle else source
                    if hasattr(s, "set_epoch"):
                        s.set_epoch(epoch)
                    return s

                envelopes = streaming.iter_streaming_batches(
                    factory, self.tokenizer, num_epochs=self.plan.epochs, dataset_text_field=a.dataset_text_field,
                    max_sequence_length=a.max_sequence_length, pad_token_id=self._pad_token_id(),
                    assistant_only_loss=a.assistant_only_loss, last_assistant_only_loss=a.last_assistant_only_loss,
                    endprompt=endprompt_settings(a), packing=a.packing, packing_batch_size=a.packing_batch_size,
                    retry_initial_delay=a.hf_retry_initial_delay, retry_max_delay=a.hf_retry_max_delay)
            ck = self.checkpoint
            it = streaming_batching.iter_streaming_global_batches(
                envelopes, self.plan, assistant_only_loss=a.uses_assistant_loss_mask, start_step=self.start_step,
                expected_source_examples_before=ck.source_examples_seen if ck else None,
                expected_stream_digest_before=ck.streaming_data_digest if ck else None)
        if a.maskgit_probability:
            it = maskgit.MaskGITBatchTransform(self.tokenizer, probability=a.maskgit_probability,
                                               seed=a.seed).batches(it, start_step=self.start_step)
        return it

    def vote_on_stream_batch(self, batch, error: BaseException | None) -> str:
        """One byte of status plus the batch digest from every rank: BATCH, EOF or ERROR must agree."""
        if error is not None:
            payload = b"E" + bytes(32)
        elif batch is None:
            payload = b"F" + bytes(32)
        else:
            payload = b"B" + streaming_batching.streaming_global_batch_digest(batch)
        votes = rt.host_allgather_bytes(payload, 33)
        kinds = {v[:1] for v in votes}
        if b"E" in kinds:
            raise error if error is not None else RuntimeError("another process failed while reading the stream")
        if len(kinds) != 1 or len({v for v in votes}) != 1:
            raise RuntimeError("processes disagree on the streaming batch (different data or end of stream)")
        return "eof" if batch is None else "batch"

    def to_device(self, data: dict[str, np.ndarray]) -> list[dict[str, torch.Tensor]]:
        """This rank's rows of a global batch as device micro-batches (pinned staging, async copies)."""
        a = self.args
        ranks = self.lattice.size("dp") * self.lattice.size("fsdp")
        idx = self.lattice.index_in(("dp", "fsdp")) if ranks > 1 else 0
        per_micro = a.total_batch_size // ranks
        micro = []
        split = batching.split_accumulation(data, a.gradient_accumulation_steps)
        for g in range(a.gradient_accumulation_steps):
            rows = {}
            if a.balance_rows and ranks > 1:
                # the same global batch on every rank; which rows a rank keeps is free, so they are dealt by
                # cost: the step ends when the slowest rank does
                costs = batching.attention_cost_per_row(
                    split["segment_ids"][g], split["attention_end"][g] if "attention_end" in split else None)
                keep = batching.balanced_row_assignment(costs, ranks)[idx]
            else:
                keep = np.arange(idx * per_micro, (idx + 1) * per_micro)
            for k, v in split.items():
                t = torch.from_numpy(np.ascontiguousarray(v[g][keep]))
                if self.cuda:
                    t = t.pin_memory().to(self.device, non_blocking=True)
                rows[k] = t
            sub = a.micro_batch_rows or per_micro
            longest = batching.longest_document(split["segment_ids"][g][keep])
            for r0 in range(0, per_micro, sub):
                micro.append({k: v[r0:r0 + sub] for k, v in rows.items()})
                micro[-1]["longest_document"] = longest      # host-side hint for block-sparse layers
        return micro

    def check_device_waits(self) -> None:
        """Collective (all ranks reach it at the same steps): reads the status word the bounded
        device waits write when they give up, and fails the run on every rank if any rank has a
        record.  Called only where metrics were just read back, so the device is idle."""
        from ..ops import lib as oplib

        rt.raise_if_any_process_error(oplib.poll_device_status() if self.cuda else None, "device wait")

    # ---- the loop ----
    def train(self) -> None:
        a = self.args
        out = Path(a.output_dir)
        if self.action == "complete":
            log.info("training is already complete at step %d", self.start_step)
            return
        if a.weight_distribution_log_steps:
            log.warning("weight_distribution_log_steps is accepted for command compatibility; weight histograms are "
                        "not logged (src/causal_trainer/training/runner.py:1760-1763 does the same)")
        if rt.process_index() == 0:
            out.mkdir(parents=True, exist_ok=True)
            (out / "training_args.json").write_text(json.dumps(
                {f.name: getattr(a, f.name) for f in dataclasses.fields(a)}, indent=2, sort_keys=True, default=str))
        rt.sync_processes("training-args-written")
        tracker = tlog.ThroughputTracker(self.cfg, a.max_sequence_length, rt.process_count())
        wandb_run = tlog.init_wandb(a) if rt.process_index() == 0 else None
        window = MetricWindow(a.async_dispatch_steps)
        profiler = tlog.StepProfiler(a.profile_steps, self.device if self.cuda else None,
                                     tokens_per_step=a.effective_batch_size * a.max_sequence_length,
                                     flops_per_token=self.cfg.flops_per_token(a.max_sequence_length),
                                     n_gpus=rt.process_count())
        step = self.start_step
        if self.action != "finalize":
            batches = batching.prefetch_map(self.global_batches(), lambda b: (b, self.to_device(
                b if isinstance(b, dict) else b.data)), prefetch_batches=a.prefetch_batches)
            it = iter(batches)
            while step < self.plan.total_steps:
                item, error = None, None
                try:
                    item = next(it)
                except StopIteration:
                    item = None
                except Exception as exc:  # noqa: BLE001
                    error = exc
                if self.streaming:
                    if self.vote_on_stream_batch(item[0] if item else None, error) == "eof":
                        break
                else:
                    # every rank takes part in the vote each iteration: a rank whose reader failed
                    # must not be left alone in it while its peers enter the step's collectives
                    rt.raise_if_any_process_error(error, "read batch")
                    if item is None:
                        break
                raw, micro = item
                t0 = time.monotonic()
                lr_position = None
                if self.streaming and a.max_steps <= 0 and self.plan.steps_per_epoch:
                    lr_position = streaming_schedule_position(
                        step - raw.epoch * self.plan.steps_per_epoch if hasattr(raw, "epoch") else step,
                        getattr(raw, "epoch", 0), self.plan.steps_per_epoch)
                profiler.begin()
                metrics = self.step_fn.run(micro, lr_position=lr_position)
                profiler.end()
                step += 1
                if hasattr(raw, "source_examples_seen"):
                    self.source_examples_seen, self.stream_digest = raw.source_examples_seen, raw.stream_digest
                window.push(step, metrics)
                tracker.step(a.effective_batch_size, time.monotonic() - t0)
                first_or_last = step == self.start_step + 1 or step == self.plan.total_steps
                if step % a.logging_steps == 0 or first_or_last:
                    latest = window.drain()
                    if self.cuda:
                        torch.cuda.synchronize(self.device)
                    self.check_device_waits()
                    tlog.log_step(latest, tracker, self.device if a.track_memory else None, wandb_run)
                if a.save_steps and step % a.save_steps == 0 and step < self.plan.total_steps:
                    window.drain()
                    self.check_device_waits()
                    self.save_bundle(out / f"checkpoint-{step}", step)
                    bundles.prune_periodic_exports(out, a.save_total_limit, self.signature)
            window.drain()
            self.check_device_waits()
        profile = profiler.finish()
        if profile is not None and rt.process_index() == 0:
            log.info("profiled %(profiled_steps)d steps: %(ms_per_step).2f ms/step, %(tokens_per_second).0f tok/s, "
                     "mfu %(mfu).3f (%(clock)s)", profile)
            (out / "profile_steps.json").write_text(json.dumps(profile, indent=2, sort_keys=True) + "\n")
        if self.streaming and not self.plan.has_exact_step_limit:
            self.training_complete = True
            self.plan = dataclasses.replace(self.plan, total_steps=step)
        self.save_bundle(out, step)
        rt.sync_processes("training-complete")
        if wandb_run is not None:
            wandb_run.finish()


def main(argv: list[str] | None = None) -> int:
    args = parse_args(argv)
    run = TrainingRun(args)
    run.resolve_model()
    run.load_data()
    run.discover_resume()
    run.build_model()
    run.train()
    return 0
