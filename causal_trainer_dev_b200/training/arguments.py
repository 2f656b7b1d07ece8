"""``causal-train`` flag surface.

The command line is the reference's (src/causal_trainer/training/arguments.py:205-725): every
option is spelled both ``--a-b`` and ``--a_b``; booleans accept ``--x``, ``--x True`` and
``--no-x``; a mesh that starts with ``-1`` may be passed as a separate word; block sizes, the
MLP tile and ``scan_layers`` get the same derived defaults; the same cross-field rules are
enforced.  The table below is the single source of truth: parser, dataclass and help text
are generated from it.

Differences, all additive: the non-TPU refusal is gone (this framework runs on CUDA), the
default mesh still reads ``-1,1,1,4,1`` (dp, fsdp, ep, tp, sp), and three options exist
only here (``--fused_collectives``, ``--micro_batch_rows``, ``--optimizer_moment_dtype``).
"""
from __future__ import annotations

import argparse
import math
import sys
from dataclasses import dataclass, field, make_dataclass
from pathlib import Path
from typing import Any

from ..models.moba import AttentionOptions

FROZEN_PARAMETER_COMPONENTS = ("lm_head", "embed", "norm")
_MESH_FLAGS = {"--sharding-axis", "--sharding_axis", "--sharding-dcn-axis", "--sharding_dcn_axis"}


def parse_bool(value: str | bool) -> bool:
    if isinstance(value, bool):
        return value
    text = value.strip().lower()
    if text in ("1", "true", "yes", "y", "on"):
        return True
    if text in ("0", "false", "no", "n", "off"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean value, got {value!r}")


def parse_frozen_parameter_components(value: str | None) -> tuple[str, ...]:
    if value is None:
        return ()
    wanted = {part.strip() for part in value.replace(",", "|").split("|")} - {""}
    if not wanted:
        raise ValueError("frozen_parameters must name at least one component")
    unknown = wanted - set(FROZEN_PARAMETER_COMPONENTS)
    if unknown:
        raise ValueError("unsupported frozen_parameters components: " + ", ".join(sorted(unknown)))
    return tuple(c for c in FROZEN_PARAMETER_COMPONENTS if c in wanted)


@dataclass(frozen=True)
class Flag:
    name: str
    kind: Any                      # type callable, "bool", or "tribool" (bool with None default)
    default: Any = None
    help: str = ""
    choices: tuple | None = None
    required: bool = False


FLAGS: tuple[Flag, ...] = (
    # ---- model / tokenizer / dataset sources ----
    Flag("repo_id", str, required=True, help="Local checkpoint directory or Hugging Face repository ID."),
    Flag("dataset_name", str, required=True, help="Local dataset file/directory or Hugging Face dataset ID."),
    Flag("maskgit_probability", float, 0.0,
         "Probability per complete assistant image grid of MaskGIT instead of AR training; 0 disables it."),
    Flag("dataset_format", str, "raw", "raw: tokenize/pack while training; prepared: a causal-prepare artifact.",
         choices=("raw", "prepared")),
    Flag("dataset_split", str, "train"),
    Flag("dataset_text_field", str, "text", "Use 'messages' for conversational records."),
    Flag("dataset_streaming", "bool", False, "Stream records without materializing the split."),
    Flag("dataset_config_name", str, None, "Optional dataset configuration/subset name."),
    Flag("dataset_revision", str, None, "Optional dataset revision, independent of the model revision."),
    Flag("streaming_shuffle_buffer", int, 10_000, "In-memory shuffle buffer used for streaming datasets."),
    Flag("hf_retry_initial_delay", float, 1.0, "Initial delay in seconds before retrying a transient read failure."),
    Flag("hf_retry_max_delay", float, 60.0, "Maximum delay in seconds between retries."),
    Flag("processor_repo_id", str, None),
    Flag("processor_revision", str, None, "Revision of a separately provided processor repository."),
    Flag("output_dir", Path, Path("causal-trainer-output")),
    Flag("revision", str, None),
    Flag("token", str, None, "HF token; prefer the HF_TOKEN environment variable."),
    # ---- preprocessing ----
    Flag("max_sequence_length", int, 4096),
    Flag("packing", "bool", False, "Pack multiple records into fixed-length rows."),
    Flag("packing_batch_size", int, 1000, "Per-process packing window; its final short window is retained."),
    Flag("assistant_only_loss", "bool", False, "Supervise only chat-template generation spans."),
    Flag("last_assistant_only_loss", "bool", False, "Supervise only the final generation span of each record."),
    Flag("endprompt_enable", "bool", False, "Append a terminal anchor prompt to records."),
    Flag("endprompt_logical_length", int, None, "Maximum logical context length for terminal-anchor positions."),
    Flag("endprompt_logical_length_min", int, None, "Minimum logical context length."),
    Flag("endprompt_prompts", str, "This is the end of text, please pay attention here",
         "Terminal prompt text; separate multiple prompts with '||'."),
    Flag("endprompt_prompt_loss_weight", float, 0.1),
    Flag("endprompt_context_loss_weight", float, 1.0),
    Flag("preprocessing_num_workers", int, None, "Tokenizer worker processes inside each training process."),
    Flag("preprocessing_mode", str, "shard_then_merge",
         "Shard source rows across processes and merge the packed arrays, or preprocess everything everywhere.",
         choices=("shard_then_merge", "replicated")),
    # ---- attention ----
    Flag("attn_mechanism", str, "efficient",
         "efficient: the sm_100a flash kernels; vanilla: O(S^2) reference; splash: accepted, validated with the "
         "reference block rules and run by the flash kernels.", choices=("splash", "vanilla", "efficient")),
    Flag("attention_method", str, "dense", "Opt-in attention approximation.", choices=("dense", "moba")),
    Flag("attention_sparse_backend", str, "auto",
         "auto/pallas: native sparse kernels on GPU; reference: the indexed-attention oracle.",
         choices=("auto", "pallas", "reference")),
    Flag("attention_query_chunk_size", int, 128, "Sparse attention query workspace tile."),
    Flag("attention_key_chunk_size", int, 512, "Sparse attention key workspace tile."),
    Flag("moba_block_size", int, 4096, "Sample-relative MoBA routing block size."),
    Flag("moba_top_k", int, 12, "MoBA block budget per query/head, including its current block."),
    Flag("attention_dense_prefix_layers", int, 0, "Leading layers kept dense."),
    Flag("attention_dense_suffix_layers", int, 0, "Trailing layers kept dense."),
    Flag("attention_dense_after_step", int, None, "Use dense attention from this zero-based optimizer step."),
    Flag("block_size_q", int, None, "Query block size (auto: 128 below 131072 tokens, 256 below 262144, 512 below "
         "524288, 1024 from there on)."),
    Flag("block_size_k", int, None, "Key block size (same automatic ladder)."),
    # ---- loss / memory ----
    Flag("loss_token_budget", int, 128, "Maximum local token rows of a chunked-logits slab."),
    Flag("loss_implementation", str, "auto",
         "cut: projection-fused kernels; pallas: chunked logits; xla: PyTorch oracle; auto: cut.",
         choices=("auto", "xla", "pallas", "cut")),
    Flag("mlp_chunk_size", int, None, "Per-sequence MLP tile; auto: 1024 for full-parameter training at contexts of "
         "4096 to 131071 tokens, off otherwise and always off for LoRA and sequence-parallel runs."),
    Flag("scan_layers", "tribool", None, "Layer-loop representation flag kept for command compatibility (auto: on "
         "for full-parameter training at contexts of at least 524288 tokens, and for single-row bf16 runs at 131072 "
         "tokens, 262144 with MoBA; part of the resume identity)."),
    Flag("projection_chunk_size", int, 0, "SP-local token rows per projection tile; 0 disables."),
    Flag("remat_group_size", int, 1, "Layers per rematerialized group."),
    Flag("cut_chunk_size", int, 0, "Local token rows per Cut loss chunk; 0 keeps the default."),
    Flag("async_dispatch_steps", int, 2, "Steps whose metrics may stay on the device without a host sync."),
    Flag("prefetch_batches", int, 1, "Converted global batches prepared ahead."),
    # ---- optimisation ----
    Flag("total_batch_size", int, 32, "Global micro-batch size."),
    Flag("gradient_accumulation_steps", int, 1),
    Flag("learning_rate", float, 2e-5),
    Flag("learning_rate_end", float, 0.0),
    Flag("scheduler", str, "cosine", choices=("cosine", "linear", "constant")),
    Flag("warmup_steps", int, 0),
    Flag("weight_decay", float, 0.0),
    Flag("max_grad_norm", float, 1.0),
    Flag("adam_beta1", float, 0.9),
    Flag("adam_beta2", float, 0.999),
    Flag("adam_epsilon", float, 1e-8),
    Flag("num_train_epochs", float, 1.0),
    Flag("max_steps", int, -1),
    Flag("shuffle", "bool", True, "Shuffle records deterministically each epoch."),
    Flag("seed", int, 42),
    Flag("gradient_checkpointing", str, "nothing_saveable", choices=("nothing_saveable", "disabled")),
    # ---- PEFT / freezing ----
    Flag("lora", "bool", False, "Train rank-decomposition adapters on the seven decoder projections."),
    Flag("lora_rank", int, 256),
    Flag("lora_train_embed_and_lm_head", "bool", False, "Also update the embedding and LM head."),
    Flag("lora_save_adapter_only", "bool", False, "Save a PEFT-compatible adapter checkpoint."),
    Flag("frozen_parameters", str, None, "Pipe- or comma-separated components to freeze: lm_head, embed, norm."),
    # ---- precision / distribution ----
    Flag("param_dtype", str, "bfloat16", choices=("bfloat16", "float32")),
    Flag("dtype", str, "bfloat16", choices=("bfloat16", "float32")),
    Flag("sharding_axis", str, "-1,1,1,4,1", "dp,fsdp,ep,tp,sp mesh dimensions."),
    Flag("sharding_dcn_axis", str, None, "Optional explicit cross-node mesh dimensions."),
    Flag("coordinator_address", str, None),
    Flag("num_processes", int, None),
    Flag("process_id", int, None),
    Flag("local_device_ids", str, None, "Comma-separated local device IDs."),
    Flag("distributed", "bool", True, "Auto-initialize torch.distributed from the environment."),
    # ---- checkpoint / logging ----
    Flag("save_steps", int, 0, "Periodic export interval; 0 disables it."),
    Flag("save_total_limit", int, 1, "Periodic exports to retain; 0 keeps all."),
    Flag("save_optimizer_state", "bool", False, "Save optimizer state with every checkpoint."),
    Flag("use_wandb", "bool", False, "Log scalar metrics to Weights & Biases on process zero."),
    Flag("wandb_project", str, "causal-trainer"),
    Flag("wandb_run_name", str, None),
    Flag("logging_steps", int, 10, "Host-log interval; the first and final update are always logged."),
    Flag("track_memory", "bool", False, "Log device memory statistics."),
    Flag("weight_distribution_log_steps", int, 0),
    # ---- this framework only ----
    Flag("fused_collectives", "bool", True, "In-kernel NVLink collectives (False: NCCL-only baseline path)."),
    Flag("micro_batch_rows", int, 0, "Rows per device micro-batch inside one step (0: all local rows at once)."),
    Flag("profile_steps", int, 0, "Device-time this many steps with CUDA events and report tokens/s and MFU."),
    Flag("balance_rows", "bool", True, "Deal the rows of every global batch to the data ranks by attention cost (equal "
         "rows, near-equal visible query-key pairs per rank) instead of by position."),
    Flag("sp_layout", str, "contiguous", "Which tokens of a row a sequence-parallel rank computes: contiguous (one "
         "slice per rank) or zigzag (chunks r and 2 sp - 1 - r of 2 sp chunks, equal causal attention work on every rank; "
         "rows that do not split into whole 128-token tiles use contiguous slices).", choices=("contiguous", "zigzag")),
    Flag("activation_memory", str, "auto", "What the CUDA engine does with layer activations: auto keeps those of as "
         "many layers as fit in free HBM and recomputes the rest; recompute always recomputes (the meaning of "
         "gradient_checkpointing=nothing_saveable on small-memory devices); keep never recomputes. "
         "gradient_checkpointing=disabled forces keep.", choices=("auto", "recompute", "keep")),
)

_FIELD_ORDER = [f.name for f in FLAGS]


def _spellings(name: str) -> tuple[str, ...]:
    dashed, under = f"--{name.replace('_', '-')}", f"--{name}"
    return (dashed,) if dashed == under else (dashed, under)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        prog="causal-train",
        description="Distributed full-parameter or LoRA training of Llama-family decoders on B200.",
        formatter_class=argparse.ArgumentDefaultsHelpFormatter,
    )
    for flag in FLAGS:
        if flag.kind in ("bool", "tribool"):
            parser.add_argument(*_spellings(flag.name), dest=flag.name, nargs="?", const=True, default=flag.default,
                                type=parse_bool, help=flag.help or None)
            parser.add_argument(f"--no-{flag.name.replace('_', '-')}", dest=flag.name, action="store_false",
                                default=flag.default if flag.kind == "tribool" else argparse.SUPPRESS)
        else:
            kw: dict[str, Any] = dict(dest=flag.name, type=flag.kind, default=flag.default, help=flag.help or None)
            if flag.choices:
                kw["choices"] = flag.choices
            if flag.required:
                kw["required"] = True
                kw.pop("default")
            parser.add_argument(*_spellings(flag.name), **kw)
    return parser


def _annotation(flag: Flag) -> Any:
    return bool if flag.kind == "bool" else (object if flag.kind == "tribool" else flag.kind)


class _ArgumentViews:
    """Derived properties mixed into the generated dataclass."""

    @property
    def attention_options(self) -> AttentionOptions | None:
        opts = AttentionOptions(
            method=self.attention_method, backend=self.attention_sparse_backend,
            query_chunk_size=self.attention_query_chunk_size, key_chunk_size=self.attention_key_chunk_size,
            moba_block_size=self.moba_block_size, moba_top_k=self.moba_top_k,
            dense_prefix_layers=self.attention_dense_prefix_layers,
            dense_suffix_layers=self.attention_dense_suffix_layers, dense_after_step=self.attention_dense_after_step,
        )
        return None if opts.method == "dense" else opts

    @property
    def effective_batch_size(self) -> int:
        return self.total_batch_size * self.gradient_accumulation_steps

    @property
    def uses_assistant_loss_mask(self) -> bool:
        return self.assistant_only_loss or self.last_assistant_only_loss

    @property
    def uses_raw_streaming(self) -> bool:
        return self.dataset_format == "raw" and self.dataset_streaming

    @property
    def effective_processor_revision(self) -> str | None:
        return self.revision if self.processor_repo_id is None else self.processor_revision

    @property
    def effective_endprompt_logical_length(self) -> int:
        return self.max_sequence_length if self.endprompt_logical_length is None else self.endprompt_logical_length

    @property
    def effective_endprompt_logical_length_min(self) -> int:
        if self.endprompt_logical_length_min is None:
            return self.effective_endprompt_logical_length
        return self.endprompt_logical_length_min

    @property
    def endprompt_prompt_texts(self) -> tuple[str, ...]:
        return tuple(p for p in self.endprompt_prompts.split("||") if p)

    @property
    def frozen_parameter_components(self) -> tuple[str, ...]:
        return parse_frozen_parameter_components(self.frozen_parameters)

    @property
    def mesh_sizes(self) -> tuple[int, ...]:
        return tuple(int(x.strip()) for x in self.sharding_axis.split(","))


TrainingArguments = make_dataclass(
    "TrainingArguments",
    [(f.name, _annotation(f), field(default=f.default)) if not f.required else (f.name, _annotation(f)) for f in
     sorted(FLAGS, key=lambda f: not f.required)],
    bases=(_ArgumentViews,),
    frozen=True,
)
TrainingArguments.__doc__ = "Frozen view of every causal-train option after defaults and validation."


def automatic_attention_block_size(sequence_length: int) -> int:
    if sequence_length < 131072:
        return 128
    if sequence_length < 262144:
        return 256
    if sequence_length < 524288:
        return 512
    return 1024


def _join_negative_mesh(raw: list[str]) -> list[str]:
    # argparse reads "-1,1,1,4,1" after --sharding_axis as another option; glue it on.
    out = list(raw)
    for i in range(len(out) - 1):
        if out[i] in _MESH_FLAGS and out[i + 1].lstrip().startswith("-1") and "," in out[i + 1]:
            out[i] = f"{out[i]}={out[i + 1]}"
            out[i + 1] = ""
    return [x for x in out if x]


def _fail(msg: str) -> None:
    raise ValueError(msg)


def _validate(a: Any) -> None:
    _ = a.attention_options
    if a.projection_chunk_size < 0 or a.cut_chunk_size < 0 or a.remat_group_size < 1:
        _fail("projection_chunk_size and cut_chunk_size must be nonnegative; remat_group_size must be positive")
    explicit_memory = a.projection_chunk_size > 0 or a.cut_chunk_size > 0 or a.remat_group_size > 1
    if explicit_memory and (a.lora or a.frozen_parameters):
        _fail("projection_chunk_size, remat_group_size and cut_chunk_size require full-parameter training")
    if a.projection_chunk_size > 0:
        if a.dtype != "bfloat16" or a.param_dtype != "bfloat16":
            _fail("projection_chunk_size requires BF16 compute and parameters")
        if a.attn_mechanism != "efficient" or a.total_batch_size != 1:
            _fail("projection_chunk_size requires efficient attention and total_batch_size=1")
    if a.remat_group_size > 1 and (not a.scan_layers or a.gradient_checkpointing != "nothing_saveable"):
        _fail("remat_group_size>1 requires scan_layers=True and gradient_checkpointing=nothing_saveable")
    if a.cut_chunk_size > 0 and a.loss_implementation not in ("auto", "cut"):
        _fail("cut_chunk_size requires the Cut loss backend")
    if a.max_sequence_length <= 1:
        _fail("max_sequence_length must be greater than one")
    if a.num_train_epochs <= 0 and a.max_steps <= 0:
        _fail("num_train_epochs must be positive unless max_steps is set")
    if a.uses_raw_streaming and a.max_steps <= 0 and not float(a.num_train_epochs).is_integer():
        _fail("streaming datasets require an integer num_train_epochs unless max_steps is set")
    if a.total_batch_size <= 0 or a.gradient_accumulation_steps <= 0:
        _fail("batch size and gradient accumulation must be positive")
    if a.packing_batch_size <= 0 or a.logging_steps <= 0:
        _fail("packing_batch_size and logging_steps must be positive")
    if a.streaming_shuffle_buffer <= 0:
        _fail("streaming_shuffle_buffer must be positive")
    delays = (a.hf_retry_initial_delay, a.hf_retry_max_delay)
    if any(not math.isfinite(d) or d <= 0 for d in delays):
        _fail("Hugging Face retry delays must be positive")
    if a.hf_retry_initial_delay > a.hf_retry_max_delay:
        _fail("hf_retry_initial_delay cannot exceed hf_retry_max_delay")
    if a.uses_raw_streaming and a.preprocessing_num_workers is not None:
        _fail("preprocessing_num_workers is not supported with dataset_streaming")
    if a.preprocessing_num_workers is not None and a.preprocessing_num_workers <= 0:
        _fail("preprocessing_num_workers must be positive when provided")
    if a.warmup_steps < 0 or a.weight_distribution_log_steps < 0 or a.seed < 0:
        _fail("warmup_steps, weight_distribution_log_steps, and seed cannot be negative")
    if a.block_size_q <= 0 or a.block_size_k <= 0 or a.loss_token_budget <= 0:
        _fail("attention block sizes and loss_token_budget must be positive")
    if a.mlp_chunk_size < 0:
        _fail("mlp_chunk_size cannot be negative")
    if a.async_dispatch_steps <= 0 or a.prefetch_batches < 0:
        _fail("async_dispatch_steps must be positive and prefetch_batches cannot be negative")
    if a.lora_rank <= 0:
        _fail("lora_rank must be positive")
    if a.lora_train_embed_and_lm_head and not a.lora:
        _fail("lora_train_embed_and_lm_head requires --lora True")
    if a.lora_save_adapter_only and not a.lora:
        _fail("lora_save_adapter_only requires --lora True")
    if a.save_steps < 0 or a.save_total_limit < 0:
        _fail("checkpoint intervals and limits must be non-negative")
    if a.learning_rate <= 0 or a.learning_rate_end < 0:
        _fail("learning rates must be non-negative and the initial rate must be positive")
    if a.learning_rate_end > a.learning_rate and a.scheduler != "constant":
        _fail("learning_rate_end cannot exceed learning_rate for a decay schedule")
    if not math.isfinite(a.maskgit_probability) or not 0.0 <= a.maskgit_probability <= 1.0:
        _fail("maskgit_probability must be between 0 and 1")
    if a.maskgit_probability:
        if a.dataset_format == "raw" and a.dataset_text_field != "messages":
            _fail("maskgit_probability requires --dataset_text_field messages")
        if a.attn_mechanism == "splash" or a.attention_method != "dense":
            _fail("MaskGIT requires dense attention with the efficient or vanilla backend")
    if a.assistant_only_loss and a.last_assistant_only_loss:
        _fail("assistant_only_loss and last_assistant_only_loss are mutually exclusive")
    if a.dataset_format == "raw" and a.uses_assistant_loss_mask and a.dataset_text_field != "messages":
        option = "last_assistant_only_loss" if a.last_assistant_only_loss else "assistant_only_loss"
        _fail(f"{option} requires --dataset_text_field messages")
    if a.endprompt_enable:
        hi, lo = a.effective_endprompt_logical_length, a.effective_endprompt_logical_length_min
        if hi < a.max_sequence_length or lo < a.max_sequence_length:
            _fail("EndPrompt logical lengths must be at least max_sequence_length")
        if lo > hi:
            _fail("endprompt_logical_length_min cannot exceed endprompt_logical_length")
        if not a.endprompt_prompt_texts:
            _fail("endprompt_prompts must contain at least one non-empty prompt")
        weights = (a.endprompt_context_loss_weight, a.endprompt_prompt_loss_weight)
        if any(not math.isfinite(w) or w < 0.0 for w in weights):
            _fail("EndPrompt loss weights must be finite and non-negative")
        if not any(w > 0.0 for w in weights):
            _fail("at least one EndPrompt loss weight must be positive")
    if a.lora and a.save_optimizer_state and not a.lora_save_adapter_only:
        _fail("LoRA optimizer state can be saved only with --lora_save_adapter_only True")
    if a.micro_batch_rows < 0 or a.profile_steps < 0:
        _fail("micro_batch_rows and profile_steps cannot be negative")


def parse_args(argv: list[str] | None = None):
    raw = _join_negative_mesh(list(sys.argv[1:] if argv is None else argv))
    ns = build_parser().parse_args(raw)
    auto_block = automatic_attention_block_size(ns.max_sequence_length)
    if ns.block_size_q is None:
        ns.block_size_q = auto_block
    if ns.block_size_k is None:
        ns.block_size_k = auto_block
    if ns.mlp_chunk_size is None:
        try:
            requested_sp = int(ns.sharding_axis.split(",")[-1].strip())
        except (AttributeError, ValueError):
            requested_sp = -1
        tiled = not ns.lora and requested_sp == 1 and 4096 <= ns.max_sequence_length < 131072
        ns.mlp_chunk_size = 1024 if tiled else 0
    if ns.scan_layers is None:
        mid_context = (
            ns.attn_mechanism == "efficient" and ns.total_batch_size == 1
            and ns.dtype == ns.param_dtype == "bfloat16"
            and (ns.max_sequence_length == 131072
                 or (ns.attention_method == "moba" and ns.max_sequence_length == 262144))
        )
        ns.scan_layers = (
            not ns.lora and (ns.max_sequence_length >= 524288 or mid_context) and ns.mlp_chunk_size == 0
            and ns.gradient_checkpointing == "nothing_saveable"
        )
    if ns.frozen_parameters is not None:
        ns.frozen_parameters = "|".join(parse_frozen_parameter_components(ns.frozen_parameters))
    args = TrainingArguments(**{name: getattr(ns, name) for name in _FIELD_ORDER})
    _validate(args)
    return args


__all__ = ["FLAGS", "TrainingArguments", "build_parser", "parse_args", "parse_bool",
           "parse_frozen_parameter_components", "automatic_attention_block_size"]
