"""``causal-prepare``: offline tokenisation + packing into a prepared dataset artifact.

Writes ``data/shard-XXXXX-of-XXXXX.parquet`` files and ``causal-trainer-prepared.json`` into an
empty output directory, optionally uploading the folder to a Hub dataset repository.  The
source split is cut into ``num_shards`` contiguous intervals; each interval is tokenised and
packed independently with a *global* example index offset so EndPrompt lengths do not depend
on the shard count.  The manifest is written last (through ``.incomplete`` + rename) and the
output is removed again if anything fails (src/causal_trainer/prepare.py:433-538).  This
module imports neither torch nor any GPU code.
"""
from __future__ import annotations

import argparse
import hashlib
import math
import shutil
import sys
from dataclasses import dataclass
from pathlib import Path
from typing import Any


from .data.pipeline import (load_training_split, packed_dataset_to_arrays, select_process_shard,
                            prepare_training_dataset)
from .data.prepared import (PREPARED_MANIFEST_FILENAME, PreparedDatasetManifest, PreparedShard, field_names, sha256_file,
                            validate_prepared_batch, write_prepared_manifest, write_prepared_shard)
from .data.preprocessing import EndPromptSettings
from .data.tokenizer import TrainingTokenizer

TOKENIZER_GLOBS = ("tokenizer.json", "tokenizer_config.json", "special_tokens_map.json", "chat_template.json",
                   "chat_template.jinja", "chat_templates/*.jinja", "added_tokens.json", "vocab.json", "merges.txt",
                   "tokenizer.model")


def _parse_bool(value: str | bool) -> bool:
    if isinstance(value, bool):
        return value
    text = value.strip().lower()
    if text in ("1", "true", "yes", "y", "on"):
        return True
    if text in ("0", "false", "no", "n", "off"):
        return False
    raise argparse.ArgumentTypeError(f"expected a boolean value, got {value!r}")


@dataclass(frozen=True)
class PrepareArguments:
    dataset_name: str
    dataset_split: str
    dataset_text_field: str
    dataset_config_name: str | None
    dataset_revision: str | None
    tokenizer_name_or_path: str
    tokenizer_revision: str | None
    token: str | None
    output_dir: Path
    num_shards: int
    max_sequence_length: int
    packing: bool
    packing_batch_size: int
    assistant_only_loss: bool
    last_assistant_only_loss: bool
    endprompt_enable: bool
    endprompt_logical_length: int | None
    endprompt_logical_length_min: int | None
    endprompt_prompts: str
    endprompt_prompt_loss_weight: float
    endprompt_context_loss_weight: float
    preprocessing_num_workers: int | None
    hub_repo_id: str | None
    hub_revision: str | None
    private: bool

    @property
    def uses_assistant_loss_mask(self) -> bool:
        return self.assistant_only_loss or self.last_assistant_only_loss

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


_OPTIONS: tuple[tuple[str, Any, Any, bool], ...] = (
    # name, type ("bool" for flags), default, required
    ("dataset_name", str, None, True), ("dataset_split", str, "train", False),
    ("dataset_text_field", str, "text", False), ("dataset_config_name", str, None, False),
    ("dataset_revision", str, None, False), ("tokenizer_name_or_path", str, None, True),
    ("tokenizer_revision", str, None, False), ("token", str, None, False), ("output_dir", Path, None, True),
    ("num_shards", int, 1, False), ("max_sequence_length", int, 4096, False), ("packing", "bool", False, False),
    ("packing_batch_size", int, 1000, False), ("assistant_only_loss", "bool", False, False),
    ("last_assistant_only_loss", "bool", False, False), ("endprompt_enable", "bool", False, False),
    ("endprompt_logical_length", int, None, False), ("endprompt_logical_length_min", int, None, False),
    ("endprompt_prompts", str, "This is the end of text, please pay attention here", False),
    ("endprompt_prompt_loss_weight", float, 0.1, False), ("endprompt_context_loss_weight", float, 1.0, False),
    ("preprocessing_num_workers", int, None, False), ("hub_repo_id", str, None, False),
    ("hub_revision", str, None, False), ("private", "bool", False, False),
)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        prog="causal-prepare",
        description="Tokenize and optionally pack a dataset into Parquet shards for causal-train.",
        formatter_class=argparse.ArgumentDefaultsHelpFormatter,
    )
    for name, kind, default, required in _OPTIONS:
        dashed, under = f"--{name.replace('_', '-')}", f"--{name}"
        flags = (dashed,) if dashed == under else (dashed, under)
        if kind == "bool":
            parser.add_argument(*flags, dest=name, nargs="?", const=True, default=default, type=_parse_bool)
            parser.add_argument(f"--no-{name.replace('_', '-')}", dest=name, action="store_false")
        elif required:
            parser.add_argument(*flags, dest=name, type=kind, required=True)
        else:
            parser.add_argument(*flags, dest=name, type=kind, default=default)
    return parser


def parse_args(argv: list[str] | None = None) -> PrepareArguments:
    a = PrepareArguments(**vars(build_parser().parse_args(argv)))
    if a.num_shards <= 0:
        raise ValueError("num_shards must be positive")
    if a.max_sequence_length <= 1:
        raise ValueError("max_sequence_length must be greater than one")
    if a.packing_batch_size <= 0:
        raise ValueError("packing_batch_size must be positive")
    if a.preprocessing_num_workers is not None and a.preprocessing_num_workers <= 0:
        raise ValueError("preprocessing_num_workers must be positive when provided")
    if a.assistant_only_loss and a.last_assistant_only_loss:
        raise ValueError("assistant_only_loss and last_assistant_only_loss are mutually exclusive")
    if a.uses_assistant_loss_mask and a.dataset_text_field != "messages":
        option = "last_assistant_only_loss" if a.last_assistant_only_loss else "assistant_only_loss"
        raise ValueError(f"{option} requires --dataset_text_field messages")
    if a.hub_revision is not None and a.hub_repo_id is None:
        raise ValueError("hub_revision requires hub_repo_id")
    if a.private and a.hub_repo_id is None:
        raise ValueError("private requires hub_repo_id")
    if a.endprompt_enable:
        lo, hi = a.effective_endprompt_logical_length_min, a.effective_endprompt_logical_length
        if lo < a.max_sequence_length or hi < a.max_sequence_length:
            raise ValueError("EndPrompt logical lengths must be at least max_sequence_length")
        if lo > hi:
            raise ValueError("endprompt_logical_length_min cannot exceed endprompt_logical_length")
        if not a.endprompt_prompt_texts:
            raise ValueError("endprompt_prompts must contain at least one non-empty prompt")
        weights = (a.endprompt_context_loss_weight, a.endprompt_prompt_loss_weight)
        if any(not math.isfinite(w) or w < 0.0 for w in weights):
            raise ValueError("EndPrompt loss weights must be finite and non-negative")
        if not any(w > 0.0 for w in weights):
            raise ValueError("at least one EndPrompt loss weight must be positive")
    return a


def endprompt_settings(a) -> EndPromptSettings | None:
    if not a.endprompt_enable:
        return None
    return EndPromptSettings(a.effective_endprompt_logical_length_min, a.effective_endprompt_logical_length,
                             a.endprompt_prompt_texts, a.endprompt_prompt_loss_weight, a.endprompt_context_loss_weight)


def snapshot_download(*args, **kwargs):
    """``huggingface_hub.snapshot_download``, imported on first use; a module-level name so that a
    caller (or a test) can substitute it."""
    from huggingface_hub import snapshot_download as impl

    return impl(*args, **kwargs)


def HfApi(*args, **kwargs):  # noqa: N802 - keeps the Hub client's own name
    """``huggingface_hub.HfApi``, imported on first use; substitutable like :func:`snapshot_download`."""
    from huggingface_hub import HfApi as impl

    return impl(*args, **kwargs)


def publish_to_hub(a: "PrepareArguments", out: Path) -> None:
    """Create the dataset repository (and the branch ``--hub-revision`` names, which an upload does
    not create by itself), then upload manifest and shards in one commit
    (src/causal_trainer/prepare.py:404-430)."""
    from .hf_retry import retry_hf_call

    api = HfApi()
    retry_hf_call(lambda: api.create_repo(a.hub_repo_id, token=a.token, private=a.private, repo_type="dataset",
                                          exist_ok=True), description=f"create dataset repo {a.hub_repo_id}")
    if a.hub_revision is not None:
        retry_hf_call(lambda: api.create_branch(repo_id=a.hub_repo_id, branch=a.hub_revision, token=a.token,
                                                repo_type="dataset", exist_ok=True),
                      description=f"create branch {a.hub_revision}")
    retry_hf_call(lambda: api.upload_folder(repo_id=a.hub_repo_id, folder_path=str(out), path_in_repo="",
                                            token=a.token, repo_type="dataset", revision=a.hub_revision,
                                            commit_message="Upload prepared dataset"),
                  description=f"upload prepared dataset to {a.hub_repo_id}")


def resolve_tokenizer_directory(a: PrepareArguments) -> Path:
    local = Path(a.tokenizer_name_or_path).expanduser()
    if local.is_dir():
        return local.resolve()
    if local.exists():
        raise ValueError(f"tokenizer_name_or_path must be a directory, got {local}")
    from .hf_retry import retry_hf_call

    return Path(retry_hf_call(lambda: snapshot_download(a.tokenizer_name_or_path, repo_type="model",
                                                        revision=a.tokenizer_revision, token=a.token,
                                                        allow_patterns=list(TOKENIZER_GLOBS)),
                              description=f"download tokenizer {a.tokenizer_name_or_path}"))


def tokenizer_digest(directory: Path) -> tuple[str, tuple[str, ...]]:
    """SHA-256 over the names and bytes of every tokenizer/template file (sorted by relative path)."""
    files: dict[str, Path] = {}
    for pattern in TOKENIZER_GLOBS:
        for p in directory.glob(pattern):
            if p.is_file():
                rel = p.relative_to(directory).as_posix()
                if any(part in ("", ".", "..") for part in Path(rel).parts) or "\\" in rel:
                    raise ValueError(f"unsafe tokenizer file path: {rel!r}")
                files[rel] = p
    if "tokenizer.json" not in files:
        raise FileNotFoundError(f"missing {directory / 'tokenizer.json'}")
    h = hashlib.sha256()
    for rel in sorted(files):
        raw = rel.encode("utf-8")
        h.update(len(raw).to_bytes(8, "big"))
        h.update(raw)
        data = files[rel].read_bytes()
        h.update(len(data).to_bytes(8, "big"))
        h.update(data)
    return h.hexdigest(), tuple(sorted(files))


def prepare_dataset(a: PrepareArguments) -> PreparedDatasetManifest:
    out = a.output_dir
    if out.exists() and any(out.iterdir()):
        raise ValueError(f"output_dir must be empty or absent: {out}")
    tok_dir = resolve_tokenizer_directory(a)
    tokenizer = TrainingTokenizer.from_directory(tok_dir)
    tok_sha, tok_files = tokenizer_digest(tok_dir)
    pad_id = tokenizer.pad_token_id if tokenizer.pad_token_id is not None else (tokenizer.eos_token_id or 0)
    source = load_training_split(a.dataset_name, a.dataset_split, token=a.token, config_name=a.dataset_config_name,
                                 revision=a.dataset_revision, streaming=False)
    total = len(source)
    if total == 0:
        raise ValueError("the source split is empty")
    out.mkdir(parents=True, exist_ok=True)
    shards: list[PreparedShard] = []
    max_token, max_position = 0, 0
    names = field_names(a.uses_assistant_loss_mask)
    try:
        for index in range(a.num_shards):
            part, start = select_process_shard(source, process_index=index, process_count=a.num_shards)
            rows = prepare_training_dataset(
                part, tokenizer, dataset_text_field=a.dataset_text_field, max_sequence_length=a.max_sequence_length,
                packing=a.packing, packing_batch_size=a.packing_batch_size, pad_token_id=pad_id,
                assistant_only_loss=a.assistant_only_loss, last_assistant_only_loss=a.last_assistant_only_loss,
                endprompt=endprompt_settings(a), num_proc=a.preprocessing_num_workers, example_index_offset=start,
                allow_empty=True,
            )
            if not rows:
                raise ValueError(f"prepared shard {index} is empty; reduce num_shards or remove source rows that "
                                 "are filtered by the loss settings")
            for r in rows:  # final weights are part of the artifact
                if "loss_weights" not in r:
                    src = "assistant_masks" if a.uses_assistant_loss_mask else "attention_mask"
                    r["loss_weights"] = [float(v) for v in r[src]]
            cols = packed_dataset_to_arrays(rows, max_sequence_length=a.max_sequence_length,
                                            assistant_only_loss=a.uses_assistant_loss_mask,
                                            has_explicit_loss_weights=True)
            cols = {n: cols[n] for n in names}
            cols["loss_weights"] = cols["loss_weights"] * (cols["attention_mask"] != 0)
            max_token = max(max_token, int(cols["input_ids"].max()))
            max_position = max(max_position, int(cols["position_ids"].max()))
            validate_prepared_batch(cols, max_sequence_length=a.max_sequence_length, max_token_id=max_token,
                                    max_position_id=max_position, uses_assistant_loss_mask=a.uses_assistant_loss_mask)
            rel = f"data/shard-{index:05d}-of-{a.num_shards:05d}.parquet"
            n = write_prepared_shard(cols, out / rel)
            shards.append(PreparedShard(rel, n, sha256_file(out / rel)))
        manifest = PreparedDatasetManifest(
            max_sequence_length=a.max_sequence_length, split=a.dataset_split, shards=tuple(shards),
            tokenizer={"name_or_path": a.tokenizer_name_or_path, "revision": a.tokenizer_revision, "sha256": tok_sha,
                       "files": list(tok_files), "pad_token_id": int(pad_id), "vocab_size": len(tokenizer)},
            source={"dataset_name": a.dataset_name, "dataset_config_name": a.dataset_config_name,
                    "dataset_revision": a.dataset_revision, "dataset_split": a.dataset_split, "rows": total,
                    "fingerprint": getattr(source, "_fingerprint", None)},
            # same keys as the manifests written by the reference's prepare command
            # (src/causal_trainer/prepare.py:379-400); never the access token
            preprocessing={
                "dataset_text_field": a.dataset_text_field, "packing": a.packing,
                "packing_batch_size": a.packing_batch_size, "assistant_only_loss": a.assistant_only_loss,
                "last_assistant_only_loss": a.last_assistant_only_loss,
                "preprocessing_num_workers": a.preprocessing_num_workers, "num_shards": a.num_shards,
                "endprompt": None if not a.endprompt_enable else {
                    "logical_length_min": a.effective_endprompt_logical_length_min,
                    "logical_length_max": a.effective_endprompt_logical_length,
                    "prompts": list(a.endprompt_prompt_texts),
                    "prompt_loss_weight": a.endprompt_prompt_loss_weight,
                    "context_loss_weight": a.endprompt_context_loss_weight,
                },
            },
            max_token_id=max_token, max_position_id=max_position,
            uses_assistant_loss_mask=a.uses_assistant_loss_mask,
        )
        tmp = out / (PREPARED_MANIFEST_FILENAME + ".incomplete")
        write_prepared_manifest(manifest, tmp)
        tmp.replace(out / PREPARED_MANIFEST_FILENAME)
    except BaseException:
        shutil.rmtree(out, ignore_errors=True)
        raise
    if a.hub_repo_id is not None:
        publish_to_hub(a, out)
    return manifest


def main(argv: list[str] | None = None) -> int:
    manifest = prepare_dataset(parse_args(argv))
    print(f"prepared {manifest.total_rows} rows in {len(manifest.shards)} shard(s); digest {manifest.global_digest}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
