"""Checkpoint bundles: completion manifest, validation, resume discovery, pruning.

A bundle is a directory (``output_dir`` for the final export, ``output_dir/checkpoint-<step>``
for periodic ones) whose ``checkpoint_manifest.json`` is written **last** and deleted
**first** on overwrite, so a directory with a manifest is complete by construction.  The
manifest (format ``training-checkpoint-bundle``, version 4) records sizes and SHA-256 digests
of every artifact, the checkpoint id shared by all tensor files, the step, and the training
signature of the run that wrote it (src/causal_trainer/checkpointing/bundles.py:926-943).

Discovery (``find_latest_checkpoint``) treats a bundle with another signature or artifact kind
as *incompatible* and a bundle that fails structural or digest validation as *corrupt*; both
are hard errors, never silently skipped (``bundles.py:620-775``).  Among valid candidates the
preference is: completed-streaming root, then highest step, then the root at equal step.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from ..parallel import runtime as rt
from . import safetensors_io as st

BUNDLE_FORMAT = "training-checkpoint-bundle"
BUNDLE_FORMAT_VERSION = 4
ARTIFACT_KINDS = ("merged", "peft-adapter")
MANIFEST_NAME = "checkpoint_manifest.json"


@dataclass(frozen=True)
class ResumeCheckpoint:
    path: Path
    global_step: int
    total_steps: int
    has_optimizer_state: bool
    checkpoint_id: str
    manifest_digest: str
    artifact_kind: str = "merged"
    source_examples_seen: int = 0
    training_complete: bool = False
    streaming_data_digest: str | None = None


def training_signature(payload: Any) -> str:
    raw = json.dumps(payload, ensure_ascii=False, separators=(",", ":"), sort_keys=True).encode("utf-8")
    return hashlib.sha256(raw).hexdigest()


def file_sha256(path: Path) -> str:
    h = hashlib.sha256()
    with path.open("rb") as f:
        for block in iter(lambda: f.read(1 << 22), b""):
            h.update(block)
    return h.hexdigest()


def _is_hex(value: Any, length: int) -> bool:
    return isinstance(value, str) and len(value) == length and all(c in "0123456789abcdef" for c in value)


def _read_manifest(path: Path) -> dict[str, Any] | None:
    m = path / MANIFEST_NAME
    if m.is_symlink() or not m.is_file():
        return None
    try:
        value = json.loads(m.read_text(encoding="utf-8"))
    except (OSError, ValueError):
        return None
    return value if isinstance(value, dict) else None


# What counts as part of a bundle.  Anything else that turns up beside it (a log, a hub cache, an
# editor's swap file, training_args.json, profile_steps.json) is not hashed and cannot invalidate
# a completed checkpoint.  Same convention on disk as src/causal_trainer/checkpointing/bundles.py:
# 46-61, 315-385.
_ASSET_FILES = frozenset({
    "config.json", "generation_config.json", "tokenizer.json", "tokenizer.model", "tokenizer_config.json",
    "special_tokens_map.json", "added_tokens.json", "vocab.json", "merges.txt", "chat_template.json",
    "preprocessor_config.json", "processor_config.json",
})
_ASSET_ENDINGS = (".jinja", ".model", ".tiktoken")
_ADAPTER_FILES = frozenset({"adapter_config.json", "adapter_model.safetensors"})
_TOKENIZER_DATA = frozenset({"tokenizer.json", "tokenizer.model", "vocab.json"})


def _top_level_class(name: str) -> str | None:
    """``"asset" | "merged" | "adapter"`` for a file name directly under the bundle, else None."""
    if name in _ADAPTER_FILES:
        return "adapter"
    if name in ("model.safetensors", "model.safetensors.index.json") or (
            name.startswith("model-") and name.endswith(".safetensors")):
        return "merged"
    if name in _ASSET_FILES or name.startswith("tokenizer.") or name.endswith(_ASSET_ENDINGS):
        return "asset"
    return None


def _real_file(p: Path) -> Path:
    if "\\" in p.name or p.is_symlink() or not p.is_file():
        raise RuntimeError(f"checkpoint artifact must be a regular file: {p}")
    return p


def artifact_files(path: Path, kind: str, has_optimizer: bool) -> list[Path]:
    """The files that make up a bundle of ``kind``, sorted by relative path.

    Top level: model assets, tokenizer files and the weights of ``kind``; one level down
    ``chat_templates/*.jinja`` and, when the bundle carries optimizer state, ``optimizer/*``.
    Raises ``RuntimeError`` for a bundle that cannot be valid: weights of the other kind left
    over from an earlier export, missing weights / config / tokenizer data, an ``optimizer``
    directory the manifest does not announce (or the reverse), artifacts that are not regular
    files.  Everything else in the directory is ignored."""
    if kind not in ARTIFACT_KINDS:
        raise ValueError(f"unknown checkpoint artifact kind {kind!r}")
    found: dict[str, Path] = {}
    classes: dict[str, set[str]] = {"asset": set(), "merged": set(), "adapter": set()}
    for p in path.iterdir():
        cls = _top_level_class(p.name)
        if cls is not None:
            found[p.name] = _real_file(p)
            classes[cls].add(p.name)
    templates = path / "chat_templates"
    if templates.exists():
        if templates.is_symlink() or not templates.is_dir():
            raise RuntimeError(f"chat_templates must be a directory: {templates}")
        for p in templates.iterdir():
            if p.suffix != ".jinja":
                raise RuntimeError(f"chat_templates may only hold .jinja files: {p}")
            found[f"chat_templates/{p.name}"] = _real_file(p)
    other = "adapter" if kind == "merged" else "merged"
    if classes[other]:
        raise RuntimeError(f"{kind} checkpoint holds stale {other} weights: {sorted(classes[other])}")
    if kind == "merged":
        if "model.safetensors" not in found or "config.json" not in found:
            raise RuntimeError(f"checkpoint is missing model.safetensors or config.json: {path}")
        if not any(n in _TOKENIZER_DATA or n.endswith((".model", ".tiktoken")) for n in classes["asset"]):
            raise RuntimeError(f"checkpoint is missing tokenizer data: {path}")
    elif classes["adapter"] != _ADAPTER_FILES:
        raise RuntimeError(f"checkpoint is missing adapter weights or adapter_config.json: {path}")
    opt = path / "optimizer"
    if has_optimizer:
        if opt.is_symlink() or not opt.is_dir():
            raise RuntimeError(f"checkpoint is missing optimizer state: {opt}")
        names = set()
        for p in opt.iterdir():
            found[f"optimizer/{p.name}"] = _real_file(p)
            names.add(p.name)
        if "manifest.json" not in names or not any(n.endswith(".safetensors") for n in names):
            raise RuntimeError(f"optimizer state is incomplete: {opt}")
    elif opt.exists():
        raise RuntimeError(f"checkpoint holds stale optimizer state: {opt}")
    return [found[k] for k in sorted(found)]


def _header_matches(path: Path, checkpoint_id: str, layout: dict[str, tuple[str, tuple[int, ...]]] | None) -> bool:
    try:
        tensors, meta, _ = st.read_header(path)
    except (OSError, ValueError):
        return False
    if meta.get("checkpoint_id") != checkpoint_id:
        return False
    if layout is not None:
        got = {k: (v.dtype, tuple(v.shape)) for k, v in tensors.items()}
        want = {k: (dt, tuple(shape)) for k, (dt, shape) in layout.items()}
        if got != want:
            return False
    return True


def _optimizer_state_valid(path: Path, step: int, checkpoint_id: str) -> bool:
    d = path / "optimizer"
    try:
        manifest = json.loads((d / "manifest.json").read_text(encoding="utf-8"))
    except (OSError, ValueError):
        return False
    if (manifest.get("format") != "optimizer-state-safetensors" or manifest.get("format_version") != 1
            or manifest.get("global_step") != step or manifest.get("checkpoint_id") != checkpoint_id):
        return False
    try:
        tensors, meta, _ = st.read_header(d / "state.safetensors")
    except (OSError, ValueError):
        return False
    entries = manifest.get("tensors")
    if meta.get("checkpoint_id") != checkpoint_id or not isinstance(entries, list) \
            or manifest.get("tensor_count") != len(tensors) or len(entries) != len(tensors):
        return False
    fingerprint = hashlib.sha256(json.dumps(entries, separators=(",", ":"), sort_keys=True).encode("utf-8")).hexdigest()
    if manifest.get("layout_fingerprint") != fingerprint:
        return False
    for e in entries:
        if not isinstance(e, dict):
            return False
        info = tensors.get(e.get("key"))
        # the manifest spells dtypes the numpy way ("int32"); the safetensors header says "I32"
        if info is None or e.get("dtype") not in (info.dtype, st.PLAIN_DTYPE_NAMES.get(info.dtype)) \
                or list(info.shape) != e.get("shape"):
            return False
    return True


def _artifacts_match(path: Path, manifest: dict[str, Any], verify_digests: bool) -> bool:
    sizes, digests = manifest.get("artifact_sizes"), manifest.get("artifact_digests")
    if not isinstance(sizes, dict) or not isinstance(digests, dict) or set(sizes) != set(digests):
        return False
    try:
        files = {p.relative_to(path).as_posix(): p
                 for p in artifact_files(path, manifest["artifact_kind"], manifest["has_optimizer_state"])}
        if set(files) != set(sizes):
            return False
        for rel, p in files.items():
            if type(sizes[rel]) is not int or p.stat().st_size != sizes[rel] or not _is_hex(digests[rel], 64):
                return False
            if verify_digests and file_sha256(p) != digests[rel]:
                return False
    except (OSError, RuntimeError, ValueError):
        return False
    return True


def find_latest_checkpoint(output_dir: str | Path, expected_signature: str, *,
                           expected_model_layout: dict[str, tuple[str, tuple[int, ...]]] | None = None,
                           expected_artifact_kind: str = "merged", verify_artifact_digests: bool = True
                           ) -> ResumeCheckpoint | None:
    if expected_artifact_kind not in ARTIFACT_KINDS:
        raise ValueError(f"unknown expected artifact kind {expected_artifact_kind!r}")
    root = Path(output_dir)
    paths = [root]
    if root.is_dir():
        paths += sorted(p for p in root.glob("checkpoint-*") if p.is_dir() and not p.is_symlink())
    good: list[ResumeCheckpoint] = []
    incompatible: list[Path] = []
    corrupt: list[Path] = []
    for path in paths:
        mpath = path / MANIFEST_NAME
        m = _read_manifest(path)
        if m is None:
            if mpath.exists() or mpath.is_symlink():
                corrupt.append(path)
            continue
        if m.get("format") != BUNDLE_FORMAT:
            corrupt.append(path)
            continue
        kind = m.get("artifact_kind")
        if (m.get("format_version") != BUNDLE_FORMAT_VERSION or m.get("training_signature") != expected_signature
                or kind != expected_artifact_kind or kind not in ARTIFACT_KINDS):
            incompatible.append(path)
            continue
        step, total, cid = m.get("global_step"), m.get("total_steps"), m.get("checkpoint_id")
        seen, done, sdig = m.get("source_examples_seen", 0), m.get("training_complete", False), m.get("streaming_data_digest")
        ok = (
            type(step) is int and type(total) is int and 0 <= step <= total and total > 0 and _is_hex(cid, 32)
            and isinstance(m.get("has_optimizer_state"), bool) and type(seen) is int and seen >= 0
            and isinstance(done, bool) and (sdig is None or _is_hex(sdig, 64)) and not (seen > 0 and sdig is None)
            and not (done and (path != root or step != total or sdig is None))
        )
        if ok and path != root:
            try:
                ok = int(path.name.removeprefix("checkpoint-")) == step
            except ValueError:
                ok = False
        if ok:
            ok = _artifacts_match(path, m, verify_artifact_digests)
        if ok and kind == "merged":
            ok = (path / "config.json").is_file() and _header_matches(path / "model.safetensors", cid, expected_model_layout)
        if ok and kind == "peft-adapter":
            ok = (path / "adapter_config.json").is_file() and _header_matches(
                path / "adapter_model.safetensors", cid, expected_model_layout)
        if ok and m["has_optimizer_state"]:
            ok = _optimizer_state_valid(path, step, cid)
        if not ok:
            corrupt.append(path)
            continue
        good.append(ResumeCheckpoint(path, step, total, m["has_optimizer_state"], cid, training_signature(m), kind,
                                     seen, done, sdig))
    if incompatible:
        raise ValueError("output_dir contains checkpoints from an incompatible training configuration: "
                         + ", ".join(str(p) for p in incompatible[:3]))
    if corrupt:
        raise ValueError("output_dir contains corrupt completed checkpoints: " + ", ".join(str(p) for p in corrupt[:3]))
    if not good:
        return None
    return max(good, key=lambda c: (c.training_complete and c.path == root, c.global_step, c.path == root))


def resume_action(checkpoint: ResumeCheckpoint | None, *, output_dir: Path, total_steps: int) -> str:
    """What a launch does with the newest valid checkpoint: ``start`` (none), ``continue`` (partial run
    with optimizer state), ``finalize`` (all steps done but only in a periodic directory) or
    ``complete`` (nothing left to do).  Anything that would silently reset training state is an error
    (decision table of src/causal_trainer/training/runner.py:573-600)."""
    if checkpoint is None:
        return "start"
    at_root = checkpoint.path == output_dir
    if checkpoint.training_complete:        # a stream that ended before its estimated horizon
        if not at_root:
            raise ValueError("a completed streaming checkpoint must be stored at output_dir")
        return "complete"
    if checkpoint.total_steps != total_steps:
        raise ValueError(f"checkpoint total_steps={checkpoint.total_steps} does not match current plan {total_steps}")
    finished = checkpoint.global_step == total_steps
    if finished:
        return "complete" if at_root else "finalize"
    if not checkpoint.has_optimizer_state:
        raise ValueError(
            "the latest checkpoint does not contain optimizer state, so exact continuation is impossible; optimizer "
            "state must have been saved before the interruption with --save_optimizer_state True, and enabling it "
            "only now cannot repair this checkpoint")
    return "continue"


def invalidate(path: Path) -> None:
    """Deletes the manifest first so a half-overwritten bundle can never look complete."""
    (path / MANIFEST_NAME).unlink(missing_ok=True)


def write_manifest(path: Path, *, artifact_kind: str, checkpoint_id: str, global_step: int, total_steps: int,
                   has_optimizer_state: bool, signature: str, source_examples_seen: int = 0,
                   streaming_data_digest: str | None = None, training_complete: bool = False) -> dict[str, Any]:
    files = artifact_files(path, artifact_kind, has_optimizer_state)
    manifest = {
        "format": BUNDLE_FORMAT, "format_version": BUNDLE_FORMAT_VERSION, "artifact_kind": artifact_kind,
        "artifact_sizes": {p.relative_to(path).as_posix(): p.stat().st_size for p in files},
        "artifact_digests": {p.relative_to(path).as_posix(): file_sha256(p) for p in files},
        "checkpoint_id": checkpoint_id, "global_step": int(global_step), "total_steps": int(total_steps),
        "has_optimizer_state": bool(has_optimizer_state), "source_examples_seen": int(source_examples_seen),
        "streaming_data_digest": streaming_data_digest, "training_complete": bool(training_complete),
        "training_signature": signature,
    }
    tmp = path / (MANIFEST_NAME + ".tmp")
    tmp.write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n", encoding="utf-8")
    with tmp.open("rb") as f:
        os.fsync(f.fileno())
    os.replace(tmp, path / MANIFEST_NAME)
    return manifest


def save_checkpoint_bundle(destination: str | Path, *, export_model, export_optimizer=None, artifact_kind: str = "merged",
                           global_step: int, total_steps: int, signature: str, source_examples_seen: int = 0,
                           streaming_data_digest: str | None = None, training_complete: bool = False) -> str:
    """Collective.  ``export_model(dest, checkpoint_id)`` and ``export_optimizer(dest, checkpoint_id)`` do the
    tensor I/O (both collective); rank 0 then hashes every artifact and writes the manifest last."""
    from .huggingface import new_checkpoint_id, remove_optimizer_checkpoint

    dest = Path(destination)
    error: BaseException | None = None
    cid = new_checkpoint_id()
    if rt.process_index() == 0:
        try:
            dest.mkdir(parents=True, exist_ok=True)
            invalidate(dest)
        except BaseException as exc:  # noqa: BLE001
            error = exc
    rt.raise_if_process_zero_error(error, "prepare checkpoint directory")
    remove_optimizer_checkpoint(dest)
    export_model(dest, cid)
    if export_optimizer is not None:
        export_optimizer(dest, cid)
    if rt.process_index() == 0:
        try:
            write_manifest(dest, artifact_kind=artifact_kind, checkpoint_id=cid, global_step=global_step,
                           total_steps=total_steps, has_optimizer_state=export_optimizer is not None,
                           signature=signature, source_examples_seen=source_examples_seen,
                           streaming_data_digest=streaming_data_digest, training_complete=training_complete)
        except BaseException as exc:  # noqa: BLE001
            error = exc
    rt.raise_if_process_zero_error(error, "write checkpoint manifest")
    rt.sync_processes(f"checkpoint-{global_step}")
    return cid


def save_adapter_checkpoint_bundle(lora, destination: str | Path, *, base_model_name_or_path: str, global_step: int,
                                   total_steps: int, signature: str, revision: str | None = None,
                                   export_optimizer=None, **manifest_fields) -> str:
    """A ``peft-adapter`` bundle: the adapter files, optionally the optimizer state, then the
    manifest (src/causal_trainer/checkpointing/bundles.py:951-1113).  Collective like
    :func:`save_checkpoint_bundle`, which does the work."""
    from .huggingface import export_adapter_checkpoint

    def export_model(dest: Path, checkpoint_id: str) -> None:
        export_adapter_checkpoint(dest, lora, base_model_name_or_path=base_model_name_or_path,
                                  checkpoint_id=checkpoint_id, revision=revision)

    return save_checkpoint_bundle(destination, export_model=export_model, export_optimizer=export_optimizer,
                                  artifact_kind="peft-adapter", global_step=global_step, total_steps=total_steps,
                                  signature=signature, **manifest_fields)


def prune_periodic_exports(output_dir: str | Path, limit: int, signature: str) -> list[Path]:
    """Keeps the newest ``limit`` fully valid periodic bundles of this run (0 keeps all); rank 0 only."""
    if limit <= 0 or rt.process_index() != 0:
        return []
    root = Path(output_dir)
    valid: list[tuple[int, Path]] = []
    for p in root.glob("checkpoint-*"):
        m = _read_manifest(p)
        if (p.is_dir() and not p.is_symlink() and m is not None and m.get("format") == BUNDLE_FORMAT
                and m.get("training_signature") == signature and type(m.get("global_step")) is int
                and p.name == f"checkpoint-{m['global_step']}" and _artifacts_match(p, m, verify_digests=False)):
            valid.append((m["global_step"], p))
    valid.sort()
    removed = []
    for _, p in valid[:-limit]:
        invalidate(p)
        shutil.rmtree(p)
        removed.append(p)
    return removed
