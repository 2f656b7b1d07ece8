"""Prepared datasets: ``causal-prepare`` artifacts (manifest + Parquet shards) and their loaders.

An artifact is a directory (or Hub dataset repo) holding ``causal-trainer-prepared.json`` and
``data/shard-XXXXX-of-XXXXX.parquet`` files.  Rows are final: fixed-length int32 model fields,
optional ``assistant_masks`` and float32 ``loss_weights``; masks and weights are not
recomputed at training time.  The manifest records schema, shard row counts and SHA-256
digests, the tokenizer / source / preprocessing identity, and the largest token and
position ids (src/causal_trainer/data/prepared.py:84-330).

Loading assigns one contiguous interval of *files* to each process (``:372-387``), verifies
each file's digest and validates every row semantically (``:469-560``): binary masks, ids in
range, segment ids positive exactly on valid tokens and contiguous, positions and weights
zero outside the mask, finite non-negative weights, and at least one positive-weight target
per row.  Parquet I/O goes through ``pyarrow`` directly.
"""
from __future__ import annotations

import hashlib
import json
import re
from dataclasses import dataclass
from pathlib import Path, PurePosixPath, PureWindowsPath
from typing import Any, Iterator, Mapping, Sequence

import numpy as np

from .batching import MODEL_FIELDS
from .pipeline import contiguous_shard_bounds
from .streaming import StreamingBatchEnvelope

PREPARED_DATASET_FORMAT = "causal-trainer-prepared"
PREPARED_MANIFEST_FILENAME = "causal-trainer-prepared.json"
PREPARED_REQUIRED_FIELDS = (*MODEL_FIELDS, "loss_weights")
_DIGEST_DOMAIN = b"causal-trainer-prepared-manifest\0"
_SHA256 = re.compile(r"[0-9a-f]{64}")
_SPLIT = re.compile(r"[A-Za-z0-9_][A-Za-z0-9._-]*")


def _plain_int(value: Any, name: str, minimum: int = 0) -> int:
    if type(value) is not int or value < minimum:
        raise ValueError(f"{name} must be an integer greater than or equal to {minimum}")
    return value


def _json_object(value: Any, name: str) -> dict[str, Any]:
    if not isinstance(value, Mapping):
        raise TypeError(f"{name} must be a JSON object")
    if any(not isinstance(k, str) for k in value):
        raise TypeError(f"{name} keys must be strings")
    try:
        raw = json.dumps(dict(value), ensure_ascii=False, allow_nan=False, separators=(",", ":"), sort_keys=True)
    except (TypeError, ValueError) as exc:
        raise ValueError(f"{name} must contain finite JSON values") from exc
    return json.loads(raw)


def validate_shard_path(value: Any) -> str:
    if not isinstance(value, str) or not value:
        raise ValueError("prepared shard path must be a non-empty string")
    if "\\" in value:
        raise ValueError("prepared shard paths must use forward slashes")
    p = PurePosixPath(value)
    if p.is_absolute() or PureWindowsPath(value).drive or str(p) != value or any(x in ("", ".", "..") for x in p.parts):
        raise ValueError(f"prepared shard path must be a normalized relative path, got {value!r}")
    if p.suffix.lower() != ".parquet":
        raise ValueError(f"prepared shard path must name a Parquet file, got {value!r}")
    return value


@dataclass(frozen=True)
class PreparedShard:
    path: str
    rows: int
    sha256: str

    def __post_init__(self) -> None:
        validate_shard_path(self.path)
        _plain_int(self.rows, "prepared shard rows")
        if not isinstance(self.sha256, str) or _SHA256.fullmatch(self.sha256) is None:
            raise ValueError("prepared shard sha256 must be a lowercase SHA-256 digest")

    def to_dict(self) -> dict[str, Any]:
        return {"path": self.path, "rows": self.rows, "sha256": self.sha256}

    @classmethod
    def from_dict(cls, value: Any) -> "PreparedShard":
        if not isinstance(value, Mapping):
            raise TypeError("prepared shard metadata must be a JSON object")
        want = {"path", "rows", "sha256"}
        if set(value) != want:
            raise ValueError(f"prepared shard metadata fields mismatch: missing={sorted(want - set(value))}, "
                             f"extra={sorted(set(value) - want)}")
        return cls(value["path"], value["rows"], value["sha256"])


def field_names(uses_assistant_loss_mask: bool) -> tuple[str, ...]:
    return (*MODEL_FIELDS, *(("assistant_masks",) if uses_assistant_loss_mask else ()), "loss_weights")


def schema_dict(max_sequence_length: int, uses_assistant_loss_mask: bool) -> dict[str, dict[str, Any]]:
    return {n: {"dtype": "float32" if n == "loss_weights" else "int32", "length": max_sequence_length}
            for n in field_names(uses_assistant_loss_mask)}


_MANIFEST_KEYS = {"format", "split", "max_sequence_length", "total_rows", "max_token_id", "max_position_id",
                  "uses_assistant_loss_mask", "schema", "shards", "tokenizer", "source", "preprocessing"}


@dataclass(frozen=True)
class PreparedDatasetManifest:
    max_sequence_length: int
    split: str
    shards: tuple[PreparedShard, ...]
    tokenizer: Mapping[str, Any]
    source: Mapping[str, Any]
    preprocessing: Mapping[str, Any]
    max_token_id: int
    max_position_id: int
    uses_assistant_loss_mask: bool = False

    def __post_init__(self) -> None:
        _plain_int(self.max_sequence_length, "prepared max_sequence_length", 1)
        if not isinstance(self.split, str) or _SPLIT.fullmatch(self.split) is None:
            raise ValueError(f"invalid prepared split name: {self.split!r}")
        object.__setattr__(self, "shards", tuple(self.shards))
        if not self.shards or any(not isinstance(s, PreparedShard) for s in self.shards):
            raise ValueError("prepared manifest requires at least one PreparedShard")
        if len({s.path for s in self.shards}) != len(self.shards):
            raise ValueError("prepared manifest shard paths must be unique")
        if sum(s.rows for s in self.shards) <= 0:
            raise ValueError("prepared manifest must contain at least one row")
        _plain_int(self.max_token_id, "prepared max_token_id")
        _plain_int(self.max_position_id, "prepared max_position_id")
        if type(self.uses_assistant_loss_mask) is not bool:
            raise TypeError("uses_assistant_loss_mask must be a boolean")
        for name in ("tokenizer", "source", "preprocessing"):
            object.__setattr__(self, name, _json_object(getattr(self, name), f"prepared {name} metadata"))

    @property
    def total_rows(self) -> int:
        return sum(s.rows for s in self.shards)

    @property
    def has_assistant_masks(self) -> bool:
        return self.uses_assistant_loss_mask

    @property
    def schema(self) -> dict[str, dict[str, Any]]:
        return schema_dict(self.max_sequence_length, self.uses_assistant_loss_mask)

    def to_dict(self) -> dict[str, Any]:
        return {
            "format": PREPARED_DATASET_FORMAT, "split": self.split, "max_sequence_length": self.max_sequence_length,
            "total_rows": self.total_rows, "max_token_id": self.max_token_id, "max_position_id": self.max_position_id,
            "uses_assistant_loss_mask": self.uses_assistant_loss_mask, "schema": self.schema,
            "shards": [s.to_dict() for s in self.shards], "tokenizer": dict(self.tokenizer),
            "source": dict(self.source), "preprocessing": dict(self.preprocessing),
        }

    @classmethod
    def from_dict(cls, value: Any) -> "PreparedDatasetManifest":
        if not isinstance(value, Mapping):
            raise TypeError("prepared manifest must be a JSON object")
        if set(value) != _MANIFEST_KEYS:
            raise ValueError(f"prepared manifest fields mismatch: missing={sorted(_MANIFEST_KEYS - set(value))}, "
                             f"extra={sorted(set(value) - _MANIFEST_KEYS)}")
        if value["format"] != PREPARED_DATASET_FORMAT:
            raise ValueError(f"unsupported prepared dataset format marker: {value['format']!r}")
        shards = value["shards"]
        if not isinstance(shards, Sequence) or isinstance(shards, (str, bytes)):
            raise TypeError("prepared manifest shards must be a JSON array")
        m = cls(value["max_sequence_length"], value["split"], tuple(PreparedShard.from_dict(s) for s in shards),
                value["tokenizer"], value["source"], value["preprocessing"], value["max_token_id"],
                value["max_position_id"], value["uses_assistant_loss_mask"])
        if value["total_rows"] != m.total_rows:
            raise ValueError(f"prepared manifest total_rows={value['total_rows']!r} does not match the shard total "
                             f"{m.total_rows}")
        if value["schema"] != m.schema:
            raise ValueError("prepared manifest schema does not match its canonical settings")
        return m

    def to_json(self, indent: int | None = 2) -> str:
        return json.dumps(self.to_dict(), ensure_ascii=False, allow_nan=False, indent=indent, sort_keys=True) + (
            "\n" if indent is not None else "")

    @classmethod
    def from_json(cls, value: str | bytes | bytearray) -> "PreparedDatasetManifest":
        try:
            return cls.from_dict(json.loads(value))
        except (json.JSONDecodeError, UnicodeDecodeError) as exc:
            raise ValueError(f"invalid prepared manifest JSON: {exc}") from exc

    @property
    def global_digest(self) -> str:
        raw = json.dumps(self.to_dict(), ensure_ascii=False, allow_nan=False, separators=(",", ":"), sort_keys=True)
        return hashlib.sha256(_DIGEST_DOMAIN + raw.encode("utf-8")).hexdigest()

    digest = global_digest
    _fingerprint = global_digest


def sha256_file(path: str | Path, chunk_size: int = 1 << 20) -> str:
    if type(chunk_size) is not int or chunk_size <= 0:
        raise ValueError("chunk_size must be a positive integer")
    h = hashlib.sha256()
    with Path(path).open("rb") as f:
        while block := f.read(chunk_size):
            h.update(block)
    return h.hexdigest()


def read_prepared_manifest(path: str | Path) -> PreparedDatasetManifest:
    return PreparedDatasetManifest.from_json(Path(path).read_bytes())


def write_prepared_manifest(manifest: PreparedDatasetManifest, path: str | Path) -> None:
    if not isinstance(manifest, PreparedDatasetManifest):
        raise TypeError("manifest must be a PreparedDatasetManifest")
    Path(path).write_text(manifest.to_json(), encoding="utf-8")


def hf_hub_download(**kwargs):
    """``huggingface_hub.hf_hub_download``, imported on first use; a module-level name so that a
    caller (or a test) can substitute it."""
    from huggingface_hub import hf_hub_download as impl

    return impl(**kwargs)


def HfApi(*args, **kwargs):  # noqa: N802 - keeps the Hub client's own name
    """``huggingface_hub.HfApi``, imported on first use; substitutable like :func:`hf_hub_download`."""
    from huggingface_hub import HfApi as impl

    return impl(*args, **kwargs)


def load_prepared_manifest(name: str, *, token: str | None = None, revision: str | None = None,
                           cache_dir: str | Path | None = None, filename: str = PREPARED_MANIFEST_FILENAME
                           ) -> PreparedDatasetManifest:
    p = Path(name).expanduser()
    if p.is_file():
        return read_prepared_manifest(p)
    if p.is_dir():
        return read_prepared_manifest(p / filename)
    from ..hf_retry import retry_hf_call

    return read_prepared_manifest(retry_hf_call(lambda: hf_hub_download(
        repo_id=name, filename=filename, repo_type="dataset", revision=revision, token=token,
        cache_dir=None if cache_dir is None else str(cache_dir)), description=f"download manifest of {name}"))


def resolve_prepared_revision(name: str, *, token: str | None = None, revision: str | None = None) -> str | None:
    """Pins a Hub reference to a commit once so manifest and shards cannot race."""
    if Path(name).expanduser().exists():
        return None
    commit = getattr(HfApi().dataset_info(repo_id=name, revision=revision, token=token), "sha", None)
    if not isinstance(commit, str) or not commit:
        raise RuntimeError("Hugging Face did not return a prepared dataset commit SHA")
    return commit


def assigned_prepared_shards(manifest: PreparedDatasetManifest, *, process_index: int, process_count: int
                             ) -> tuple[PreparedShard, ...]:
    start, stop = contiguous_shard_bounds(len(manifest.shards), process_index, process_count)
    return manifest.shards[start:stop]


# ----------------------------------------------------------------------------------------- validation
def _as_array(values: Any, name: str, rows: int, length: int) -> np.ndarray:
    dtype = np.float32 if name == "loss_weights" else np.int64
    try:
        arr = np.asarray(values, dtype=dtype)
    except (TypeError, ValueError) as exc:
        raise ValueError(f"prepared field {name!r} must be rectangular with shape {(rows, length)}") from exc
    if arr.shape != (rows, length):
        raise ValueError(f"prepared field {name!r} has shape {arr.shape}, expected {(rows, length)}")
    if name != "loss_weights":
        if arr.size and (arr.min() < np.iinfo(np.int32).min or arr.max() > np.iinfo(np.int32).max):
            raise ValueError(f"prepared field {name!r} contains a value outside int32 range")
        arr = arr.astype(np.int32)
    return arr


def validate_prepared_batch(columns: Mapping[str, Any], *, max_sequence_length: int, max_token_id: int,
                            max_position_id: int, uses_assistant_loss_mask: bool) -> dict[str, np.ndarray]:
    """Checks one batch of rows against every semantic rule; returns typed arrays."""
    names = field_names(uses_assistant_loss_mask)
    if set(columns) != set(names):
        raise ValueError(f"prepared batch fields mismatch: missing={sorted(set(names) - set(columns))}, "
                         f"extra={sorted(set(columns) - set(names))}")
    rows = len(columns["input_ids"])
    out = {n: _as_array(columns[n], n, rows, max_sequence_length) for n in names}
    ids, mask, pos, seg, w = (out[k] for k in ("input_ids", "attention_mask", "position_ids", "segment_ids",
                                               "loss_weights"))
    if (ids < 0).any():
        raise ValueError("prepared input_ids must be non-negative")
    if ids.size and ids.max() > max_token_id:
        raise ValueError(f"prepared input_ids exceed manifest max_token_id={max_token_id}")
    if not np.isin(mask, (0, 1)).all():
        raise ValueError("prepared attention_mask must contain only 0/1 values")
    if (pos < 0).any():
        raise ValueError("prepared position_ids must be non-negative")
    if pos.size and pos.max() > max_position_id:
        raise ValueError(f"prepared position_ids exceed manifest max_position_id={max_position_id}")
    if (seg < 0).any():
        raise ValueError("prepared segment_ids must be non-negative")
    if ((seg > 0) != (mask == 1)).any():
        raise ValueError("prepared segment_ids must be positive exactly where attention_mask is one")
    if (pos[mask == 0] != 0).any():
        raise ValueError("prepared position_ids must be zero outside the attention mask")
    if not np.isfinite(w).all() or (w < 0).any():
        raise ValueError("prepared loss_weights must be finite and non-negative")
    if (w[mask == 0] != 0).any():
        raise ValueError("prepared loss_weights must be zero outside the attention mask")
    if uses_assistant_loss_mask:
        am = out["assistant_masks"]
        if not np.isin(am, (0, 1)).all():
            raise ValueError("prepared assistant_masks must contain only 0/1 values")
        if (am[mask == 0] != 0).any():
            raise ValueError("prepared assistant_masks must be zero outside the attention mask")
    # a segment id may not come back after its run ended, be it at another segment or at padding
    for r in range(rows):
        row = seg[r]
        if row.size:
            runs = row[np.r_[True, row[1:] != row[:-1]]]
            seen: set[int] = set()
            for sid in runs[runs > 0].tolist():
                if sid in seen:
                    raise ValueError(f"prepared row {r} reuses segment_id={sid} after its contiguous run")
                seen.add(sid)
    edge = (mask[:, :-1] == 1) & (mask[:, 1:] == 1) & (seg[:, :-1] == seg[:, 1:]) & (w[:, 1:] > 0)
    if rows and not edge.any(axis=1).all():
        bad = int(np.flatnonzero(~edge.any(axis=1))[0])
        raise ValueError(f"prepared row {bad} has no positive-weight causal target with a valid same-segment "
                         "predecessor")
    return out


_INT32_MAX = int(np.iinfo(np.int32).max)


def canonical_prepared_features(max_sequence_length: int, *, uses_assistant_loss_mask: bool = False
                                ) -> dict[str, dict[str, Any]]:
    """The fixed schema of a prepared row: per field its dtype and length (the manifest's ``schema``)."""
    _plain_int(max_sequence_length, "max_sequence_length", minimum=1)
    if type(uses_assistant_loss_mask) is not bool:
        raise TypeError("uses_assistant_loss_mask must be a boolean")
    return schema_dict(max_sequence_length, uses_assistant_loss_mask)


def canonical_prepared_dataset(columns: Mapping[str, Any], *, max_sequence_length: int,
                               uses_assistant_loss_mask: bool = False) -> dict[str, np.ndarray]:
    """Typed ``[rows, S]`` int32 / float32 columns from any rectangular input, after every semantic
    check (src/causal_trainer/data/prepared.py:557-576); what :func:`write_prepared_shard` takes."""
    return validate_prepared_batch(columns, max_sequence_length=max_sequence_length, max_token_id=_INT32_MAX,
                                   max_position_id=_INT32_MAX, uses_assistant_loss_mask=uses_assistant_loss_mask)


def validate_prepared_dataset(columns: Mapping[str, Any], *, max_sequence_length: int,
                              uses_assistant_loss_mask: bool = False, expected_rows: int | None = None,
                              max_token_id: int | None = None, max_position_id: int | None = None) -> None:
    """Row count, schema, value maxima and row semantics of materialised columns."""
    if max_token_id is not None:
        _plain_int(max_token_id, "prepared max_token_id")
    if max_position_id is not None:
        _plain_int(max_position_id, "prepared max_position_id")
    arrays = validate_prepared_batch(columns, max_sequence_length=max_sequence_length,
                                     max_token_id=_INT32_MAX if max_token_id is None else max_token_id,
                                     max_position_id=_INT32_MAX if max_position_id is None else max_position_id,
                                     uses_assistant_loss_mask=uses_assistant_loss_mask)
    rows = len(arrays["input_ids"])
    if expected_rows is not None and rows != expected_rows:
        raise ValueError(f"prepared dataset has {rows} rows, expected {expected_rows}")


# ----------------------------------------------------------------------------------------- parquet
def write_prepared_shard(columns: Mapping[str, np.ndarray], path: str | Path) -> int:
    """Writes typed ``[rows, S]`` columns as fixed-size-list Parquet columns; returns the row count."""
    import pyarrow as pa
    import pyarrow.parquet as pq

    arrays, names = [], []
    rows = None
    for name, col in columns.items():
        col = np.ascontiguousarray(col, dtype=np.float32 if name == "loss_weights" else np.int32)
        rows = col.shape[0] if rows is None else rows
        flat = pa.array(col.reshape(-1), type=pa.float32() if name == "loss_weights" else pa.int32())
        arrays.append(pa.FixedSizeListArray.from_arrays(flat, col.shape[1]))
        names.append(name)
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    pq.write_table(pa.Table.from_arrays(arrays, names=names), str(path))
    return int(rows or 0)


def read_prepared_shard(path: str | Path, manifest: PreparedDatasetManifest, batch_rows: int = 2048
                        ) -> Iterator[dict[str, np.ndarray]]:
    """Validated typed batches of one shard file."""
    import pyarrow.parquet as pq

    pf = pq.ParquetFile(str(path))
    names = field_names(manifest.uses_assistant_loss_mask)
    if set(pf.schema_arrow.names) != set(names):
        raise ValueError(f"{path}: columns {sorted(pf.schema_arrow.names)} do not match the manifest schema")
    for rb in pf.iter_batches(batch_size=batch_rows, columns=list(names)):
        cols = {}
        for name in names:
            arr = rb.column(name)
            flat = arr.flatten().to_numpy(zero_copy_only=False)
            cols[name] = flat.reshape(len(arr), -1)
        yield validate_prepared_batch(cols, max_sequence_length=manifest.max_sequence_length,
                                      max_token_id=manifest.max_token_id, max_position_id=manifest.max_position_id,
                                      uses_assistant_loss_mask=manifest.uses_assistant_loss_mask)


def _resolve_shard(name: str, shard: PreparedShard, token: str | None, revision: str | None,
                   cache_dir: str | Path | None = None) -> Path:
    root = Path(name).expanduser()
    if root.is_file():
        root = root.parent
    if root.is_dir():
        return root / shard.path
    from ..hf_retry import retry_hf_call

    return Path(retry_hf_call(lambda: hf_hub_download(repo_id=name, filename=shard.path, repo_type="dataset",
                                                      revision=revision, token=token,
                                                      cache_dir=None if cache_dir is None else str(cache_dir)),
                              description=f"download {shard.path}"))


def _verify_shard(path: Path, shard: PreparedShard) -> None:
    actual = sha256_file(path)
    if actual != shard.sha256:
        raise RuntimeError(f"prepared shard checksum mismatch for {shard.path!r}: expected {shard.sha256}, "
                           f"got {actual}")


class PreparedRowStream:
    """Lazy, re-iterable rows of every shard of a prepared artifact, in manifest order; each pass
    validates what it reads and checks every shard's row count."""

    def __init__(self, files: Sequence[Path], manifest: PreparedDatasetManifest):
        self.files = list(files)
        self.manifest = manifest

    def __iter__(self) -> Iterator[dict[str, list]]:
        for path, shard in zip(self.files, self.manifest.shards):
            rows = 0
            for batch in read_prepared_shard(path, self.manifest):
                n = len(batch["input_ids"])
                rows += n
                for i in range(n):
                    yield {k: v[i].tolist() for k, v in batch.items()}
            if rows != shard.rows:
                raise ValueError(f"prepared shard {shard.path} has {rows} rows, manifest says {shard.rows}")


def load_prepared_dataset(name: str, manifest: PreparedDatasetManifest | None = None, *, token: str | None = None,
                          revision: str | None = None, streaming: bool = False, process_index: int | None = None,
                          process_count: int | None = None, cache_dir: str | Path | None = None,
                          verify_checksums: bool = True):
    """Typed columns of this process's contiguous shard interval (all shards when no process is
    given); only that interval is downloaded.  ``streaming`` selects every shard instead (each
    process reproduces the same global stream), checks the checksums up front and returns a lazy
    :class:`PreparedRowStream` (src/causal_trainer/data/prepared.py:665-790)."""
    if (process_index is None) != (process_count is None):
        raise ValueError("process_index and process_count must be provided together")
    manifest = manifest or load_prepared_manifest(name, token=token, revision=revision, cache_dir=cache_dir)
    if not isinstance(manifest, PreparedDatasetManifest):
        raise TypeError("manifest must be a PreparedDatasetManifest")
    if streaming:
        files = [_resolve_shard(name, shard, token, revision, cache_dir) for shard in manifest.shards]
        if verify_checksums:
            for path, shard in zip(files, manifest.shards):
                _verify_shard(path, shard)
        return PreparedRowStream(files, manifest)
    shards = manifest.shards if process_index is None else assigned_prepared_shards(
        manifest, process_index=process_index, process_count=process_count)
    files = [_resolve_shard(name, shard, token, revision, cache_dir) for shard in shards]
    if verify_checksums:
        for path, shard in zip(files, shards):
            _verify_shard(path, shard)
    names = field_names(manifest.uses_assistant_loss_mask)
    parts: dict[str, list[np.ndarray]] = {n: [] for n in names}
    for path, shard in zip(files, shards):
        rows = 0
        for batch in read_prepared_shard(path, manifest):
            rows += len(batch["input_ids"])
            for n in names:
                parts[n].append(batch[n])
        if rows != shard.rows:
            raise RuntimeError(f"prepared shard {shard.path} has {rows} rows, manifest says {shard.rows}")
    s = manifest.max_sequence_length
    return {n: (np.concatenate(v) if v else np.zeros((0, s), dtype=np.float32 if n == "loss_weights" else np.int32))
            for n, v in parts.items()}


def iter_prepared_streaming_batches(name: str, manifest: PreparedDatasetManifest, *, num_epochs: int | None,
                                    window_size: int = 1000, token: str | None = None, revision: str | None = None,
                                    cache_dir: str | Path | None = None, verify_checksums: bool = True
                                    ) -> Iterator[StreamingBatchEnvelope]:
    """Streams a prepared artifact shard by shard as packing-window envelopes (one source row = one record)."""
    if type(window_size) is not int or window_size <= 0:
        raise ValueError("window_size must be a positive integer")
    if num_epochs is not None and (type(num_epochs) is not int or num_epochs <= 0):
        raise ValueError("num_epochs must be a positive integer or None")
    import itertools

    for epoch in (itertools.count() if num_epochs is None else range(num_epochs)):
        for shard in manifest.shards:
            path = _resolve_shard(name, shard, token, revision, cache_dir)
            if verify_checksums:
                _verify_shard(path, shard)
            rows = 0
            for batch in read_prepared_shard(path, manifest, batch_rows=window_size):
                n = len(batch["input_ids"])
                rows += n
                records = tuple({k: v[i].tolist() for k, v in batch.items()} for i in range(n))
                yield StreamingBatchEnvelope(records, n, tuple([1] * n), epoch)
            if rows != shard.rows:
                raise ValueError(f"prepared shard {shard.path} has {rows} rows, manifest says {shard.rows}")
        yield StreamingBatchEnvelope((), 0, (), epoch, is_epoch_end=True)
