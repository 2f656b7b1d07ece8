"""Materialised data path: load a split, shard it by process, tokenise, pack, make arrays.

Follows the reference pipeline (src/causal_trainer/data/pipeline.py): local JSON / JSONL /
Parquet / CSV / TSV files or a Hub dataset; one balanced contiguous source interval per
process (``:181-214``); tokenise + pack in memory into typed ``[rows, S]`` columns (int32,
``loss_weights`` float32) (``:255-400``); virtual zero-loss rows so the row count divides the
effective global batch without copying the columns (``:441-467``).  Rows that carry no
positive-weight shifted target are an error, never silently dropped.

Local files are read without the ``datasets`` package (plain ``json`` / ``pyarrow`` / ``csv``)
so the path works on a box without a Hub cache; Hub ids go through ``datasets.load_dataset``
with the retry policy.
"""
from __future__ import annotations

import csv
import hashlib
import json
from pathlib import Path
from typing import Any, Iterator, Mapping, Sequence

import numpy as np

from .batching import MODEL_FIELDS
from .packing import pack_examples, pad_examples
from .preprocessing import EndPromptSettings, Preprocessor, RowTable

LOCAL_SUFFIXES = {".json", ".jsonl", ".parquet", ".csv", ".tsv"}


class RecordList:
    """In-memory list of source records with the small ``datasets.Dataset`` surface we use."""

    def __init__(self, records: list[dict[str, Any]], fingerprint: str, column_names: list[str] | None = None):
        self.records = records
        self._fingerprint = fingerprint
        # kept explicitly so that an empty selection (a process with no rows) still knows its schema
        self._column_names = list(column_names) if column_names is not None else (sorted(records[0]) if records else [])

    def __len__(self) -> int:
        return len(self.records)

    def __getitem__(self, index):
        if isinstance(index, slice):
            return RecordList(self.records[index], f"{self._fingerprint}[{index.start}:{index.stop}]", self._column_names)
        if isinstance(index, str):
            return [r[index] for r in self.records]
        return self.records[index]

    def __iter__(self) -> Iterator[dict[str, Any]]:
        return iter(self.records)

    @property
    def column_names(self) -> list[str]:
        return list(self._column_names)

    @property
    def cache_files(self) -> list:
        """Always empty: records live in memory, nothing is spilled to Arrow cache files."""
        return []

    def select(self, indices, keep_in_memory: bool = True) -> "RecordList":
        idx = list(indices)
        return RecordList([self.records[i] for i in idx], hashlib.sha256(
            (self._fingerprint + json.dumps(idx[:1] + idx[-1:] + [len(idx)])).encode()).hexdigest(), self._column_names)


def iter_local_records(path: Path) -> Iterator[dict[str, Any]]:
    suffix = path.suffix.lower()
    if suffix == ".jsonl":
        with path.open("r", encoding="utf-8") as f:
            for line in f:
                if line.strip():
                    yield json.loads(line)
    elif suffix == ".json":
        text = path.read_text(encoding="utf-8").lstrip()
        if text.startswith("["):
            yield from json.loads(text)
        else:  # JSON lines in a .json file, or {"data": [...]}
            try:
                value = json.loads(text)
                yield from (value["data"] if isinstance(value, dict) and "data" in value else [value])
            except json.JSONDecodeError:
                for line in text.splitlines():
                    if line.strip():
                        yield json.loads(line)
    elif suffix == ".parquet":
        import pyarrow.parquet as pq

        pf = pq.ParquetFile(path)
        for batch in pf.iter_batches(batch_size=1024):
            yield from batch.to_pylist()
    elif suffix in (".csv", ".tsv"):
        with path.open("r", encoding="utf-8", newline="") as f:
            yield from csv.DictReader(f, delimiter="\t" if suffix == ".tsv" else ",")
    else:
        raise ValueError(f"unsupported local dataset extension: {suffix}")


def load_dataset(*args, **kwargs):
    """``datasets.load_dataset``, imported on first use (the import is slow and only Hub ids need it);
    a module-level name so that a caller (or a test) can substitute it."""
    from datasets import load_dataset as impl

    return impl(*args, **kwargs)


def load_training_split(name: str, split: str, *, token: str | None = None, config_name: str | None = None,
                        revision: str | None = None, streaming: bool = False):
    """A local tabular file (materialised, or lazily iterated when ``streaming``) or a Hub dataset."""
    path = Path(name)
    if path.is_file():
        if path.suffix.lower() not in LOCAL_SUFFIXES:
            raise ValueError(f"unsupported local dataset extension: {path.suffix.lower()}")
        if config_name is not None:
            raise ValueError("dataset_config_name is not supported for a local dataset file")
        if streaming:
            return LocalStream(path)
        stat = path.stat()
        fp = hashlib.sha256(f"{path.resolve()}:{stat.st_size}:{stat.st_mtime_ns}".encode()).hexdigest()
        return RecordList(list(iter_local_records(path)), fp)
    from ..hf_retry import retry_hf_call

    return retry_hf_call(lambda: load_dataset(name, config_name, split=split, token=token, revision=revision,
                                              streaming=streaming), description=f"load dataset {name}")


class LocalStream:
    """Re-iterable lazy reader of a local file (the streaming counterpart of :class:`RecordList`)."""

    def __init__(self, path: Path):
        self.path = path

    def __iter__(self) -> Iterator[dict[str, Any]]:
        return iter_local_records(self.path)

    def shuffle(self, seed: int, buffer_size: int) -> "ShuffledStream":
        return ShuffledStream(self, seed, buffer_size)

    def set_epoch(self, epoch: int) -> None:
        pass


class ShuffledStream:
    """Deterministic buffer shuffle of a stream; the order depends on ``seed + epoch`` only."""

    def __init__(self, source, seed: int, buffer_size: int):
        self.source, self.seed, self.buffer_size, self.epoch = source, seed, buffer_size, 0

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def __iter__(self) -> Iterator[dict[str, Any]]:
        rng = np.random.default_rng(self.seed + self.epoch)
        buf: list[dict[str, Any]] = []
        for rec in self.source:
            if len(buf) < self.buffer_size:
                buf.append(rec)
                continue
            j = int(rng.integers(0, self.buffer_size))
            buf[j], rec = rec, buf[j]
            yield rec
        rng.shuffle(buf)
        yield from buf


def contiguous_shard_bounds(size: int, process_index: int, process_count: int) -> tuple[int, int]:
    if size < 0:
        raise ValueError(f"dataset size cannot be negative, got {size}")
    if process_count <= 0:
        raise ValueError(f"process_count must be positive, got {process_count}")
    if not 0 <= process_index < process_count:
        raise ValueError(f"process_index must be in [0, {process_count}), got {process_index}")
    base, rem = divmod(size, process_count)
    start = process_index * base + min(process_index, rem)
    return start, start + base + int(process_index < rem)


def select_process_shard(dataset, *, process_index: int, process_count: int):
    """``(shard, first_source_index)``: one gap-free interval per process; empty shards keep the schema."""
    start, stop = contiguous_shard_bounds(len(dataset), process_index, process_count)
    if process_count == 1:
        return dataset, 0
    if start == stop:
        return dataset.select([], keep_in_memory=True), start
    return dataset.select(range(start, stop), keep_in_memory=True), start


def source_dataset_identity(dataset) -> bytes:
    """32-byte identity for the cross-process "same source dataset" check."""
    features = getattr(dataset, "features", None)
    if hasattr(features, "to_dict"):
        features = features.to_dict()
    payload = {"rows": len(dataset), "fingerprint": getattr(dataset, "_fingerprint", None),
               "columns": list(getattr(dataset, "column_names", ())), "features": features}
    return hashlib.sha256(json.dumps(payload, ensure_ascii=False, sort_keys=True, default=str).encode()).digest()


def prepare_training_dataset(dataset, tokenizer, *, dataset_text_field: str, max_sequence_length: int, packing: bool,
                             packing_batch_size: int, pad_token_id: int | None = None, assistant_only_loss: bool = False,
                             last_assistant_only_loss: bool = False, endprompt: EndPromptSettings | None = None,
                             num_proc: int | None = None, example_index_offset: int = 0,
                             allow_empty: bool = False, preprocessing_num_workers: int | None = None
                             ) -> list[dict[str, list]]:
    """Tokenise and pack (or pad) one process shard into fixed-length rows
    (``preprocessing_num_workers`` is the flag's own name for ``num_proc``)."""
    if num_proc is None:
        num_proc = preprocessing_num_workers
    if pad_token_id is None:       # the tokenizer's own padding id, else its end-of-text id
        pad_token_id = getattr(tokenizer, "pad_token_id", None)
        if pad_token_id is None:
            pad_token_id = getattr(tokenizer, "eos_token_id", None) or 0
    pre = Preprocessor(tokenizer, dataset_text_field, max_sequence_length, assistant_only_loss,
                       last_assistant_only_loss, endprompt)
    examples = pre.run(dataset, example_index_offset=example_index_offset, allow_empty=allow_empty,
                       num_workers=num_proc)
    if not examples:
        return RowTable()
    if packing:
        return RowTable(pack_examples(examples, max_length=max_sequence_length, pad_token_id=pad_token_id,
                                      packing_batch_size=packing_batch_size))
    return RowTable(pad_examples(examples, max_length=max_sequence_length, pad_token_id=pad_token_id))


def packed_dataset_to_arrays(rows: Sequence[Mapping[str, Sequence]], *, max_sequence_length: int,
                             assistant_only_loss: bool = False, last_assistant_only_loss: bool = False,
                             has_explicit_loss_weights: bool | None = None) -> dict[str, np.ndarray]:
    """Typed ``[rows, S]`` columns: model fields int32 (+ ``assistant_masks``) and always a float32
    ``loss_weights`` column: the rows' own weights when they carry them (EndPrompt), else the assistant
    mask in the assistant-loss modes, else the attention mask
    (src/causal_trainer/data/pipeline.py:338-393)."""
    if assistant_only_loss and last_assistant_only_loss:
        raise ValueError("assistant_only_loss and last_assistant_only_loss are mutually exclusive")
    use_assistant_mask = assistant_only_loss or last_assistant_only_loss
    names = list(MODEL_FIELDS)
    if use_assistant_mask:
        names.append("assistant_masks")
    count = len(rows)
    if has_explicit_loss_weights is None:
        has_explicit_loss_weights = count > 0 and "loss_weights" in rows[0]
    if has_explicit_loss_weights:
        names.append("loss_weights")
    out: dict[str, np.ndarray] = {}
    for name in names:
        dtype = np.float32 if name == "loss_weights" else np.int32
        col = np.zeros((count, max_sequence_length), dtype=dtype)
        for i in range(count):
            row = rows[i]
            if name not in row:
                raise ValueError(f"packed row {i} is missing field {name!r}")
            if len(row[name]) != max_sequence_length:
                raise ValueError(f"packed row {i} field {name!r} has length {len(row[name])}, expected {max_sequence_length}")
            col[i] = row[name]
        out[name] = col
    if "loss_weights" not in out:
        source = out["assistant_masks"] if use_assistant_mask else out["attention_mask"]
        out["loss_weights"] = source.astype(np.float32, copy=True)
    if not np.isfinite(out["loss_weights"]).all() or (out["loss_weights"] < 0).any():
        raise ValueError("prepared loss_weights must be finite and non-negative")
    return out


class PackedArrayDataset:
    """Row view over typed columns, with ``dummy_rows`` virtual zero-loss rows at the end."""

    def __init__(self, columns: Mapping[str, np.ndarray], dummy_rows: int = 0):
        if not columns:
            raise ValueError("a packed dataset needs at least one column")
        sizes = {int(v.shape[0]) for v in columns.values()}
        if len(sizes) != 1:
            raise ValueError("packed columns have different row counts")
        self.columns = dict(columns)
        self.real_rows = sizes.pop()
        self.dummy_rows = int(dummy_rows)
        self._dummy: dict[str, np.ndarray] | None = None
        if self.dummy_rows:
            if self.real_rows == 0:
                raise ValueError("cannot derive dummy rows from an empty dataset")
            last = {k: v[self.real_rows - 1] for k, v in self.columns.items()}
            dummy = dict(last)
            # same finite attention context as the last real row, but nothing to learn from
            dummy["loss_weights"] = np.zeros_like(last["input_ids"], dtype=np.float32)
            if "assistant_masks" in dummy:
                dummy["assistant_masks"] = np.zeros_like(last["assistant_masks"])
            self._dummy = dummy

    def __len__(self) -> int:
        return self.real_rows + self.dummy_rows

    def __getitem__(self, index: int) -> dict[str, np.ndarray]:
        if index < 0:
            index += len(self)
        if not 0 <= index < len(self):
            raise IndexError(index)
        if index >= self.real_rows:
            return dict(self._dummy)
        row = {k: v[index] for k, v in self.columns.items()}
        if self._dummy is not None and "loss_weights" not in row:
            # dummy rows carry explicit zero weights, so real rows of the same batches state theirs too
            source = row["assistant_masks"] if "assistant_masks" in row else row["attention_mask"]
            row["loss_weights"] = source.astype(np.float32)
        return row


    def take(self, indices: np.ndarray) -> dict[str, np.ndarray]:
        """Columns of the rows ``indices`` (one fancy-index per column; virtual rows included)."""
        indices = np.asarray(indices, dtype=np.int64)
        indices = np.where(indices < 0, indices + len(self), indices)
        if ((indices < 0) | (indices >= len(self))).any():
            raise IndexError("row index out of range")
        virtual = indices >= self.real_rows
        source = np.minimum(indices, self.real_rows - 1)        # a virtual row copies the last real row
        out = {k: v[source] for k, v in self.columns.items()}
        if self._dummy is not None:
            if "loss_weights" not in out:
                basis = out["assistant_masks"] if "assistant_masks" in out else out["attention_mask"]
                out["loss_weights"] = basis.astype(np.float32)
            if virtual.any():
                out["loss_weights"] = out["loss_weights"].copy()
                out["loss_weights"][virtual] = 0.0
                if "assistant_masks" in out:
                    out["assistant_masks"] = out["assistant_masks"].copy()
                    out["assistant_masks"][virtual] = 0
        return out


def first_row_without_target(columns: Mapping[str, np.ndarray], chunk: int = 4096) -> int | None:
    attention, segments = columns["attention_mask"], columns["segment_ids"]
    for start in range(0, attention.shape[0], chunk):
        a, s = attention[start:start + chunk], segments[start:start + chunk]
        if "loss_weights" in columns:
            w = columns["loss_weights"][start:start + chunk]
        elif "assistant_masks" in columns:
            w = columns["assistant_masks"][start:start + chunk].astype(np.float32)
        else:
            w = a.astype(np.float32)
        edge = (a[:, :-1] != 0) & (a[:, 1:] != 0) & (s[:, :-1] != 0) & (s[:, :-1] == s[:, 1:]) & (w[:, 1:] > 0)
        ok = edge.any(axis=1)
        if not ok.all():
            return start + int(np.flatnonzero(~ok)[0])
    return None


def pad_packed_arrays_to_batch_multiple(columns: Mapping[str, np.ndarray], *, batch_multiple: int
                                        ) -> tuple[PackedArrayDataset, int]:
    if batch_multiple <= 0:
        raise ValueError(f"batch_multiple must be positive, got {batch_multiple}")
    ds = PackedArrayDataset(columns)
    if len(ds) == 0:
        raise ValueError("global preprocessing produced no trainable packed rows")
    bad = first_row_without_target(ds.columns)
    if bad is not None:
        raise ValueError(
            f"prepared packed row {bad} has no positive-weight causal target with a valid same-segment predecessor; "
            "the trainer will not silently drop it or execute an empty optimizer step")
    dummy = (-len(ds)) % batch_multiple
    return (ds, 0) if dummy == 0 else (PackedArrayDataset(columns, dummy_rows=dummy), dummy)
