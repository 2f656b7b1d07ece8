"""Safetensors container: memory-mapped reader, streaming writer, header validation.

The format is written and read here directly (no ``safetensors`` package on the path), as the
reference does (src/causal_trainer/checkpointing/huggingface.py:197-330, 634-655):
8-byte little-endian header length, a JSON header padded with spaces to a multiple of 8
bytes, then the tensors back to back in header order.  BF16 is handled natively through
``torch.frombuffer``.  The reader hands out zero-copy views and row slices, so a rank that
owns a shard touches only its bytes; the writer appends one tensor at a time and never holds
more than the tensor being written.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterator, Mapping, Sequence

import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

DTYPES: dict[str, torch.dtype] = {
    "BF16": torch.bfloat16, "F16": torch.float16, "F32": torch.float32, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
DTYPE_NAMES = {v: k for k, v in DTYPES.items()}
# numpy-style spellings used by the optimizer-state manifest (src/causal_trainer/checkpointing/huggingface.py:1517-1600)
PLAIN_DTYPE_NAMES = {
    "BF16": "bfloat16", "F16": "float16", "F32": "float32", "F64": "float64", "I64": "int64", "I32": "int32",
    "I16": "int16", "I8": "int8", "U8": "uint8", "BOOL": "bool",
}


def dtype_size(name: str) -> int:
    return torch.empty(0, dtype=DTYPES[name]).element_size()


@dataclass(frozen=True)
class TensorInfo:
    dtype: str
    shape: tuple[int, ...]
    data_offsets: tuple[int, int]

    @property
    def nbytes(self) -> int:
        return self.data_offsets[1] - self.data_offsets[0]


def read_header(path: str | os.PathLike[str]) -> tuple[dict[str, TensorInfo], dict[str, str], int]:
    """Parses and validates a header without touching the payload.

    Returns ``(tensors, metadata, data_start)``.  Checks: header length sane, every dtype
    known, byte extents equal ``prod(shape) * itemsize``, extents tile the payload exactly
    (no gaps, no overlap) and end at the end of the file.
    """
    path = Path(path)
    size = path.stat().st_size
    with path.open("rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: truncated safetensors file")
        (hlen,) = struct.unpack("<Q", raw)
        if hlen <= 0 or hlen > MAX_HEADER_BYTES or 8 + hlen > size:
            raise ValueError(f"{path}: invalid safetensors header length {hlen}")
        try:
            header = json.loads(f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise ValueError(f"{path}: header is not valid JSON") from exc
    if not isinstance(header, dict):
        raise ValueError(f"{path}: header must be a JSON object")
    meta = header.pop("__metadata__", {}) or {}
    if not isinstance(meta, dict) or any(not isinstance(v, str) for v in meta.values()):
        raise ValueError(f"{path}: __metadata__ must map strings to strings")
    tensors: dict[str, TensorInfo] = {}
    for name, entry in header.items():
        try:
            dt, shape, (b0, b1) = entry["dtype"], tuple(int(x) for x in entry["shape"]), entry["data_offsets"]
        except (KeyError, TypeError, ValueError) as exc:
            raise ValueError(f"{path}: malformed entry for {name!r}") from exc
        if not isinstance(dt, str) or dt not in DTYPES:
            raise ValueError(f"{path}: unsupported dtype {dt!r} for {name!r}")
        count = 1
        for s in shape:
            if s < 0:
                raise ValueError(f"{path}: negative dimension in {name!r}")
            count *= s
        if b1 - b0 != count * dtype_size(dt) or b0 < 0:
            raise ValueError(f"{path}: byte extent of {name!r} does not match its shape")
        tensors[name] = TensorInfo(dt, shape, (int(b0), int(b1)))
    data_start = 8 + hlen
    cursor = 0
    for name, info in sorted(tensors.items(), key=lambda kv: kv[1].data_offsets[0]):
        if info.data_offsets[0] != cursor:
            raise ValueError(f"{path}: payload has a gap or overlap before {name!r}")
        cursor = info.data_offsets[1]
    if data_start + cursor != size:
        raise ValueError(f"{path}: payload size {size - data_start} does not match the header ({cursor})")
    return tensors, meta, data_start


def _view_of(buffer, **kwargs) -> torch.Tensor:
    """``torch.frombuffer`` on a read-only mapping (callers never write through these views)."""
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)
        return torch.frombuffer(buffer, **kwargs)


class SafeTensorsFile:
    """Memory-mapped read access to one file."""

    def __init__(self, path: str | os.PathLike[str]):
        self.path = Path(path)
        self.tensors, self.metadata, self._data_start = read_header(self.path)
        self._file = self.path.open("rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ) if self.path.stat().st_size else None

    def close(self) -> None:
        if self._map is not None:
            try:
                self._map.close()
            except BufferError:
                pass  # live zero-copy views keep the mapping alive until they are released
            self._map = None
        self._file.close()

    def __enter__(self) -> "SafeTensorsFile":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def keys(self) -> list[str]:
        return list(self.tensors)

    def tensor(self, name: str) -> torch.Tensor:
        """Zero-copy view of a whole tensor (read-only memory: clone before writing)."""
        info = self.tensors[name]
        count = 1
        for s in info.shape:
            count *= s
        if count == 0:
            return torch.empty(info.shape, dtype=DTYPES[info.dtype])
        flat = _view_of(self._map, dtype=DTYPES[info.dtype], count=count,
                                offset=self._data_start + info.data_offsets[0])
        return flat.view(info.shape)

    def rows(self, name: str, start: int, stop: int) -> torch.Tensor:
        """Rows ``[start, stop)`` along dim 0 — only those bytes are paged in."""
        info = self.tensors[name]
        if not info.shape:
            raise ValueError("cannot slice a scalar")
        start, stop = max(0, start), min(info.shape[0], stop)
        inner = 1
        for s in info.shape[1:]:
            inner *= s
        n = max(0, stop - start)
        if n * inner == 0:
            return torch.empty((n, *info.shape[1:]), dtype=DTYPES[info.dtype])
        esize = dtype_size(info.dtype)
        flat = _view_of(self._map, dtype=DTYPES[info.dtype], count=n * inner,
                                offset=self._data_start + info.data_offsets[0] + start * inner * esize)
        return flat.view((n, *info.shape[1:]))

    def flat_range(self, name: str, start: int, stop: int) -> torch.Tensor:
        """Elements ``[start, stop)`` of the flattened tensor."""
        info = self.tensors[name]
        esize = dtype_size(info.dtype)
        if stop <= start:
            return torch.empty(0, dtype=DTYPES[info.dtype])
        return _view_of(self._map, dtype=DTYPES[info.dtype], count=stop - start,
                                offset=self._data_start + info.data_offsets[0] + start * esize)


class SafeTensorIndex:
    """All tensors of a checkpoint directory: one ``model.safetensors`` or an indexed shard set."""

    def __init__(self, directory: str | os.PathLike[str], stem: str = "model"):
        self.directory = Path(directory)
        self.files: dict[str, SafeTensorsFile] = {}
        self.where: dict[str, str] = {}
        index = self.directory / f"{stem}.safetensors.index.json"
        single = self.directory / f"{stem}.safetensors"
        if index.is_file():
            weight_map = json.loads(index.read_text(encoding="utf-8")).get("weight_map")
            if not isinstance(weight_map, dict) or not weight_map:
                raise ValueError(f"{index}: missing weight_map")
            for key, fname in weight_map.items():
                self.where[key] = fname
            for fname in sorted(set(weight_map.values())):
                self.files[fname] = SafeTensorsFile(self.directory / fname)
            for key, fname in self.where.items():
                if key not in self.files[fname].tensors:
                    raise ValueError(f"{index}: {key!r} is not in {fname}")
        elif single.is_file():
            self.files[single.name] = SafeTensorsFile(single)
            self.where = {k: single.name for k in self.files[single.name].tensors}
        else:
            raise FileNotFoundError(f"no {stem}.safetensors or {stem}.safetensors.index.json in {self.directory}")

    def keys(self) -> list[str]:
        return list(self.where)

    def info(self, name: str) -> TensorInfo:
        return self.files[self.where[name]].tensors[name]

    def file_of(self, name: str) -> SafeTensorsFile:
        return self.files[self.where[name]]

    def tensor(self, name: str) -> torch.Tensor:
        return self.file_of(name).tensor(name)

    def close(self) -> None:
        for f in self.files.values():
            f.close()


def build_header(entries: Sequence[tuple[str, str, Sequence[int]]], metadata: Mapping[str, str] | None = None
                 ) -> tuple[bytes, dict[str, TensorInfo]]:
    """Header bytes (length prefix included) for tensors laid out in ``entries`` order."""
    header: dict[str, Any] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    infos: dict[str, TensorInfo] = {}
    cursor = 0
    for name, dt, shape in entries:
        if name in infos:
            raise ValueError(f"duplicate tensor name {name!r}")
        count = 1
        for s in shape:
            count *= int(s)
        nbytes = count * dtype_size(dt)
        infos[name] = TensorInfo(dt, tuple(int(s) for s in shape), (cursor, cursor + nbytes))
        header[name] = {"dtype": dt, "shape": [int(s) for s in shape], "data_offsets": [cursor, cursor + nbytes]}
        cursor += nbytes
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    return struct.pack("<Q", len(raw)) + raw, infos


class StreamingWriter:
    """Writes tensors one at a time, in the declared order, into ``path`` (atomically at close)."""

    def __init__(self, path: str | os.PathLike[str], entries: Sequence[tuple[str, str, Sequence[int]]],
                 metadata: Mapping[str, str] | None = None):
        self.path = Path(path)
        self.tmp = self.path.with_name(self.path.name + ".tmp")
        head, self.infos = build_header(entries, metadata)
        self.order = [e[0] for e in entries]
        self._next = 0
        self.path.parent.mkdir(parents=True, exist_ok=True)
        self._f = self.tmp.open("wb")
        self._f.write(head)

    def write(self, name: str, tensor: torch.Tensor) -> None:
        if self._next >= len(self.order) or self.order[self._next] != name:
            want = self.order[self._next] if self._next < len(self.order) else "<end>"
            raise ValueError(f"tensors must be written in header order: expected {want!r}, got {name!r}")
        info = self.infos[name]
        if tuple(tensor.shape) != info.shape or DTYPE_NAMES.get(tensor.dtype) != info.dtype:
            raise ValueError(f"{name}: tensor {tuple(tensor.shape)}/{tensor.dtype} does not match the header")
        t = tensor.detach().contiguous().cpu()
        if t.numel():
            self._f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool
                          else t.numpy().tobytes())
        self._next += 1

    def write_chunks(self, name: str, chunks: Iterator[torch.Tensor]) -> None:
        """Same as :meth:`write` for a tensor delivered as consecutive flat pieces."""
        if self._next >= len(self.order) or self.order[self._next] != name:
            raise ValueError(f"tensors must be written in header order (got {name!r})")
        info = self.infos[name]
        written = 0
        for piece in chunks:
            p = piece.detach().contiguous().cpu().reshape(-1)
            if DTYPE_NAMES.get(p.dtype) != info.dtype:
                raise ValueError(f"{name}: chunk dtype does not match the header")
            self._f.write(p.view(torch.uint8).numpy().tobytes())
            written += p.numel() * p.element_size()
        if written != info.nbytes:
            raise ValueError(f"{name}: wrote {written} bytes, header says {info.nbytes}")
        self._next += 1

    def abort(self) -> None:
        self._f.close()
        self.tmp.unlink(missing_ok=True)

    def close(self) -> None:
        if self._next != len(self.order):
            self.abort()
            raise ValueError(f"only {self._next} of {len(self.order)} tensors were written")
        self._f.flush()
        os.fsync(self._f.fileno())
        self._f.close()
        os.replace(self.tmp, self.path)


def save_file(tensors: Mapping[str, torch.Tensor], path: str | os.PathLike[str],
              metadata: Mapping[str, str] | None = None) -> None:
    entries = [(k, DTYPE_NAMES[v.dtype], tuple(v.shape)) for k, v in tensors.items()]
    w = StreamingWriter(path, entries, metadata)
    try:
        for k, v in tensors.items():
            w.write(k, v)
    except BaseException:
        w.abort()
        raise
    w.close()


def load_file(path: str | os.PathLike[str]) -> dict[str, torch.Tensor]:
    with SafeTensorsFile(path) as f:
        return {k: f.tensor(k).clone() for k in f.keys()}
