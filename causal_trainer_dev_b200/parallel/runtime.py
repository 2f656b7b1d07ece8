"""Distributed runtime: process bootstrap, the 5-axis rank lattice and the host control plane.

One process per GPU.  Device collectives run on NCCL (or inside our own kernels); everything
the *host* needs to agree on travels over a separate Gloo group on CPU tensors, so a control
message can never touch, let alone hang, a GPU.

Kept from the reference (src/causal_trainer/distributed/runtime.py):

* axis order ``(dp, fsdp, ep, tp, sp)``, one ``-1`` inferred, later axes vary fastest so TP
  and SP neighbours are adjacent GPUs (``:23, 187-244``);
* bootstrap from explicit flags or from the environment (torchrun, SLURM, Open MPI)
  (``:54-158``);
* named barriers whose tags must agree on every rank (``:699-705``);
* the collective **error bus**: any rank's exception is re-raised on every rank before the
  next collective (src/causal_trainer/checkpointing/huggingface.py:991-1047);
* merging per-process packed datasets in rank order as raw bytes, in bounded rounds
  (``:457-697``).
"""
from __future__ import annotations

import hashlib
import os
import pickle
from dataclasses import dataclass
from datetime import timedelta
from typing import Any, Sequence

import numpy as np
import torch
import torch.distributed as dist

AXES = ("dp", "fsdp", "ep", "tp", "sp")
_ERROR_BYTES = 4096
_MERGE_CHUNK_BYTES = 64 * 1024 * 1024
_DEFAULT_TIMEOUT_S = 1800


# --------------------------------------------------------------------------------------- bootstrap
@dataclass(frozen=True)
class ProcessEnvironment:
    coordinator: str | None
    num_processes: int
    process_id: int
    local_rank: int
    source: str


def parse_local_device_ids(value: str | Sequence[int] | None) -> tuple[int, ...] | None:
    """``--local_device_ids`` as distinct non-negative integers (None for an empty value).  One
    process drives one GPU here, so the first id is the device this process uses."""
    if value is None:
        return None
    if isinstance(value, str):
        if not value.strip():
            return None
        values = tuple(int(part.strip()) for part in value.split(","))
    else:
        values = tuple(int(item) for item in value)
    if not values or any(v < 0 for v in values) or len(set(values)) != len(values):
        raise ValueError(f"local device IDs must be distinct non-negative integers, got {values!r}")
    return values


def detect_environment(coordinator_address: str | None = None, num_processes: int | None = None,
                       process_id: int | None = None, local_device_ids: str | None = None,
                       env: dict[str, str] | None = None) -> ProcessEnvironment:
    """Explicit flags win; otherwise torchrun, SLURM, then Open MPI variables; else one process."""
    e = os.environ if env is None else env
    if num_processes is not None or process_id is not None or coordinator_address is not None:
        if num_processes is None or process_id is None:
            raise ValueError("num_processes and process_id must be given together")
        if num_processes > 1 and coordinator_address is None:
            raise ValueError("coordinator_address is required for more than one process")
        ids = parse_local_device_ids(local_device_ids)
        local = ids[0] if ids else int(e.get("LOCAL_RANK", process_id))
        return ProcessEnvironment(coordinator_address, num_processes, process_id, local, "flags")
    if "RANK" in e and "WORLD_SIZE" in e:
        addr = f"{e.get('MASTER_ADDR', '127.0.0.1')}:{e.get('MASTER_PORT', '29500')}"
        return ProcessEnvironment(addr, int(e["WORLD_SIZE"]), int(e["RANK"]), int(e.get("LOCAL_RANK", 0)), "torchrun")
    if "SLURM_PROCID" in e and "SLURM_NTASKS" in e:
        host = e.get("SLURM_LAUNCH_NODE_IPADDR") or e.get("MASTER_ADDR", "127.0.0.1")
        addr = f"{host}:{e.get('MASTER_PORT', '29500')}"
        return ProcessEnvironment(addr, int(e["SLURM_NTASKS"]), int(e["SLURM_PROCID"]), int(e.get("SLURM_LOCALID", 0)),
                                  "slurm")
    if "OMPI_COMM_WORLD_RANK" in e:
        addr = f"{e.get('MASTER_ADDR', '127.0.0.1')}:{e.get('MASTER_PORT', '29500')}"
        return ProcessEnvironment(addr, int(e["OMPI_COMM_WORLD_SIZE"]), int(e["OMPI_COMM_WORLD_RANK"]),
                                  int(e.get("OMPI_COMM_WORLD_LOCAL_RANK", 0)), "openmpi")
    return ProcessEnvironment(None, 1, 0, 0, "single")


_HOST_GROUP = None
_BARRIER_COUNT = 0


def initialize_distributed(coordinator_address: str | None = None, num_processes: int | None = None,
                           process_id: int | None = None, local_device_ids: str | None = None,
                           enabled: bool = True, timeout_s: int = _DEFAULT_TIMEOUT_S) -> ProcessEnvironment:
    """Starts ``torch.distributed`` (NCCL on GPUs, Gloo otherwise) plus the Gloo host group."""
    global _HOST_GROUP
    env = detect_environment(coordinator_address, num_processes, process_id, local_device_ids)
    if not enabled or env.num_processes == 1:
        return env
    if dist.is_initialized():
        if _HOST_GROUP is None and dist.get_backend() != "gloo":
            _HOST_GROUP = dist.new_group(backend="gloo", timeout=timedelta(seconds=timeout_s))
        return env
    host, _, port = (env.coordinator or "127.0.0.1:29500").rpartition(":")
    os.environ.setdefault("MASTER_ADDR", host or "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", port)
    cuda = torch.cuda.is_available()
    kw: dict[str, Any] = {}
    if cuda:
        torch.cuda.set_device(env.local_rank)
        kw["device_id"] = torch.device("cuda", env.local_rank)
    dist.init_process_group("nccl" if cuda else "gloo", rank=env.process_id, world_size=env.num_processes,
                            timeout=timedelta(seconds=timeout_s), **kw)
    if cuda:
        _HOST_GROUP = dist.new_group(backend="gloo", timeout=timedelta(seconds=timeout_s))
    return env


def host_group():
    """Gloo group used for every host collective (the default group when it is Gloo already)."""
    if not (dist.is_available() and dist.is_initialized()):
        return None
    return _HOST_GROUP if _HOST_GROUP is not None else dist.group.WORLD


def process_count() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def process_index() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


# --------------------------------------------------------------------------------------- mesh
def resolve_mesh_shape(spec: str | Sequence[int], world: int) -> tuple[int, ...]:
    sizes = [int(x.strip()) for x in spec.split(",")] if isinstance(spec, str) else [int(x) for x in spec]
    if len(sizes) != len(AXES):
        raise ValueError(f"sharding axis must have {len(AXES)} comma-separated entries (dp,fsdp,ep,tp,sp)")
    if sum(1 for s in sizes if s == -1) > 1:
        raise ValueError("at most one sharding axis may be -1")
    if any(s == 0 or s < -1 for s in sizes):
        raise ValueError("sharding axis sizes must be positive or -1")
    known = 1
    for s in sizes:
        if s != -1:
            known *= s
    if -1 in sizes:
        if world % known:
            raise ValueError(f"cannot infer the -1 axis: {world} devices are not divisible by {known}")
        sizes[sizes.index(-1)] = world // known
    elif known != world:
        raise ValueError(f"sharding axis product {known} does not match {world} devices")
    return tuple(sizes)


resolve_axis_dims = resolve_mesh_shape      # the name src/causal_trainer/distributed/runtime.py:187 gives it

_COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "embed_tokens", "lm_head")
_ROW_PARALLEL = ("o_proj", "down_proj")


def parameter_partition_spec(name: str) -> tuple[str | None, ...]:
    """Which mesh axis cuts which dimension of a parameter, as a tuple over the tensor's dimensions
    in the Hugging Face ``[out, in]`` layout (the rule table of
    src/causal_trainer/distributed/runtime.py:334-360, transposed to this layout).  Column-parallel
    weights (q / k / v / gate / up, embedding, head) are cut over ``tp`` along the output rows and
    row-parallel ones (o / down) along the input columns; ``fsdp`` cuts the other dimension there,
    and here cuts the flat per-layer buffer that holds a rank's tensor-parallel part.  Biases follow
    their weight's rows; norm scales are replicated over ``tp``.  ``name`` is a Hugging Face tensor
    name or a ``/``-separated path (``.../kernel`` paths are read as ``[in, out]`` and answered in
    that order)."""
    parts = [p for p in name.replace("/", ".").split(".") if p]
    leaf = parts[-1] if parts else ""
    module = next((p for p in reversed(parts) if p in _COLUMN_PARALLEL + _ROW_PARALLEL), None)
    if module is None or leaf in ("scale",) or "norm" in ".".join(parts[-2:]):
        return ()
    if leaf == "bias":
        return ("tp",) if module in _COLUMN_PARALLEL else ()
    spec = ("tp", "fsdp") if module in _COLUMN_PARALLEL else ("fsdp", "tp")
    return spec[::-1] if leaf == "kernel" else spec


@dataclass
class RankLattice:
    """Row-major lattice of ranks over ``(dp, fsdp, ep, tp, sp)``; the last axis varies fastest."""

    shape: tuple[int, ...]
    rank: int

    def __post_init__(self) -> None:
        self.world = int(np.prod(self.shape))
        self._groups: dict[tuple[str, ...], Any] = {}

    @classmethod
    def create(cls, spec: str | Sequence[int], world: int | None = None, rank: int | None = None) -> "RankLattice":
        world = process_count() if world is None else world
        return cls(resolve_mesh_shape(spec, world), process_index() if rank is None else rank)

    def size(self, axis: str) -> int:
        return self.shape[AXES.index(axis)]

    def coords(self, rank: int | None = None) -> dict[str, int]:
        r = self.rank if rank is None else rank
        out = {}
        for axis, n in zip(reversed(AXES), reversed(self.shape)):
            out[axis] = r % n
            r //= n
        return {a: out[a] for a in AXES}

    def rank_of(self, coords: dict[str, int]) -> int:
        r = 0
        for axis, n in zip(AXES, self.shape):
            r = r * n + coords[axis]
        return r

    def peers(self, axes: Sequence[str], rank: int | None = None) -> list[int]:
        """Ranks that differ from ``rank`` only along ``axes`` (sorted; includes ``rank``)."""
        base = self.coords(rank)
        out = [base]
        for axis in axes:
            out = [dict(c, **{axis: i}) for c in out for i in range(self.size(axis))]
        return sorted(self.rank_of(c) for c in out)

    def group(self, axes: Sequence[str]):
        """Process group over ``axes`` (every rank must call this for the same axes, in the same order)."""
        key = tuple(axes)
        if key in self._groups:
            return self._groups[key]
        if not (dist.is_available() and dist.is_initialized()):
            self._groups[key] = None
            return None
        mine = None
        seen: set[tuple[int, ...]] = set()
        for r in range(self.world):
            members = tuple(self.peers(axes, r))
            if members in seen:
                continue
            seen.add(members)
            g = dist.new_group(list(members))
            if self.rank in members:
                mine = g
        self._groups[key] = mine
        return mine

    def index_in(self, axes: Sequence[str]) -> int:
        return self.peers(axes).index(self.rank)

    def validate(self) -> None:
        if self.size("ep") != 1:
            raise ValueError("expert parallelism is not supported: the ep axis must be 1")


# --------------------------------------------------------------------------------------- host collectives
def _to_bytes_tensor(payload: bytes, size: int) -> torch.Tensor:
    buf = np.zeros(size, dtype=np.uint8)
    buf[: len(payload)] = np.frombuffer(payload, dtype=np.uint8)
    return torch.from_numpy(buf)


def host_allgather_bytes(payload: bytes, size: int | None = None) -> list[bytes]:
    """All-gathers one fixed-size byte string per rank (padded with zeros to ``size``)."""
    g = host_group()
    size = len(payload) if size is None else size
    if len(payload) > size:
        raise ValueError("payload exceeds the fixed message size")
    if g is None or process_count() == 1:
        return [payload.ljust(size, b"\0")]
    mine = _to_bytes_tensor(payload, size)
    out = [torch.zeros(size, dtype=torch.uint8) for _ in range(process_count())]
    dist.all_gather(out, mine, group=g)
    return [bytes(t.numpy().tobytes()) for t in out]


def host_broadcast_bytes(payload: bytes | None, size: int, src: int = 0) -> bytes:
    g = host_group()
    if g is None or process_count() == 1:
        return (payload or b"").ljust(size, b"\0")
    t = _to_bytes_tensor(payload or b"", size) if process_index() == src else torch.zeros(size, dtype=torch.uint8)
    dist.broadcast(t, src=src, group=g)
    return bytes(t.numpy().tobytes())


def assert_equal(digest: bytes, what: str) -> None:
    """Every rank must present the same 32-byte digest (arguments, dataset, resume identity, export plan)."""
    if len(digest) != 32:
        raise ValueError("assert_equal expects a 32-byte digest")
    got = host_allgather_bytes(digest, 32)
    bad = [i for i, d in enumerate(got) if d != got[0]]
    if bad:
        raise RuntimeError(f"{what} differs between processes: ranks {bad} disagree with rank 0")


def digest_of(obj: Any) -> bytes:
    import json

    return hashlib.sha256(json.dumps(obj, sort_keys=True, default=str).encode("utf-8")).digest()


def sync_processes(tag: str) -> None:
    """Named barrier: the n-th barrier of the program must carry the same tag on every rank."""
    global _BARRIER_COUNT
    _BARRIER_COUNT += 1
    if process_count() == 1:
        return
    assert_equal(hashlib.sha256(f"{_BARRIER_COUNT}:{tag}".encode()).digest(), f"barrier tag {tag!r}")


def _encode_error(error: BaseException | None) -> bytes:
    if error is None:
        return b""
    text = f"{type(error).__name__}: {error}".encode("utf-8", "replace")
    return b"\x01" + text[: _ERROR_BYTES - 1]


def raise_if_any_process_error(error: BaseException | None, stage: str) -> None:
    """Collective: if any rank passes an exception, every rank raises (its own error when it has one).

    Call it after every fallible host stage so no rank enters the next collective alone.
    """
    messages = host_allgather_bytes(_encode_error(error), _ERROR_BYTES)
    failed = [(i, m[1:].rstrip(b"\0").decode("utf-8", "replace")) for i, m in enumerate(messages) if m[:1] == b"\x01"]
    if error is not None:
        raise error
    if failed:
        rank, text = failed[0]
        raise RuntimeError(f"{stage} failed on process {rank}: {text}")


def raise_if_process_zero_error(error: BaseException | None, stage: str) -> None:
    """Collective: propagates an exception raised on process 0 (filesystem work) to every rank."""
    message = host_broadcast_bytes(_encode_error(error) if process_index() == 0 else None, _ERROR_BYTES)
    if process_index() == 0 and error is not None:
        raise error
    if message[:1] == b"\x01":
        raise RuntimeError(f"{stage} failed on process 0: {message[1:].rstrip(bytes(1)).decode('utf-8', 'replace')}")


def broadcast_object(obj: Any, src: int = 0) -> Any:
    if process_count() == 1:
        return obj
    box = [obj if process_index() == src else None]
    dist.broadcast_object_list(box, src=src, group=host_group())
    return box[0]


def allgather_object(obj: Any) -> list[Any]:
    if process_count() == 1:
        return [obj]
    out: list[Any] = [None] * process_count()
    dist.all_gather_object(out, obj, group=host_group())
    return out


def gather_object_to_zero(obj: Any) -> list[Any] | None:
    """Gathers one object per rank on rank 0 (``None`` elsewhere)."""
    if process_count() == 1:
        return [obj]
    out: list[Any] | None = [None] * process_count() if process_index() == 0 else None
    dist.gather_object(obj, out, dst=0, group=host_group())
    return out


# --------------------------------------------------------------------------------------- dataset merge
def merge_packed_host_arrays(local: dict[str, np.ndarray]) -> dict[str, np.ndarray]:
    """Concatenates every rank's packed columns in rank order; every rank gets the full result.

    Schemas must match.  Rows travel as raw bytes in rounds of at most 64 MiB, so floats are
    never re-encoded and host memory beyond the result stays bounded.
    """
    n = process_count()
    if n == 1:
        return local
    schema = {k: (str(v.dtype), tuple(v.shape[1:])) for k, v in sorted(local.items())}
    rows = int(next(iter(local.values())).shape[0]) if local else 0
    infos = allgather_object((schema, rows))
    error = None
    if any(i[0] != infos[0][0] for i in infos):
        error = ValueError("packed datasets have different columns or dtypes on different processes")
    raise_if_any_process_error(error, "packed dataset merge")
    counts = [i[1] for i in infos]
    total = sum(counts)
    out = {k: np.empty((total, *shape), dtype=np.dtype(dt)) for k, (dt, shape) in schema.items()}
    base = 0
    for src, cnt in enumerate(counts):
        for k, (dt, shape) in schema.items():
            row_bytes = int(np.dtype(dt).itemsize * int(np.prod(shape, dtype=np.int64)))
            step = max(1, _MERGE_CHUNK_BYTES // max(row_bytes, 1))
            for r0 in range(0, cnt, step):
                r1 = min(cnt, r0 + step)
                size = (r1 - r0) * row_bytes
                payload = None
                if process_index() == src:
                    payload = np.ascontiguousarray(local[k][r0:r1]).tobytes()
                raw = host_broadcast_bytes(payload, size, src=src)
                out[k][base + r0:base + r1] = np.frombuffer(raw, dtype=np.dtype(dt)).reshape((r1 - r0, *shape))
        base += cnt
    return out


def pickle_digest(obj: Any) -> bytes:
    return hashlib.sha256(pickle.dumps(obj, protocol=4)).digest()
