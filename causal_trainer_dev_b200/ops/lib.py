"""ctypes loader of the in-tree CUDA library and the error/status plumbing.

The library is built by :func:`causal_trainer_dev_b200.ops.build.build`.  On a machine
with a GPU a missing library is an error (ops never fall back silently to PyTorch
math); on a CPU-only host ``available()`` is False and callers use the PyTorch oracle.
"""
from __future__ import annotations

import ctypes
from functools import lru_cache

import torch

from .build import LIB_PATH


class KernelError(RuntimeError):
    """A launcher refused its arguments, a CUDA call failed, or a bounded wait ran out."""


@lru_cache(maxsize=1)
def _load() -> ctypes.CDLL | None:
    if not LIB_PATH.exists():
        return None
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.ctb_last_error.restype = ctypes.c_char_p
    return lib


def available() -> bool:
    """True when the CUDA library is built and a GPU is present."""
    return torch.cuda.is_available() and _load() is not None


def lib() -> ctypes.CDLL:
    handle = _load()
    if handle is None:
        raise KernelError(
            f"{LIB_PATH} is missing: run `python -m causal_trainer_dev_b200.ops.build` (nvcc, no GPU needed)"
        )
    return handle


def require_gpu_lib() -> None:
    """Fails loudly when a GPU is present but the native library is not."""
    if torch.cuda.is_available():
        lib()


_LAUNCHES = 0


def launch_count() -> int:
    """Number of library calls that launched kernels since import (each launches >= 1)."""
    return _LAUNCHES


def check(code: int, what: str) -> None:
    global _LAUNCHES
    _LAUNCHES += 1
    if code != 0:
        raise KernelError(f"{what}: {lib().ctb_last_error().decode()}")


def stream_ptr() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


# Where a bounded device wait gave up: the SITE_* codes of ops/csrc/*.cu.
_SITES = {
    0x0101: "gemm producer: stage never freed",
    0x0102: "gemm mma: operands never arrived",
    0x0103: "gemm mma: accumulator never drained",
    0x0104: "gemm epilogue: accumulator never completed",
    0x0105: "gemm producer: gathered-operand flag never published",
    0x0106: "gemm producer: copy still in flight at teardown",
    0x0107: "gemm: tile queue never advanced",
    0x0201: "attention forward producer: K/V slot never freed",
    0x0202: "attention forward mma: Q never arrived",
    0x0203: "attention forward mma: K/V never arrived",
    0x0204: "attention forward mma: P never published",
    0x0205: "attention forward softmax: scores never completed",
    0x0206: "attention forward softmax: P V never completed",
    0x0207: "attention forward producer: gathered K/V flag never published",
    0x0301: "attention backward producer: streamed stage never freed",
    0x0302: "attention backward mma: resident tiles never arrived",
    0x0303: "attention backward mma: streamed block never arrived",
    0x0304: "attention backward mma: P^T / dS never published",
    0x0305: "attention backward compute: S / dP never completed",
    0x0307: "attention backward compute: accumulators never completed",
    0x0401: "fsdp reduce-scatter: a peer's gradients never arrived",
    0x0402: "fsdp: flags never published",
    0x0501: "tensor-parallel all-gather: a peer's rows never became ready",
    0x0502: "tensor-parallel reduce: a peer's partial tiles never arrived",
    0x0503: "vocabulary-parallel cross-entropy: a peer's statistics never arrived",
    0x0601: "row gather: index outside the source (row skipped, zeros written)",
    0x0602: "row scatter: index outside the destination (row skipped)",
    0x0603: "MoBA grouping: gathered position outside the row space (pick dropped)",
    0x0801: "two-CTA gemm producer: stage never freed",
    0x0802: "two-CTA gemm mma: operands never arrived",
    0x0803: "two-CTA gemm mma: accumulator never drained",
    0x0804: "two-CTA gemm epilogue: accumulator never completed",
}


def device_status(raise_on_error: bool = True) -> tuple[int, int, int, int]:
    """Reads (and clears) the device status word written by bounded waits that gave up."""
    out = (ctypes.c_uint * 4)()
    if lib().ctb_status(out, stream_ptr()) != 0:        # launches nothing: not counted as a launch
        raise KernelError(f"ctb_status: {lib().ctb_last_error().decode()}")
    code, block, d0, d1 = (int(x) for x in out)
    if code and raise_on_error:
        raise KernelError(
            f"device check failed: {_SITES.get(code, hex(code))} (block {block}, detail {d0}, {d1})"
        )
    return code, block, d0, d1


def poll_device_status() -> KernelError | None:
    """The production read of the status word: call it where a step's metrics have just been read
    back (the stream is idle then, so the read costs one 16-byte copy).  Returns the error instead
    of raising so that a caller with peers can put it to a vote first; None when every bounded
    wait of the steps since the last poll completed, or when no GPU library is loaded."""
    if not available():
        return None
    try:
        device_status()
    except KernelError as exc:
        return exc
    return None
