"""Builds the sm_100a CUDA library of this package in-tree with nvcc.

One shared object, ``ops/_lib/libctb200.so``, holds every kernel and its C launcher.
It is compiled for ``compute_100a/sm_100a`` only (tcgen05, TMEM and TMA need the
architecture-specific target) and is loaded through ``ctypes`` by :mod:`.lib`.
Compilation needs no GPU: nvcc cross-compiles on a CPU-only host.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
OUT_DIR = Path(__file__).resolve().parent / "_lib"
LIB_PATH = OUT_DIR / "libctb200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def _nvcc() -> str:
    for candidate in (os.environ.get("CTB_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set CTB_NVCC")


def _digest(paths: list[Path]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(_compiler_identity().encode())
    return h.hexdigest()


def _compiler_identity() -> str:
    """Release line of ``nvcc --version`` ("" without a compiler: a shipped library is then kept
    as long as the sources match)."""
    try:
        out = subprocess.run([_nvcc(), "--version"], capture_output=True, text=True, timeout=60).stdout
    except (RuntimeError, OSError, subprocess.SubprocessError):
        return ""
    return next((line.strip() for line in out.splitlines() if "release" in line), "")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every ``csrc/*.cu`` and links the shared library; returns its path."""
    srcs = sources()
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh"))
    stamp = OUT_DIR / "build.sha256"
    want = _digest(srcs + headers)
    if not force and LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == want:
        return LIB_PATH
    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()
    header_digest = _digest(headers)

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        tag = obj_dir / (src.stem + ".sha256")
        key = hashlib.sha256(src.read_bytes() + header_digest.encode()).hexdigest()
        if not force and obj.exists() and tag.exists() and tag.read_text() == key:
            return obj
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
        if verbose:
            sys.stderr.write(res.stderr)
        tag.write_text(key)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
            "-lcudart"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp.write_text(want)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
