"""Host-side data path: throughput of packing, of the streaming batch grouper and of the
materialised batch iterator, on the CPU.

    python -m causal_trainer_dev_b200.benchmarks.data_bench [--documents 20000] [--seq_len 4096]

Every case runs this package's implementation and, when the reference's pure-Python package is
importable from ``baseline/_ref`` (installed without its JAX dependencies; its ``data`` modules
need none of them), the reference's own functions on the same input, unmodified, through their
public entry points (``causal_trainer.data.packing.pack_examples``,
``causal_trainer.data.streaming_batching.iter_streaming_global_batches``,
``causal_trainer.data.batching.iter_global_batches``).  The outputs are compared (identical rows;
identical digest of the last global batch; identical first batch) before a ratio is reported.
One JSON line per case.
"""
from __future__ import annotations

import argparse
import importlib
import json
import sys
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]


def _reference(module: str):
    ref = ROOT / "baseline" / "_ref"
    if not ref.is_dir():
        return None
    sys.path.insert(0, str(ref))
    try:
        return importlib.import_module(f"causal_trainer.data.{module}")
    except Exception:  # noqa: BLE001 - any import failure means "no reference arm"
        return None
    finally:
        sys.path.remove(str(ref))


def _documents(n: int, seq_len: int, seed: int = 0) -> tuple[list[dict], int]:
    rng = np.random.default_rng(seed)
    lens = np.clip(rng.lognormal(np.log(600), 1.0, n).astype(int), 32, seq_len)
    docs = [{"input_ids": rng.integers(3, 128256, int(m)).tolist(), "attention_mask": [1] * int(m)} for m in lens]
    return docs, int(lens.sum())


def _timed(fn):
    t0 = time.perf_counter()
    out = fn()
    return out, time.perf_counter() - t0


def packing_case(docs: list[dict], tokens: int, seq_len: int) -> dict:
    from ..data import packing as ours

    rows, dt = _timed(lambda: ours.pack_examples(docs, max_length=seq_len, pad_token_id=0, packing_batch_size=1000))
    out = {"case": "pack_examples", "documents": len(docs), "tokens": tokens, "rows": len(rows), "seconds": round(dt, 3),
           "mtokens_per_s": round(tokens / dt / 1e6, 3)}
    ref = _reference("packing")
    if ref is None:
        out["reference"] = "unavailable (baseline/_ref is not installed)"
        return out
    ref_rows, ref_dt = _timed(lambda: ref.pack_examples(docs, max_length=seq_len, pad_token_id=0, packing_batch_size=1000))
    out.update(reference_seconds=round(ref_dt, 3), reference_mtokens_per_s=round(tokens / ref_dt / 1e6, 3),
               identical_rows=bool(ref_rows == rows), speedup_over_reference=round(ref_dt / dt, 2))
    return out


def _batches(mod_batching, mod_streaming, rows: list[dict], window: int, rows_per_batch: int):
    envelopes = []
    for at in range(0, len(rows), window):
        chunk = tuple(rows[at:at + window])
        envelopes.append(mod_streaming.StreamingBatchEnvelope(chunk, len(chunk), (1,) * len(chunk), 0))
    envelopes.append(mod_streaming.StreamingBatchEnvelope((), 0, (), 0, True))
    plan = mod_batching.StreamingBatchPlan.create(len(rows), rows_per_batch, 1, 1, 0)
    last, count = None, 0
    for batch in mod_batching.iter_streaming_global_batches(envelopes, plan, assistant_only_loss=False):
        last, count = batch, count + 1
    return count, mod_batching.streaming_global_batch_digest(last).hex()


def streaming_case(docs: list[dict], tokens: int, seq_len: int) -> dict:
    from ..data import packing, streaming, streaming_batching

    rows = packing.pack_examples(docs, max_length=seq_len, pad_token_id=0, packing_batch_size=1000)
    (count, digest), dt = _timed(lambda: _batches(streaming_batching, streaming, rows, 256, 32))
    out = {"case": "iter_streaming_global_batches", "rows": len(rows), "global_batches": count, "seconds": round(dt, 3),
           "mtokens_per_s": round(len(rows) * seq_len / dt / 1e6, 3)}
    ref_b, ref_s = _reference("streaming_batching"), _reference("streaming")
    if ref_b is None or ref_s is None:
        out["reference"] = "unavailable (baseline/_ref is not installed)"
        return out
    (ref_count, ref_digest), ref_dt = _timed(lambda: _batches(ref_b, ref_s, rows, 256, 32))
    out.update(reference_seconds=round(ref_dt, 3), reference_mtokens_per_s=round(len(rows) * seq_len / ref_dt / 1e6, 3),
               identical_last_batch_digest=bool(ref_count == count and ref_digest == digest),
               speedup_over_reference=round(ref_dt / dt, 2))
    return out


def _epoch(mod, dataset, rows_per_batch: int):
    plan = mod.BatchPlan.create(len(dataset), rows_per_batch, 1, 1.0, 0)
    first, count = None, 0
    for batch in mod.iter_global_batches(dataset, plan, assistant_only_loss=False, shuffle=True, seed=7):
        first = batch if first is None else first
        count += 1
    return count, first


def batching_case(docs: list[dict], tokens: int, seq_len: int) -> dict:
    """One shuffled epoch of global batches over the packed rows.  The reference collates rows that
    are Python lists (what its dataset hands out); this package keeps the packed rows as typed
    columns (``data.pipeline.PackedArrayDataset``) and gathers them by index."""
    from ..data import batching, packing
    from ..data.pipeline import PackedArrayDataset

    rows = packing.pack_examples(docs, max_length=seq_len, pad_token_id=0, packing_batch_size=1000)
    rows = rows[: len(rows) // 32 * 32]
    columns = {k: np.asarray([r[k] for r in rows], dtype=np.int32) for k in rows[0]}
    (count, first), dt = _timed(lambda: _epoch(batching, PackedArrayDataset(columns), 32))
    out = {"case": "iter_global_batches", "rows": len(rows), "global_batches": count, "seconds": round(dt, 3),
           "mtokens_per_s": round(len(rows) * seq_len / dt / 1e6, 3)}
    ref = _reference("batching")
    if ref is None:
        out["reference"] = "unavailable (baseline/_ref is not installed)"
        return out
    (ref_count, ref_first), ref_dt = _timed(lambda: _epoch(ref, rows, 32))
    same = ref_count == count and sorted(ref_first) == sorted(first) and all(
        np.array_equal(ref_first[k], first[k]) and ref_first[k].dtype == first[k].dtype for k in first)
    out.update(reference_seconds=round(ref_dt, 3), reference_mtokens_per_s=round(len(rows) * seq_len / ref_dt / 1e6, 3),
               identical_first_batch=bool(same), speedup_over_reference=round(ref_dt / dt, 2))
    return out


def main(argv: list[str] | None = None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--documents", type=int, default=20000)
    p.add_argument("--seq_len", type=int, default=4096)
    a = p.parse_args(argv)
    docs, tokens = _documents(a.documents, a.seq_len)
    for case in (packing_case, streaming_case, batching_case):
        print(json.dumps(case(docs, tokens, a.seq_len)), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
