"""Per-phase device-time breakdown of one training step (CUDA events, max over ranks).

    python -m causal_trainer_dev_b200.benchmarks.step_phases --force-sharded-runtime
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m causal_trainer_dev_b200.benchmarks.step_phases --steps 3

Phases on the main stream (one row per engine section, summed over micro-batches): embedding,
layers forward, head, layers backward, embedding backward, the optimizer tail (from the last
``grads_ready`` to the end of ``apply_update``), and the gap between steps.  Beside them, for the
sharded runtime: the busy time of the all-gather pulls and of the fused reduce kernels on their
own streams, the time the main stream spent in explicit flag waits (vector parameters, slot
reuse), and the time GEMM producer warps spent waiting for chunk flags of gathered weights (the
exposed part of all-gather -> GEMM, from a cycle counter inside the kernel).

The same model, batch and options as ``bench.py``; it prints one JSON object.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
from collections import defaultdict
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=2)
    p.add_argument("--model", default="llama3-8b")
    p.add_argument("--layers", type=int, default=0)
    p.add_argument("--seq-len", type=int, default=4096)
    p.add_argument("--global-batch", type=int, default=32)
    p.add_argument("--micro-batch", type=int, default=4)
    p.add_argument("--impl", choices=("ours", "nccl"), default="ours")
    p.add_argument("--force-sharded-runtime", action="store_true")
    p.add_argument("--contiguous-rows", action="store_true",
                   help="give rank r rows [r * n, (r + 1) * n) instead of dealing rows by attention cost")
    args = p.parse_args()

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 or args.force_sharded_runtime:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29534")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from causal_trainer_dev_b200.api import Trainer, TrainerConfig
    from causal_trainer_dev_b200.data.synthetic import pretraining_rows
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.ops import lib as _lib
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig

    cfg = preset(args.model, **({"num_hidden_layers": args.layers} if args.layers else {}))
    rows_per_rank = args.global_batch // world
    micro = min(args.micro_batch, rows_per_rank)
    tcfg = TrainerConfig(micro_batch_rows=micro, adamw=AdamWConfig(weight_decay=0.1, max_grad_norm=1.0),
                         schedule=ScheduleConfig(learning_rate=2e-5, learning_rate_end=2e-6, scheduler="cosine",
                                                 warmup_steps=2, total_steps=1000),
                         fused_collectives=args.impl == "ours", force_sharded_runtime=args.force_sharded_runtime)
    trainer = Trainer(cfg, tcfg)
    eos = int(cfg.eos_token_id if isinstance(cfg.eos_token_id, int) else cfg.eos_token_id[0])
    data = pretraining_rows(args.global_batch, args.seq_len, cfg.vocab_size, eos_token_id=eos,
                            pad_token_id=cfg.pad_token_id, median_len=600.0, sigma=1.0, min_len=32, seed=11)
    if args.contiguous_rows:
        mine = {k: torch.from_numpy(v[rank * rows_per_rank:(rank + 1) * rows_per_rank].copy()).pin_memory()
                for k, v in data.items()}
    else:
        mine = trainer.local_rows(data)
    batch = trainer.upload(mine)
    for _ in range(args.warmup):
        trainer.train_step_device(batch)
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()

    runtime = getattr(trainer, "runtime", None)
    L = _lib.lib()
    cycles = ctypes.c_ulonglong(0)
    L.ctb_gemm_flag_wait_cycles(ctypes.byref(cycles))       # clear
    sums: dict[str, float] = defaultdict(float)
    step_ms = []
    ends = []
    for _ in range(args.steps):
        trainer.engine.marks = []
        if runtime is not None:
            runtime.trace = []
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        trainer.train_step_device(batch)
        t1.record()
        torch.cuda.synchronize()
        step_ms.append(t0.elapsed_time(t1))
        marks = trainer.engine.marks
        # engine sections: each mark closes the section it names; "begin" opens a micro-batch
        prev = t0
        first_begin = None
        for name, ev in marks:
            if name == "begin":
                if first_begin is None:
                    first_begin = ev
                    sums["step prologue (loss-weight total, host sync)"] += t0.elapsed_time(ev)
                prev = ev
                continue
            sums[name] += prev.elapsed_time(ev)
            prev = ev
        sums["optimizer tail (after last backward section)"] += prev.elapsed_time(t1)
        if runtime is not None:
            for kind, name, a, b in runtime.trace:
                key = {"pull": "all-gather pulls busy (side stream)", "reduce": "reduce kernels busy (reduce stream)",
                       "wait": "main stream: flag waits before a unit", "slot": "main stream: staging-slot reuse waits",
                       "adamw": "main stream: AdamW sweep", "norm": "main stream: norm all-reduce + clip"}.get(kind, kind)
                sums[key] += a.elapsed_time(b)
            last_reduce = [b for kind, _, _, b in runtime.trace if kind == "reduce"]
            if last_reduce:
                sums["last reduce end -> step end"] += max(0.0, last_reduce[-1].elapsed_time(t1))
        ends.append(t1)
    L.ctb_gemm_flag_wait_cycles(ctypes.byref(cycles))
    trainer.engine.marks = None
    if runtime is not None:
        runtime.trace = None

    n = float(args.steps)
    names = sorted(sums)
    vals = torch.tensor([sums[k] / n for k in names] + [sum(step_ms) / n], device="cuda", dtype=torch.float64)
    wait = torch.tensor([float(cycles.value) / n], device="cuda", dtype=torch.float64)
    if dist.is_initialized() and world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(wait, op=dist.ReduceOp.MAX)
    if rank == 0:
        sm_clock_khz = torch.cuda.get_device_properties(local).clock_rate if hasattr(
            torch.cuda.get_device_properties(local), "clock_rate") else 1_965_000
        out = {
            "what": "per-step device time by phase, ms, max over ranks", "n_gpus": world, "impl": args.impl,
            "forced_sharded_runtime": bool(args.force_sharded_runtime), "model": args.model, "layers": cfg.num_hidden_layers,
            "micro_batches_per_step": rows_per_rank // micro, "steps_averaged": args.steps,
            "ms_per_step": float(vals[-1]),
            "tokens_per_s": args.global_batch * args.seq_len / (float(vals[-1]) / 1e3),
            "phases_ms": {k: round(float(v), 3) for k, v in zip(names, vals[:-1].tolist())},
            "gemm_producer_flag_wait": {
                "cycles_summed_over_ctas_per_step": float(wait[0]),
                "ms_per_cta_at_max_clock": float(wait[0]) / 148.0 / (sm_clock_khz * 1e3) * 1e3,
            },
        }
        print(json.dumps(out))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
