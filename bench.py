#!/usr/bin/env python
"""Headline benchmark: training tokens/s of a Llama-3-8B-shape model, seq 4096, global batch
32 sequences, bf16, FSDP over N B200s of one node (strong scaling: the global batch is fixed).
``--config`` selects the other named configurations (assistant-only SFT under FSDP x TP, 32768-token
MoBA rows, mixed AR + MaskGIT); without it the headline runs.

    python bench.py --gpus 1 --steps 3 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 3 --warmup 3

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks) on
inputs already resident on the GPU; ``e2e`` repeats the measurement through
``Trainer.train_step`` with the step's inputs copied from pinned host memory and the loss
read back every step.  Data is synthetic (packed log-normal documents, uniform token ids),
weights are random N(0, 0.02).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))



def parse() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", choices=("ours", "reference", "nccl", "torch"), default="ours",
                   help="ours: fused in-kernel collectives; nccl: same engine with NCCL-only collectives; "
                        "torch: stock PyTorch (cuBLAS, SDPA, autograd, FSDP2 over NCCL), none of our kernels; "
                        "reference: the unmodified reference trainer")
    p.add_argument("--config", default="llama8b-pretrain",
                   help="named benchmark configuration (causal_trainer_dev_b200/benchmarks/configs.py); the default is "
                        "the headline: Llama-3-8B shape, seq 4096, 32 rows, FSDP")
    p.add_argument("--attention", choices=("auto", "dense", "sparse"), default="auto",
                   help="for MoBA configurations.  auto: block-sparse passes, except on batches whose every document has at "
                        "most top_k blocks (nothing to drop: the dense kernel computes the same function); sparse: always "
                        "the block-sparse passes; dense: dense segment-masked attention (comparison)")
    p.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; invalid as a result)")
    p.add_argument("--seq-len", type=int, default=0, help="override the configuration's sequence length")
    p.add_argument("--global-batch", type=int, default=0, help="override the configuration's global batch (rows)")
    p.add_argument("--micro-batch", type=int, default=0, help="override the configuration's micro-batch rows")
    p.add_argument("--remat", choices=("auto", "full", "none"), default="auto")
    p.add_argument("--force-sharded-runtime", action="store_true",
                   help="diagnostic: run the FSDP runtime on one GPU to measure its overhead without communication")
    p.add_argument("--tp", type=int, default=0, help="tensor-parallel degree inside the N GPUs (the rest is FSDP); "
                                                     "0: what the configuration names, capped by N")
    p.add_argument("--sp", type=int, default=1, help="sequence-parallel degree (queries sharded over sp ranks, K/V gathered; "
                                                     "the sp ranks are also FSDP ranks); not with MoBA layers")
    p.add_argument("--sp-layout", choices=("contiguous", "zigzag"), default="contiguous",
                   help="which tokens of a row an sp rank computes: one slice, or chunks r and 2 sp - 1 - r (equal causal work)")
    return p.parse_args()


def reference_arm() -> None:
    """Runs the unmodified reference from ``baseline/_ref`` when that is possible at all.

    The package itself installs offline (``pip --no-deps --target baseline/_ref``), but its
    trainer imports JAX, refuses every backend but TPU and every architecture but its own, so
    on a CUDA box the arm can only report why it cannot run.
    """
    ref = ROOT / "baseline" / "_ref"
    reasons = []
    if not (ref / "causal_trainer").is_dir():
        reasons.append("baseline/_ref is not installed")
    else:
        sys.path.insert(0, str(ref))
        try:
            import jax  # noqa: F401
        except ImportError:
            reasons.append("jax/jaxlib/optax are not installed and there is no network to fetch them")
    reasons.append("the reference trainer raises for any non-TPU backend (training/runner.py:337-338), rejects every "
                   "config but its fixed 40-layer MQA model (runner.py:190-216), and its attention and loss kernels "
                   "are Pallas-TPU programs with no GPU lowering")
    print(json.dumps({"impl": "reference", "unavailable": "unavailable on this box: " + "; ".join(reasons)}))


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self) -> None:
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
            if self.path and os.path.exists(self.path):
                os.unlink(self.path)

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in Path(self.path).read_text().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(smax)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def main() -> None:
    args = parse()
    if args.impl == "reference":
        reference_arm()
        return
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 or args.force_sharded_runtime:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")

    from causal_trainer_dev_b200.api import Trainer, TrainerConfig
    from causal_trainer_dev_b200.benchmarks import configs as bench_configs
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig

    if args.config not in bench_configs.CONFIGS:
        raise SystemExit(f"unknown --config {args.config!r}; known: {sorted(bench_configs.CONFIGS)}")
    bc = bench_configs.CONFIGS[args.config]
    overrides = {"num_hidden_layers": args.layers} if args.layers else {}
    cfg = bench_configs.model_of(bc, **overrides)
    seq_len = args.seq_len or bc.seq_len
    global_batch = args.global_batch or bc.global_batch
    tp = args.tp or min(bc.tp, world)
    sp = max(1, args.sp)
    if world % (tp * sp) or global_batch % (world // (tp * sp)):
        raise SystemExit("--tp x --sp must divide the GPUs, and the data ranks the global batch")
    data_world = world // (tp * sp)
    data_rank = rank // (tp * sp)
    rows_per_rank = global_batch // data_world
    micro = min(args.micro_batch or bc.micro_batch, rows_per_rank)
    attention_options = None
    if bc.moba is not None and args.attention != "dense":
        from causal_trainer_dev_b200.models.moba import AttentionOptions

        attention_options = AttentionOptions(method="moba", moba_block_size=bc.moba[0], moba_top_k=bc.moba[1])
    tcfg = TrainerConfig(
        micro_batch_rows=micro,
        adamw=AdamWConfig(weight_decay=0.1, max_grad_norm=1.0),
        schedule=ScheduleConfig(learning_rate=2e-5, learning_rate_end=2e-6, scheduler="cosine", warmup_steps=2,
                                total_steps=1000),
        fused_collectives=(args.impl == "ours"), remat=args.remat, tp=tp, sp=sp, sp_layout=args.sp_layout,
        force_sharded_runtime=args.force_sharded_runtime, attention_options=attention_options,
        moba_dense_shortcut=args.attention != "sparse",
    )
    if args.impl == "torch":
        from causal_trainer_dev_b200.benchmarks.torch_baseline import TorchBaseline

        if tp > 1 or sp > 1 or bc.moba is not None or args.config == "qwen1.5b-maskgit-fsdp8":
            print(json.dumps({"impl": "torch", "config": args.config, "unavailable": "the stock-PyTorch arm covers "
                              "FSDP-only next-token configurations (no tensor parallelism, MoBA or MaskGIT masks)"}))
            return
        trainer = TorchBaseline(cfg, micro)
    else:
        trainer = Trainer(cfg, tcfg)

    # Two distinct global batches, identical on every rank; each rank keeps its rows (pinned).
    pool = []
    executed = []
    for seed in (11, 12):
        data = bc.make_rows(cfg, global_batch, seq_len, seed)
        executed.append(bench_configs.executed_flops_per_token(cfg, data, seq_len))
        if args.impl == "torch":
            # the same assignment of rows to ranks as the product path (equal attention cost per rank)
            from causal_trainer_dev_b200.data.batching import attention_cost_per_row, balanced_row_assignment

            rows = balanced_row_assignment(attention_cost_per_row(data["segment_ids"], data.get("attention_end")),
                                           data_world)[data_rank]
            mine = {k: torch.from_numpy(v[rows].copy()).pin_memory() for k, v in data.items()}
        else:
            mine = trainer.local_rows(data)
        pool.append(mine)
    tokens_per_step = global_batch * seq_len
    moba_note = None
    if attention_options is not None:
        from causal_trainer_dev_b200.data.batching import longest_document

        longest = max(longest_document(bc.make_rows(cfg, global_batch, seq_len, seed)["segment_ids"]) for seed in (11, 12))
        dense_equal = longest <= bc.moba[0] * bc.moba[1]
        moba_note = "MoBA block %d top_k %d (grouped by key block)" % bc.moba + (
            f"; longest document {longest} tokens" + (
                " <= top_k blocks, so nothing can be dropped and the dense kernel runs (same function)"
                if dense_equal and args.attention == "auto" else ""))

    def sync() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        m = trainer.train_step(pool[i % 2])
    sync()

    # ---------------- device-timed region ----------------
    dev_batches = [trainer.upload(b) for b in pool]
    sync()
    ours = args.impl != "torch"
    launches0 = trainer.launches() if ours else 0
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    start.record()
    for i in range(args.steps):
        metrics = trainer.train_step_device(dev_batches[i % 2])
    end.record()
    sync()
    ms = start.elapsed_time(end)
    clocks = sampler.stop() if rank == 0 else {}
    launches = trainer.launches() - launches0 if ours else 0
    loss = float(metrics.loss) if ours else float(metrics[0])

    # ---------------- end-to-end region (pinned host inputs, loss read back each step) ----------------
    h2d0, d2h0 = trainer.transfer_counters()
    sync()
    t0 = time.perf_counter()
    start.record()
    marks = [t0]
    for i in range(args.steps):
        out = trainer.train_step(pool[i % 2])
        marks.append(time.perf_counter())
    end.record()
    sync()
    e2e_ms = max(start.elapsed_time(end), (time.perf_counter() - t0) * 1e3)
    if rank == 0:
        print("e2e wall per step (ms):", [round((b - a) * 1e3, 1) for a, b in zip(marks[:-1], marks[1:])],
              "allocator retries:", torch.cuda.memory_stats().get("num_alloc_retries"), file=sys.stderr)
    h2d1, d2h1 = trainer.transfer_counters()

    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
    if rank == 0:
        ms_per_step = ms / args.steps
        value = tokens_per_step / (ms_per_step / 1e3)
        e2e_value = tokens_per_step / (e2e_ms / args.steps / 1e3)
        peaks = {}
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        if peaks_file.exists():
            peaks = json.loads(peaks_file.read_text())
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0)) * 1e12
        flops_per_token = cfg.flops_per_token(seq_len)
        executed_flops = sum(executed) / len(executed)
        result = {
            "metric": bc.metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": f"synthetic ({bc.data}; random-init N(0,0.02) weights)",
            "impl": args.impl,
            "config": {
                "name": bc.name, "model": bc.model + (f"-{args.layers}layers" if args.layers else ""),
                "global_batch": global_batch, "seq_len": seq_len,
                "parallelism": f"fsdp{data_world}" + (f"xtp{tp}" if tp > 1 else "") + (f"xsp{sp}" + ("-zigzag" if args.sp_layout == "zigzag" else "") if sp > 1 else ""),
                "attention": (getattr(trainer, "attention", None) or (
                    moba_note if attention_options is not None else "dense, segment-isolated flash attention")),
                "micro_batch_rows": micro,
                "grad_accumulation": rows_per_rank // micro, "loss": "cut cross-entropy" if ours else "F.cross_entropy on 4096-row logit chunks",
                "remat": (f"auto: activations of {trainer.engine.kept_layers}/{cfg.num_hidden_layers} layers kept in "
                          "HBM, the rest recomputed per layer") if ours else "none (autograd keeps all activations)",
                "optimizer": "AdamW, bf16 moments, global-norm clip",
                "rows_to_ranks": "equal rows and near-equal attention cost per data rank", "l2": "inputs larger than L2 (weights + state "
                "are tens of GB per GPU, 126 MB L2)",
            },
            "mfu_of_measured_sustained": value * flops_per_token / (world * peak),
            "model_flops_per_token": flops_per_token,
            # the same with the attention FLOPs the segment-isolated rows actually need (documents
            # are shorter than rows; the nominal figure charges full-row causal attention)
            "mfu_executed_flops_of_measured_sustained": value * executed_flops / (world * peak),
            "executed_flops_per_token": executed_flops,
            "loss_last_step": loss,
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": (h2d1 - h2d0) // args.steps,
                    "d2h_bytes_per_step": (d2h1 - d2h0) // args.steps, "loss": out["loss"]},
            "gpu_launches": launches,
        }
        print(json.dumps(result))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
