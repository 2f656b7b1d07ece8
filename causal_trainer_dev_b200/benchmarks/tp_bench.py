"""Device-timed microbenchmarks of the fused tensor-parallel paths (run under torch.distributed.run).

For the projections of one Llama-3-8B layer at tp = world size and one micro-batch of 4 x 4096
tokens it reports, as max over ranks:

* all-gather -> GEMM (QKV and gate/up): the fused pull + flag-acquiring tcgen05 GEMM, the GEMM
  alone on resident data, and NCCL all-gather followed by the GEMM;
* GEMM -> reduce-scatter (O and down): the GEMM with the push epilogue plus the slab sum, the GEMM
  alone, and the GEMM followed by NCCL reduce-scatter;
* the vocabulary-parallel cut-CE forward (statistics GEMM + in-kernel exchange) against the same
  statistics combined with NCCL all-reduces.

Roofline of a fused path: the slower of FLOPs / measured bf16 peak and the bytes that must cross
NVLink per GPU / 770 GB/s (measured peer copy bandwidth per direction).
"""
from __future__ import annotations

import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> None:
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from causal_trainer_dev_b200.ops import cross_entropy as ce
    from causal_trainer_dev_b200.ops import lib as _lib
    from causal_trainer_dev_b200.ops.gemm import gemm
    from causal_trainer_dev_b200.parallel.tp import TpContext

    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", local)
    rows, d, q, kv, f, vocab = 16384, 4096, 4096, 1024, 14336, 128256
    tp = TpContext(dist.group.WORLD, dev, rows, d, fused=True)
    tp_nccl = TpContext(dist.group.WORLD, dev, rows, d, fused=False)
    peaks_file = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak = json.loads(peaks_file.read_text())["bf16_tflops"] if peaks_file.exists() else 1590.0
    link = 770e9
    out = {"world": world, "rows": rows, "peak_tflops_measured": peak}
    x_local = (torch.randn((tp.rows_per_rank, d), device=dev) * 0.5).bfloat16()
    x_full = (torch.randn((rows, d), device=dev) * 0.5).bfloat16()
    ag_bytes = (world - 1) * tp.rows_per_rank * d * 2

    def ag_gemm_case(name: str, n_local: int) -> None:
        w = (torch.randn((n_local, d), device=dev) * 0.02).bfloat16()
        y = torch.empty((rows, n_local), dtype=torch.bfloat16, device=dev)

        def fused():
            g = tp.next_slot()
            g.mine.copy_(x_local)
            gemm(tp.all_gather(g), w, out=y)
            tp.wait_gathered(g)

        def nccl():
            g = tp_nccl.next_slot()
            g.mine.copy_(x_local)
            gemm(tp_nccl.all_gather(g), w, out=y)

        flops = 2.0 * rows * n_local * d
        alone = timed(lambda: gemm(x_full, w, out=y))
        fu = timed(fused)
        nc = timed(nccl)
        roof = max(flops / (peak * 1e12), ag_bytes / link) * 1e3
        out[name] = {"n_local": n_local, "gemm_alone_ms": alone, "fused_ms": fu, "nccl_then_gemm_ms": nc,
                     "roofline_ms": roof, "fused_fraction_of_roofline": roof / fu,
                     "bound": "compute" if flops / (peak * 1e12) > ag_bytes / link else "nvlink"}

    def gemm_rs_case(name: str, k_local: int) -> None:
        a = (torch.randn((rows, k_local), device=dev) * 0.5).bfloat16()
        w = (torch.randn((d, k_local), device=dev) * 0.02).bfloat16()
        y = torch.empty((rows, d), dtype=torch.bfloat16, device=dev)
        o = torch.empty((tp.rows_per_rank, d), dtype=torch.bfloat16, device=dev)

        def fused():
            tp.gemm_reduce_scatter(a, w, out=o)
            # the next push into the same receive buffer must not overtake a slow reader
            dist.barrier()

        def nccl():
            tp_nccl.gemm_reduce_scatter(a, w, out=o)
            dist.barrier()

        flops = 2.0 * rows * d * k_local
        alone = timed(lambda: gemm(a, w, out=y))
        barrier_ms = timed(lambda: dist.barrier())
        fu = timed(fused) - barrier_ms
        nc = timed(nccl) - barrier_ms
        roof = max(flops / (peak * 1e12), ag_bytes / link) * 1e3
        out[name] = {"k_local": k_local, "gemm_alone_ms": alone, "fused_ms": fu, "gemm_then_nccl_ms": nc,
                     "roofline_ms": roof, "fused_fraction_of_roofline": roof / fu,
                     "bound": "compute" if flops / (peak * 1e12) > ag_bytes / link else "nvlink"}

    ag_gemm_case("ag_gemm_qkv", (q + 2 * kv) // world)
    ag_gemm_case("ag_gemm_gate_up", 2 * f // world)
    gemm_rs_case("gemm_rs_o", q // world)
    gemm_rs_case("gemm_rs_down", f // world)

    # vocabulary-parallel cut-CE forward
    vl = vocab // world
    head = (torch.randn((vl, d), device=dev) * 0.02).bfloat16()
    targets = torch.randint(0, vocab, (rows,), device=dev)
    local_t = targets.to(torch.int32) - rank * vl
    local_t = torch.where((local_t >= 0) & (local_t < vl), local_t, torch.full_like(local_t, -1))
    weights = torch.ones(rows, device=dev)
    flops = 2.0 * rows * vl * d
    fu = timed(lambda: ce.cut_ce_forward(x_full, head, local_t, weights, 1.0, exchange=tp))
    nc = timed(lambda: ce.cut_ce_forward(x_full, head, local_t, weights, 1.0, exchange=tp_nccl))
    out["vocab_parallel_cut_ce_fwd"] = {"vocab_local": vl, "fused_exchange_ms": fu, "nccl_exchange_ms": nc,
                                        "roofline_ms": flops / (peak * 1e12) * 1e3,
                                        "fused_fraction_of_roofline": flops / (peak * 1e12) * 1e3 / fu}
    torch.cuda.synchronize()
    out["status"] = _lib.device_status(raise_on_error=False)
    if rank == 0:
        print(json.dumps(out, indent=1))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
