"""Device-timed microbenchmarks of the in-kernel NVLink collectives (run under torch.distributed.run).

Reports, as max over ranks: the all-gather pull alone at several CTA counts, the fused
reduce-scatter kernel, the flagged all-gather -> GEMM against (NCCL all-gather, then GEMM),
and the NCCL collectives of the same payload.  Roofline: bytes that cross NVLink per GPU
divided by the measured 770 GB/s per direction, or GEMM FLOPs over the measured peak.
"""
from __future__ import annotations

import ctypes
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
    import torch.distributed._symmetric_memory as symm_mem

    from causal_trainer_dev_b200.ops import gemm as G
    from causal_trainer_dev_b200.ops import lib as _lib
    from causal_trainer_dev_b200.parallel.fsdp import CHUNK, _ptr_array

    world, rank = dist.get_world_size(), dist.get_rank()
    L = _lib.lib()
    gname = dist.group.WORLD.group_name
    # one Llama-3-8B layer: 218 M parameters
    rows_n, k = 28672 + 4096, 4096            # gate|up + o_proj rows as one [N,K] weight for the GEMM test
    unit = (218_112_000 + world * CHUNK - 1) // (world * CHUNK) * (world * CHUNK)
    shard = unit // world
    arena = symm_mem.empty(shard, dtype=torch.bfloat16, device="cuda")
    h = symm_mem.rendezvous(arena, gname)
    arena.normal_(0, 0.02)
    gathered = torch.zeros(unit, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(unit // CHUNK + 1, dtype=torch.int32, device="cuda")
    ptrs = _ptr_array([int(p) for p in h.buffer_ptrs])
    torch.cuda.synchronize()
    dist.barrier()
    state = {"epoch": 0}
    out = {"world": world, "unit_MB": unit * 2 / 1e6}
    stream = torch.cuda.current_stream()

    def pull(ctas):
        def run():
            state["epoch"] += 1
            _lib.check(L.ctb_ag_pull(ptrs, _lib.ptr(gathered), ctypes.c_long(shard), rank, world, CHUNK,
                                     _lib.ptr(flags), ctypes.c_uint(state["epoch"]), ctas,
                                     ctypes.c_void_p(stream.cuda_stream)), "pull")
        return run

    remote_bytes = (world - 1) * shard * 2
    for ctas in (8, 16, 24, 32, 48, 64, 96, 148):
        ms = timed(pull(ctas))
        out[f"pull_{ctas}ctas_ms"] = ms
        out[f"pull_{ctas}ctas_GBs_remote"] = remote_bytes / ms / 1e6
    ms = timed(lambda: dist.all_gather_into_tensor(gathered, arena))
    out["nccl_allgather_ms"] = ms
    out["nccl_allgather_GBs_remote"] = remote_bytes / ms / 1e6

    # fused all-gather -> GEMM: x[M,K] @ W[N,K]^T with W = first N*K elements of the gathered unit
    m = 16384
    n = 16384
    x = torch.randn(m, k, device="cuda").bfloat16()
    y = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    w = gathered[: n * k].view(n, k)
    src = G.FlagSource(gathered, flags, CHUNK)
    src.own_start, src.own_stop = rank * shard, (rank + 1) * shard
    side = torch.cuda.Stream(priority=-1)
    flops = 2.0 * m * n * k

    def fused():
        state["epoch"] += 1
        ev = torch.cuda.Event()
        ev.record(stream)
        side.wait_event(ev)
        with torch.cuda.stream(side):
            _lib.check(L.ctb_ag_pull(ptrs, _lib.ptr(gathered), ctypes.c_long(shard), rank, world, CHUNK,
                                     _lib.ptr(flags), ctypes.c_uint(state["epoch"]), 64,
                                     ctypes.c_void_p(side.cuda_stream)), "pull")
        src.epoch = state["epoch"]
        G.register_flag_source(src)
        G.gemm(x, w, out=y)
        G.unregister_flag_source(src)
        stream.wait_stream(side)

    def unfused():
        dist.all_gather_into_tensor(gathered, arena)
        G.gemm(x, w, out=y)

    out["gemm_alone_ms"] = timed(lambda: G.gemm(x, w, out=y))
    out["fused_ag_gemm_ms"] = timed(fused)
    out["nccl_ag_then_gemm_ms"] = timed(unfused)
    out["gemm_alone_tflops"] = flops / out["gemm_alone_ms"] / 1e9
    peaks = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    peak = json.loads(peaks.read_text())["bf16_tflops"] if peaks.exists() else 1590.0
    roof_ms = max(flops / (peak * 1e12) * 1e3, remote_bytes / 770e9 * 1e3)
    out["fused_ag_gemm_roofline_ms"] = roof_ms
    out["fused_ag_gemm_fraction_of_roofline"] = roof_ms / out["fused_ag_gemm_ms"]

    # fused reduce-scatter (+cast +sumsq)
    staging = symm_mem.empty(unit, dtype=torch.bfloat16, device="cuda")
    hs = symm_mem.rendezvous(staging, gname)
    staging.normal_(0, 0.01)
    pads = symm_mem.empty(4 * world + 64, dtype=torch.int32, device="cuda")
    pads.zero_()
    hp = symm_mem.rendezvous(pads, gname)
    torch.cuda.synchronize()
    dist.barrier()
    sptr = _ptr_array([int(p) for p in hs.buffer_ptrs])
    pptr = [int(p) for p in hp.buffer_ptrs]
    grad = torch.empty(shard, dtype=torch.bfloat16, device="cuda")
    sumsq = torch.zeros(128 * 8, dtype=torch.float32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    done = _ptr_array([p + 4 * (2 * world + rank) for p in pptr])

    def reduce(ctas):
        def run():
            state["epoch"] += 1
            ep = state["epoch"]
            _lib.check(L.ctb_signal_peers(_ptr_array(pptr), world, rank, ctypes.c_uint(ep),
                                          ctypes.c_void_p(stream.cuda_stream)), "signal")
            _lib.check(L.ctb_rs_reduce(sptr, ctypes.c_long(rank * shard), ctypes.c_long(shard), world, _lib.ptr(pads), 0,
                                       ctypes.c_uint(ep), None, 0, 1, _lib.ptr(grad), _lib.ptr(sumsq), 0, None, None,
                                       None, ctypes.c_long(0), *(ctypes.c_float(0.0),) * 7, done, 0,
                                       _lib.ptr(counter), ctas, ctypes.c_longlong(4_000_000_000),
                                       ctypes.c_void_p(stream.cuda_stream)), "reduce")
        return run

    for ctas in (32, 64, 128):
        ms = timed(reduce(ctas))
        out[f"rs_fused_{ctas}ctas_ms"] = ms
        out[f"rs_fused_{ctas}ctas_GBs_remote"] = remote_bytes / ms / 1e6
    red = torch.empty(shard, dtype=torch.bfloat16, device="cuda")

    def nccl_rs():
        dist.reduce_scatter_tensor(red, staging)
        return red.float().pow(2).sum()

    out["nccl_rs_then_sumsq_ms"] = timed(nccl_rs)
    out["rs_roofline_ms"] = remote_bytes / 770e9 * 1e3
    out["status"] = _lib.device_status(raise_on_error=False)
    if rank == 0:
        print(json.dumps(out, indent=1))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
