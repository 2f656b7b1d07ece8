"""The FSDP collective kernels against plain PyTorch, with several ranks' buffers on ONE GPU.

The kernels take a table of per-rank pointers, so a single launch over R local buffers is the
R-rank computation of one rank (nothing waits on another launch: the "peers' ready" flags are
set before the reduce starts).  The bounded waits are tested by letting them run out on flags
that nothing sets: the kernel returns, the status word names the site, the context stays usable.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptrs(tensors):
    arr = (ctypes.c_void_p * len(tensors))()
    for i, t in enumerate(tensors):
        arr[i] = t.data_ptr()
    return arr


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("world", [1, 4])
def test_all_gather_pull_copies_every_shard_and_publishes_every_flag(cuda_lib, world):
    L = cuda_lib.lib()
    chunk, chunks_per_shard = 65536, 3
    shard = chunk * chunks_per_shard
    shards = [torch.randn(shard, device="cuda").bfloat16() for _ in range(world)]
    gathered = torch.zeros(shard * world, dtype=torch.bfloat16, device="cuda")
    flags = torch.zeros(world * chunks_per_shard + 1, dtype=torch.int32, device="cuda")
    for rank in range(world):
        gathered.zero_()
        epoch = 7 + rank
        code = L.ctb_ag_pull(_ptrs(shards), cuda_lib.ptr(gathered), ctypes.c_long(shard), rank, world, chunk,
                             cuda_lib.ptr(flags), ctypes.c_uint(epoch), 16, cuda_lib.stream_ptr())
        cuda_lib.check(code, "ctb_ag_pull")
        torch.cuda.synchronize()
        assert torch.equal(gathered, torch.cat(shards))
        assert (flags[:world * chunks_per_shard] == epoch).all() and flags[-1] == 0


def _reduce(cuda_lib, staging, rank, shard, *, accum=None, accumulate_in=False, last=True, adam=None, epoch=3):
    L = cuda_lib.lib()
    world = len(staging)
    ready = torch.full((world,), epoch, dtype=torch.int32, device="cuda")
    grad = torch.zeros(shard, dtype=torch.bfloat16, device="cuda")
    sumsq = torch.zeros(64 * 8, dtype=torch.float32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    done = torch.zeros(world, dtype=torch.int32, device="cuda")
    done_ptrs = (ctypes.c_void_p * world)(*[done.data_ptr() + 4 * p for p in range(world)])
    f = ctypes.c_float
    if adam is None:
        adam_args = (0, None, None, None, ctypes.c_long(0), *(f(0.0),) * 7)
    else:
        p, m, v, decay_from, lr, b1, b2, eps, decay, step = adam
        adam_args = (1, cuda_lib.ptr(p), cuda_lib.ptr(m), cuda_lib.ptr(v), ctypes.c_long(decay_from), f(lr), f(b1), f(b2),
                     f(eps), f(decay), f(1 - b1 ** step), f(1 - b2 ** step))
    code = L.ctb_rs_reduce(_ptrs(staging), ctypes.c_long(rank * shard), ctypes.c_long(shard), world, cuda_lib.ptr(ready), 0,
                           ctypes.c_uint(epoch), cuda_lib.ptr(accum), int(accumulate_in), int(last),
                           None if adam is not None else cuda_lib.ptr(grad), cuda_lib.ptr(sumsq), *adam_args, done_ptrs, 0,
                           cuda_lib.ptr(counter), 64, ctypes.c_longlong(2_000_000_000), cuda_lib.stream_ptr())
    cuda_lib.check(code, "ctb_rs_reduce")
    torch.cuda.synchronize()
    assert (done == epoch).all() and counter.item() == 0
    return grad, sumsq.sum()


@pytest.mark.parametrize("world", [1, 4])
def test_reduce_scatter_sums_in_fp32_and_reports_the_rounded_sum_of_squares(cuda_lib, world):
    torch.manual_seed(world)
    shard = 8 * 5000
    staging = [(0.01 * torch.randn(shard * world, device="cuda")).bfloat16() for _ in range(world)]
    for rank in (0, world - 1):
        want = sum(s[rank * shard:(rank + 1) * shard].float() for s in staging)
        grad, sumsq = _reduce(cuda_lib, staging, rank, shard)
        assert torch.equal(grad, want.bfloat16())
        assert torch.allclose(sumsq, want.bfloat16().float().pow(2).sum(), rtol=1e-4)
    # micro-batch accumulation: first stores, middle adds, last adds and rounds once
    accum = torch.empty(shard, dtype=torch.float32, device="cuda")
    rank = world - 1
    one = sum(s[rank * shard:(rank + 1) * shard].float() for s in staging)
    _reduce(cuda_lib, staging, rank, shard, accum=accum, accumulate_in=False, last=False)
    assert torch.allclose(accum, one, rtol=1e-6, atol=1e-8)
    _reduce(cuda_lib, staging, rank, shard, accum=accum, accumulate_in=True, last=False)
    grad, _ = _reduce(cuda_lib, staging, rank, shard, accum=accum, accumulate_in=True, last=True)
    assert _rel(grad, 3 * one) < 4e-3


def test_reduce_scatter_with_adamw_inside_matches_reduce_then_adamw(cuda_lib):
    from causal_trainer_dev_b200.ops import elementwise as E

    torch.manual_seed(9)
    world, shard, decay_from = 2, 8 * 3000, 8 * 100
    staging = [(0.01 * torch.randn(shard * world, device="cuda")).bfloat16() for _ in range(world)]
    rank = 1
    g = sum(s[rank * shard:(rank + 1) * shard].float() for s in staging).bfloat16()
    p = torch.randn(shard, device="cuda").bfloat16()
    m = (0.01 * torch.randn(shard, device="cuda")).bfloat16()
    v = (1e-4 * torch.rand(shard, device="cuda")).bfloat16()
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    kw = dict(lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, step=4)
    E.adamw_reference(pr[:decay_from], g[:decay_from], mr[:decay_from], vr[:decay_from], decay=0.0, **kw)
    E.adamw_reference(pr[decay_from:], g[decay_from:], mr[decay_from:], vr[decay_from:], decay=0.1, **kw)
    _, sumsq = _reduce(cuda_lib, staging, rank, shard, adam=(p, m, v, decay_from, 1e-3, 0.9, 0.999, 1e-8, 0.1, 4))
    assert _rel(m, mr) < 4e-3 and _rel(v, vr) < 4e-3 and _rel(p, pr) < 1e-3
    assert torch.allclose(sumsq, g.float().pow(2).sum(), rtol=1e-4)


def test_embedding_rows_from_sharded_table(cuda_lib):
    L = cuda_lib.lib()
    torch.manual_seed(2)
    world, vocab, d, offset = 4, 1000, 96, 64          # rows straddle shard boundaries (96 does not divide the shard)
    unit = offset + vocab * d
    shard = -(-unit // (world * 8)) * 8
    full = torch.zeros(shard * world, dtype=torch.bfloat16, device="cuda")
    full[offset:unit] = torch.randn(vocab * d, device="cuda").bfloat16()
    shards = [full[r * shard:(r + 1) * shard].clone() for r in range(world)]
    ids = torch.randint(0, vocab, (777,), dtype=torch.int32, device="cuda")
    out = torch.empty(777, d, dtype=torch.bfloat16, device="cuda")
    code = L.ctb_embed_gather_peer(cuda_lib.ptr(ids), _ptrs(shards), world, ctypes.c_long(shard), ctypes.c_long(offset),
                                   cuda_lib.ptr(out), ctypes.c_long(777), d, vocab, cuda_lib.stream_ptr())
    cuda_lib.check(code, "ctb_embed_gather_peer")
    table = full[offset:unit].view(vocab, d)
    assert torch.equal(out, table[ids.long()])


def test_a_flag_wait_that_nothing_satisfies_runs_out_and_reports_its_site(cuda_lib):
    L = cuda_lib.lib()
    cuda_lib.device_status(raise_on_error=False)              # start from a clean status word
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    code = L.ctb_wait_flags(cuda_lib.ptr(flags), 1, 1, 2, ctypes.c_uint(5), ctypes.c_longlong(2_000_000),
                            cuda_lib.stream_ptr())           # ~1 ms of clock64 ticks
    cuda_lib.check(code, "ctb_wait_flags")
    with pytest.raises(cuda_lib.KernelError, match="flags never published"):
        cuda_lib.device_status()
    assert cuda_lib.device_status() == (0, 0, 0, 0)           # the read cleared it
    failure = None
    flags.fill_(5)                                            # the same wait now completes
    cuda_lib.check(L.ctb_wait_flags(cuda_lib.ptr(flags), 1, 1, 2, ctypes.c_uint(5), ctypes.c_longlong(2_000_000),
                                    cuda_lib.stream_ptr()), "ctb_wait_flags")
    failure = cuda_lib.poll_device_status()
    assert failure is None


def test_a_gemm_whose_gathered_operand_never_arrives_gives_up_and_the_next_gemm_is_correct(cuda_lib):
    from causal_trainer_dev_b200.ops import gemm as G

    cuda_lib.device_status(raise_on_error=False)
    torch.manual_seed(0)
    a = torch.randn(512, 256, device="cuda").bfloat16()
    b = torch.randn(768, 256, device="cuda").bfloat16()
    flags = torch.zeros(b.numel() // 65536 + 1, dtype=torch.int32, device="cuda")
    src = G.FlagSource(b, flags, 65536)
    src.epoch, src.spin_budget = 1, 2_000_000                 # nobody publishes epoch 1: ~1 ms budget
    G.register_flag_source(src)
    try:
        G.gemm(a, b)
        failure = cuda_lib.poll_device_status()
        assert failure is not None and "gathered-operand flag never published" in str(failure)
        flags.fill_(1)                                        # "the pull finished": same call, flags honoured
        out = G.gemm(a, b)
    finally:
        G.unregister_flag_source(src)
    assert cuda_lib.poll_device_status() is None
    assert _rel(out, a.float() @ b.float().t()) < 6e-3
