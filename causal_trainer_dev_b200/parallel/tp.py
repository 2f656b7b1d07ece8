"""Tensor parallelism (Megatron layout, sequence-sharded activations) over NVLink peer memory.

The reference shards column-parallel weights (q/k/v, gate/up, embedding, LM head) and
row-parallel weights (o, down) over the ``tp`` mesh axis and lets GSPMD insert the activation
collectives; with ``--projection_chunk_size`` it keeps the hidden state feature-sharded and
writes ``all_gather(tp) -> RMSNorm -> GEMM`` and ``GEMM -> psum_scatter(tp)`` per token tile
(src/causal_trainer/distributed/runtime.py:334-338, src/causal_trainer/modeling/token_tiling.py:
59-64,120-128,241-246).  Here the residual stream is sharded by *token rows* over the tp ranks
and the two collectives are fused into the tcgen05 GEMMs:

* **all-gather -> GEMM**: the producer of a row shard (RMSNorm, a backward kernel) writes its
  rows in place into a symmetric ``[R, d]`` buffer and signals; a pull kernel on a side stream
  copies the peers' rows over NVLink and publishes per-chunk flags that the consuming GEMM
  acquires per A tile, starting with the rows it already owns (``ops/csrc/tp_collectives.cu``,
  ``ops/csrc/gemm.cu``).
* **GEMM -> reduce-scatter**: the GEMM epilogue stores each bf16 partial tile straight into the
  receive buffer of the rank that owns those rows and raises a flag with the last tile; the
  owner sums the ``tp`` slabs in fp32 in rank order.
* **vocab-parallel cut cross-entropy**: per-row (max, sum-exp, target logit) are exchanged
  through peer memory inside the combine kernel.

Every shard is described by a *local* ``ModelConfig`` (heads, FFN width and vocabulary divided
by ``tp``), so parameter layouts, FSDP and the optimizer work on tensor-parallel slices
unchanged.  An NCCL-only variant of the same schedule (``fused=False``) is the baseline.
"""
from __future__ import annotations

import ctypes
import dataclasses

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..ops import lib as _lib
from ..ops.gemm import FlagSource, gemm, gemm_push, register_flag_source

N_RING = 8             # symmetric gathered buffers in rotation
N_RECV = 2             # receive buffers of the reduce-scatter in rotation
PULL_CTAS = 64
REDUCE_CTAS = 148


def kv_replicas(cfg: ModelConfig, tp: int) -> int:
    """How many tp ranks hold a copy of the same key/value head (1 when every rank has its own)."""
    if cfg.num_key_value_heads % tp == 0:
        return 1
    if tp % cfg.num_key_value_heads:
        raise ValueError(f"tp={tp} must divide, or be a multiple of, the key/value heads ({cfg.num_key_value_heads})")
    return tp // cfg.num_key_value_heads


def tp_local_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    """Shapes of one tensor-parallel slice: heads, FFN width and vocabulary divided by ``tp``.

    With fewer key/value heads than ranks (MQA: one head) every rank keeps one whole K/V head, a
    copy shared by ``tp / Hkv`` ranks, as the reference replicates its single K/V head over tp
    (src/causal_trainer/kernels/efficient_attention.py:305).
    """
    if tp == 1:
        return cfg
    if cfg.num_attention_heads % tp:
        raise ValueError(f"tp={tp} must divide the query heads ({cfg.num_attention_heads})")
    rep = kv_replicas(cfg, tp)
    if cfg.intermediate_size % tp or cfg.vocab_size % tp:
        raise ValueError(f"tp={tp} must divide intermediate_size and vocab_size")
    if (cfg.intermediate_size // tp) % 8:
        raise ValueError("the per-rank FFN width must be a multiple of 8")
    local_vocab = cfg.vocab_size // tp
    eos = cfg.eos_token_id if isinstance(cfg.eos_token_id, tuple) else (cfg.eos_token_id,)
    return dataclasses.replace(
        cfg, num_attention_heads=cfg.num_attention_heads // tp,
        num_key_value_heads=1 if rep > 1 else cfg.num_key_value_heads // tp,
        intermediate_size=cfg.intermediate_size // tp, vocab_size=local_vocab,
        # token ids stay global; the slice only needs ids that validate against its own row count
        pad_token_id=min(cfg.pad_token_id, local_vocab - 1), eos_token_id=tuple(min(e, local_vocab - 1) for e in eos))


# ------------------------------------------------------------------------------ parameter slicing
def slice_unit_tensor(name: str, full: torch.Tensor, cfg: ModelConfig, tp: int, rank: int) -> torch.Tensor:
    """Tensor-parallel slice of one unit segment (``qkv_w``, ``o_w``, ... in the full model's shape)."""
    if tp == 1 or name in ("ln1", "ln2", "norm"):
        return full
    q, kv, f = cfg.query_width, cfg.key_value_width, cfg.intermediate_size
    ql, fl = q // tp, f // tp
    rep = kv_replicas(cfg, tp)
    kvl = cfg.head_dim if rep > 1 else kv // tp
    kv_index = rank // rep if rep > 1 else rank
    if name in ("qkv_w", "qkv_b"):
        parts = [full[rank * ql:(rank + 1) * ql], full[q + kv_index * kvl:q + (kv_index + 1) * kvl],
                 full[q + kv + kv_index * kvl:q + kv + (kv_index + 1) * kvl]]
        return torch.cat(parts, 0)
    if name == "gu_w":
        return torch.cat([full[rank * fl:(rank + 1) * fl], full[f + rank * fl:f + (rank + 1) * fl]], 0)
    if name == "o_w":
        return full[:, rank * ql:(rank + 1) * ql]
    if name == "down_w":
        return full[:, rank * fl:(rank + 1) * fl]
    if name in ("embed", "lm_head"):
        rows = cfg.vocab_size // tp
        return full[rank * rows:(rank + 1) * rows]
    raise KeyError(name)


def merge_unit_tensor(name: str, parts: list[torch.Tensor], cfg: ModelConfig) -> torch.Tensor:
    """Inverse of :func:`slice_unit_tensor`: the full segment from the ``tp`` slices in rank order."""
    tp = len(parts)
    if tp == 1 or name in ("ln1", "ln2", "norm"):
        return parts[0]
    ql, fl = cfg.query_width // tp, cfg.intermediate_size // tp
    rep = kv_replicas(cfg, tp)
    kvl = cfg.head_dim if rep > 1 else cfg.key_value_width // tp
    if name in ("qkv_w", "qkv_b"):
        owners = parts[::rep]                      # one rank per key/value head
        return torch.cat([p[:ql] for p in parts] + [p[ql:ql + kvl] for p in owners] + [p[ql + kvl:] for p in owners], 0)
    if name == "gu_w":
        return torch.cat([p[:fl] for p in parts] + [p[fl:] for p in parts], 0)
    if name in ("o_w", "down_w"):
        return torch.cat(parts, 1)
    if name in ("embed", "lm_head"):
        return torch.cat(parts, 0)
    raise KeyError(name)


REPLICATED_SEGMENTS = ("ln1", "ln2", "norm")


def _ptr_array(ptrs):
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


class _Push:
    """Destination description handed to ``ops.gemm.gemm_push``."""

    def __init__(self, ctx: "TpContext", buf: int, epoch: int):
        self.dest_table = ctx.recv_tables[buf]
        self.flag_table = ctx.recv_flag_tables[buf]
        self.world = ctx.world
        self.counters = ctx.counters
        self.rows_per_rank = ctx.rows_per_rank
        self.src_rank = ctx.rank
        self.ld = ctx.width
        self.epoch = epoch
        self.spin_budget = ctx.spin_budget
        self.buf = buf


class Gathered:
    """One all-gather in flight: the full ``[R, d]`` tensor and, for the owner, its row slice."""

    def __init__(self, full: torch.Tensor, mine: torch.Tensor, slot: int):
        self.full = full
        self.mine = mine
        self.slot = slot


class TpContext:
    """Buffers, flags and launch helpers of one tensor-parallel group for activations ``[rows, width]``."""

    def __init__(self, group, device: torch.device, rows: int, width: int, fused: bool = True, stats_rows: int = 0):
        _lib.require_gpu_lib()
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device
        self.fused = fused
        if rows % (self.world * 128):
            raise ValueError(f"tokens per micro-batch ({rows}) must be a multiple of 128 * tp ({128 * self.world})")
        self.rows, self.width = rows, width
        self.rows_per_rank = rows // self.world
        self.slab = self.rows_per_rank * width
        self.chunk = 65536
        while self.slab % self.chunk:
            self.chunk //= 2
        self.spin_budget = 4_000_000_000
        self.main = torch.cuda.current_stream(device)
        self.side = torch.cuda.Stream(device, priority=-1)
        self.ag_count = 0
        self.slot_count = 0
        self.rs_count = 0
        self.ce_count = 0
        self.embed_count = 0
        self.stats_rows = stats_rows or rows
        n_flags = rows * width // self.chunk
        self.flags = [torch.zeros(n_flags + 1, dtype=torch.int32, device=device) for _ in range(N_RING)]
        self.pull_done = [torch.cuda.Event() for _ in range(N_RING)]
        self.counters = torch.zeros(64, dtype=torch.int32, device=device)
        w = self.world
        # pad layout (int32): [ag ready: N_RING*w][recv: N_RECV*w][ce: w][embed: 2*w]
        self.ag_base, self.recv_base = 0, N_RING * w
        self.ce_base = self.recv_base + N_RECV * w
        self.embed_base = self.ce_base + w
        n_pads = self.embed_base + 2 * w + 16
        if fused and w > 1:
            import torch.distributed._symmetric_memory as symm_mem

            gname = group.group_name
            try:
                symm_mem.enable_symm_mem_for_group(gname)
            except Exception:
                pass

            def sym(numel, dtype):
                t = symm_mem.empty(numel, dtype=dtype, device=device)
                h = symm_mem.rendezvous(t, gname)
                t.zero_()
                return t, [int(p) for p in h.buffer_ptrs], h

            self._handles = []
            self.ring, self.ring_ptrs = [], []
            for _ in range(N_RING):
                t, ptrs, h = sym(rows * width, torch.bfloat16)
                self.ring.append(t.view(rows, width))
                self.ring_ptrs.append(ptrs)
                self._handles.append(h)
            self.recv, self.recv_ptrs = [], []
            for _ in range(N_RECV):
                t, ptrs, h = sym(rows * width, torch.bfloat16)      # [world][rows_per_rank][width]
                self.recv.append(t)
                self.recv_ptrs.append(ptrs)
                self._handles.append(h)
            self.embed_out, self.embed_out_ptrs = [], []
            for _ in range(2):
                t, ptrs, h = sym(self.slab, torch.bfloat16)
                self.embed_out.append(t.view(self.rows_per_rank, width))
                self.embed_out_ptrs.append(ptrs)
                self._handles.append(h)
            self.stats, self.stats_ptrs, h = sym(w * 3 * self.stats_rows, torch.float32)
            self._handles.append(h)
            self.pads, self.pad_ptrs, h = sym(n_pads, torch.int32)
            self._handles.append(h)
            torch.cuda.synchronize(device)
            dist.barrier(group)
            self.ring_ptr_arrays = [_ptr_array(p) for p in self.ring_ptrs]
            # the GEMM epilogue indexes these by destination rank: device-resident address tables
            self.recv_tables = [torch.tensor(p, dtype=torch.int64, device=device) for p in self.recv_ptrs]
            self.recv_flag_tables = [
                torch.tensor([p + 4 * (self.recv_base + b * w + self.rank) for p in self.pad_ptrs], dtype=torch.int64,
                             device=device) for b in range(N_RECV)]
            self.embed_ptr_arrays = [_ptr_array(p) for p in self.embed_out_ptrs]
            self.stats_ptr_array = _ptr_array(self.stats_ptrs)
            self.ce_flag_ptr_array = _ptr_array([p + 4 * (self.ce_base + self.rank) for p in self.pad_ptrs])
            self.pad_ptr_array = _ptr_array(self.pad_ptrs)
            self.sources = []
            for i in range(N_RING):
                src = FlagSource(self.ring[i], self.flags[i], self.chunk)
                src.spin_budget = self.spin_budget
                src.own_start = self.rank * self.slab
                src.own_stop = (self.rank + 1) * self.slab
                register_flag_source(src)
                self.sources.append(src)
        else:
            self.fused = False
            self.ring = [torch.zeros((rows, width), dtype=torch.bfloat16, device=device) for _ in range(N_RING)]
            self.recv = [torch.zeros(rows * width, dtype=torch.bfloat16, device=device)]

    # ------------------------------------------------------------------ all-gather
    def rows_slice(self) -> slice:
        return slice(self.rank * self.rows_per_rank, (self.rank + 1) * self.rows_per_rank)

    def next_slot(self) -> Gathered:
        """The ring buffer of the next all-gather; the caller writes its rows into ``.mine``."""
        slot = self.slot_count % N_RING
        self.slot_count += 1
        full = self.ring[slot]
        return Gathered(full, full[self.rows_slice()], slot)

    def all_gather(self, g: Gathered) -> torch.Tensor:
        """Starts the all-gather of ``g`` (rows already written by this rank); returns the full tensor.

        GEMMs that read the result acquire its chunk flags themselves; any other consumer must
        call :meth:`wait_gathered` first.
        """
        self.ag_count += 1
        epoch = self.ag_count
        if self.world == 1:
            return g.full
        if not self.fused:
            dist.all_gather_into_tensor(g.full.view(-1), g.mine.reshape(-1).clone(), group=self.group)
            return g.full
        slot = g.slot
        L = _lib.lib()
        code = L.ctb_signal_peers(self.pad_ptr_array, self.world, self.ag_base + slot * self.world + self.rank,
                                  ctypes.c_uint(epoch), _lib.stream_ptr())
        _lib.check(code, "ctb_signal_peers")
        ev = torch.cuda.Event()
        ev.record(self.main)
        self.side.wait_event(ev)
        src = self.sources[slot]
        src.epoch = epoch
        src.complete = self.pull_done[slot]
        with torch.cuda.stream(self.side):
            code = L.ctb_tp_ag_pull(self.ring_ptr_arrays[slot], ctypes.c_long(self.slab), self.rank, self.world,
                                    self.chunk, _lib.ptr(self.flags[slot]), ctypes.c_uint(epoch),
                                    _lib.ptr(self.pads[self.ag_base + slot * self.world:]), ctypes.c_uint(epoch),
                                    PULL_CTAS, ctypes.c_longlong(self.spin_budget),
                                    ctypes.c_void_p(self.side.cuda_stream))
            _lib.check(code, "ctb_tp_ag_pull")
            self.pull_done[slot].record(self.side)
        return g.full

    def wait_gathered(self, g: Gathered) -> None:
        if self.fused and self.world > 1:
            self.main.wait_event(self.pull_done[g.slot])

    def gathered_flags(self, g: Gathered) -> tuple[torch.Tensor, int, int, int] | None:
        """``(flags, chunk elements, row elements, epoch)`` of the all-gather last started on ``g``'s
        slot, for consumers that acquire the chunk flags themselves (the attention producer warp);
        None when the buffer is plain memory (one rank, NCCL variant, or the pull already finished)."""
        if not self.fused or self.world == 1 or self.pull_done[g.slot].query():
            return None
        src = self.sources[g.slot]
        return self.flags[g.slot], self.chunk, self.width, src.epoch

    def reduce_scatter_rows(self, g: Gathered, out: torch.Tensor | None = None) -> torch.Tensor:
        """Sum over the ranks of the ``[rows, width]`` partials each rank wrote into ``g.full`` (its
        own ring slot), restricted to this rank's rows: every rank publishes "my partial is complete"
        on its peers and then sums its row slice from all peers' slots with 16-byte peer loads, in
        rank order, in fp32 (the fused reduce kernel of the FSDP runtime, ``csrc/collectives.cu``)."""
        if out is None:
            out = torch.empty((self.rows_per_rank, self.width), dtype=torch.bfloat16, device=self.device)
        if self.world == 1:
            out.copy_(g.full)
            return out
        if not self.fused:
            dist.reduce_scatter_tensor(out.view(-1), g.full.reshape(-1), group=self.group)
            return out
        self.ag_count += 1
        epoch = self.ag_count
        slot = g.slot
        L = _lib.lib()
        code = L.ctb_signal_peers(self.pad_ptr_array, self.world, self.ag_base + slot * self.world + self.rank,
                                  ctypes.c_uint(epoch), _lib.stream_ptr())
        _lib.check(code, "ctb_signal_peers")
        f = ctypes.c_float
        code = L.ctb_rs_reduce(
            self.ring_ptr_arrays[slot], ctypes.c_long(self.rank * self.slab), ctypes.c_long(self.slab), self.world,
            _lib.ptr(self.pads), self.ag_base + slot * self.world, ctypes.c_uint(epoch), None, 0, 1, _lib.ptr(out), None,
            0, None, None, None, ctypes.c_long(0), *(f(0.0),) * 7, None, 0, _lib.ptr(self.counters[48:]), PULL_CTAS,
            ctypes.c_longlong(self.spin_budget), _lib.stream_ptr())
        _lib.check(code, "ctb_rs_reduce")
        return out

    # ------------------------------------------------------------------ GEMM -> reduce-scatter
    def gemm_reduce_scatter(self, a: torch.Tensor, b: torch.Tensor, *, b_mn: bool = False,
                            out: torch.Tensor | None = None) -> torch.Tensor:
        """``sum_over_tp(A @ B^T)`` restricted to this rank's rows: ``[rows_per_rank, width]`` bf16."""
        if out is None:
            out = torch.empty((self.rows_per_rank, self.width), dtype=torch.bfloat16, device=self.device)
        if self.world == 1:
            gemm(a, b, b_mn=b_mn, out=out)
            return out
        if not self.fused:
            partial = gemm(a, b, b_mn=b_mn)
            dist.reduce_scatter_tensor(out, partial, group=self.group)
            return out
        push = self.begin_push()
        gemm_push(a, b, push, b_mn=b_mn)
        return self.finish_push(push, out)

    def begin_push(self) -> _Push:
        self.rs_count += 1
        return _Push(self, self.rs_count % N_RECV, self.rs_count)

    def finish_push(self, push: _Push, out: torch.Tensor | None = None) -> torch.Tensor:
        if out is None:
            out = torch.empty((self.rows_per_rank, self.width), dtype=torch.bfloat16, device=self.device)
        code = _lib.lib().ctb_tp_reduce(_lib.ptr(self.recv[push.buf]), ctypes.c_long(self.slab), self.world,
                                        _lib.ptr(self.pads[self.recv_base + push.buf * self.world:]),
                                        ctypes.c_uint(push.epoch), _lib.ptr(out), REDUCE_CTAS,
                                        ctypes.c_longlong(self.spin_budget), _lib.stream_ptr())
        _lib.check(code, "ctb_tp_reduce")
        return out

    # ------------------------------------------------------------------ vocab-parallel pieces
    def ce_exchange(self, pmax, psum, slabs: int, tlogit, weights, grad_scale: float):
        rows = tlogit.numel()
        dev = self.device
        lse = torch.empty(rows, dtype=torch.float32, device=dev)
        coef = torch.empty(rows, dtype=torch.float32, device=dev)
        if not self.fused:
            m = pmax.max(0).values
            s = (psum * torch.exp(pmax - m)).sum(0)
            gm = m.clone()
            dist.all_reduce(gm, op=dist.ReduceOp.MAX, group=self.group)
            packed = torch.stack([s * torch.exp(m - gm), tlogit])
            dist.all_reduce(packed, group=self.group)
            lse = gm + torch.log(packed[0])
            coef = weights * grad_scale
            nll = torch.where(weights != 0, (lse - packed[1]) * weights, torch.zeros_like(lse))
            return nll.sum(), weights.sum(), lse, coef
        L = _lib.lib()
        nblk = L.ctb_ce_exchange_blocks(rows)
        bn = torch.empty(nblk, dtype=torch.float32, device=dev)
        bw = torch.empty(nblk, dtype=torch.float32, device=dev)
        self.ce_count += 1
        code = L.ctb_ce_exchange(_lib.ptr(pmax), _lib.ptr(psum), slabs, _lib.ptr(tlogit), _lib.ptr(weights),
                                 ctypes.c_float(grad_scale), _lib.ptr(lse), _lib.ptr(coef), _lib.ptr(bn), _lib.ptr(bw),
                                 rows, self.stats_rows, self.rank, self.world, self.stats_ptr_array,
                                 self.ce_flag_ptr_array, _lib.ptr(self.pads[self.ce_base:]),
                                 ctypes.c_uint(self.ce_count), _lib.ptr(self.counters[32:]),
                                 ctypes.c_longlong(self.spin_budget), _lib.stream_ptr())
        _lib.check(code, "ctb_ce_exchange")
        return bn.sum(), bw.sum(), lse, coef

    def embed_lookup(self, ids: torch.Tensor, table: torch.Tensor, vocab: int) -> torch.Tensor:
        """Rows of this rank's tokens from a vocabulary-sharded embedding table ``[vocab/tp, d]``."""
        flat = ids.reshape(-1).to(torch.int32).contiguous()
        local_rows = table.shape[0]
        lo = self.rank * local_rows
        if not self.fused:
            idx = (flat - lo).long()
            ok = (idx >= 0) & (idx < local_rows)
            rows = torch.where(ok.unsqueeze(1), table[idx.clamp(0, local_rows - 1)], torch.zeros_like(table[:1]))
            out = torch.empty((self.rows_per_rank, self.width), dtype=table.dtype, device=self.device)
            dist.reduce_scatter_tensor(out, rows.contiguous(), group=self.group)
            return out
        L = _lib.lib()
        self.embed_count += 1
        buf = self.embed_count % 2
        code = L.ctb_embed_push(_lib.ptr(flat), _lib.ptr(table), self.embed_ptr_arrays[buf], self.world,
                                ctypes.c_long(flat.numel()), self.width, vocab, lo, local_rows, self.rows_per_rank,
                                _lib.stream_ptr())
        _lib.check(code, "ctb_embed_push")
        code = L.ctb_signal_peers(self.pad_ptr_array, self.world, self.embed_base + buf * self.world + self.rank,
                                  ctypes.c_uint(self.embed_count), _lib.stream_ptr())
        _lib.check(code, "ctb_signal_peers")
        code = L.ctb_wait_flags(_lib.ptr(self.pads), self.embed_base + buf * self.world, 1, self.world,
                                ctypes.c_uint(self.embed_count), ctypes.c_longlong(self.spin_budget),
                                _lib.stream_ptr())
        _lib.check(code, "ctb_wait_flags")
        return self.embed_out[buf]

    def all_reduce_replicated(self, tensors: list[torch.Tensor]) -> None:
        """Sums the gradients of parameters that every tp rank holds a copy of (norm scales)."""
        if self.world == 1:
            return
        for t in tensors:
            dist.all_reduce(t, group=self.group)
