"""FSDP (ZeRO-3) runtime over NVLink peer memory: explicit schedule, fused collectives.

The reference gets FSDP implicitly: weights carry an ``fsdp`` axis in their PartitionSpec
and GSPMD inserts an all-gather before each use and a reduce-scatter of the gradients
(src/causal_trainer/distributed/runtime.py:334-360, src/causal_trainer/training/steps.py:
200-208, 560-588).  There is no compiler here, so the schedule is written out:

* every *unit* (embedding, one decoder layer, final norm + LM head) is one flat bf16 buffer,
  padded to ``world * CHUNK`` elements and split evenly; rank r owns slice r together with
  its AdamW moments and (with several micro-batches) an fp32 gradient accumulator;
* parameter shards live in **symmetric memory**: every rank maps every peer's arena;
* **all-gather -> GEMM**: ``acquire(unit, prefetch=next)`` launches the pull kernel for the
  next unit on a side stream; the pull publishes a flag per 128 KiB chunk and the tcgen05
  GEMMs that read the gathered weights acquire exactly the flags their B tile needs
  (``ops/csrc/gemm.cu``), so no stream-level dependency sits between transfer and math;
* **reduce-scatter -> cast -> sum-of-squares -> AdamW**: weight gradients are written in bf16
  straight into a symmetric staging slot, ``grads_ready`` publishes a flag to all peers and
  launches the fused reduce kernel on the side stream (``ops/csrc/collectives.cu``); the
  global-norm clip needs one 4-byte all-reduce, after which AdamW sweeps the shards (when
  clipping is off the update happens inside the reduce kernel);
* an NCCL-only variant of the same schedule (``fused=False``) is the measured baseline.

All cross-rank waits are bounded device-side spins; nothing here can hang a GPU.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..models.params import Unit, UnitLayout, unit_layouts
from ..ops import elementwise as ew
from ..ops import lib as _lib
from ..ops.gemm import FlagSource, register_flag_source
from ..training import losses
from ..training.optimizer import learning_rate_at
from ..training.steps import StepMetrics

CHUNK = 65536          # elements per flag (128 KiB of bf16)
N_GATHER = 3           # gathered-unit buffers (current, prefetched, draining)
N_SLOTS = 3            # gradient staging slots
PULL_CTAS = 64
REDUCE_CTAS = 64


def _ptr_array(ptrs: list[int]):
    arr = (ctypes.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


@dataclass
class _UnitState:
    layout: UnitLayout
    padded: int
    shard_elems: int
    arena_offset: int          # element offset of this unit's shard in the parameter arena
    has_gaps: bool


class _Gathered:
    def __init__(self, elems: int, device):
        self.buffer = torch.zeros(elems, dtype=torch.bfloat16, device=device)
        self.flags = torch.zeros(elems // CHUNK + 1, dtype=torch.int32, device=device)
        self.source = FlagSource(self.buffer, self.flags, CHUNK)
        self.unit: str | None = None
        self.epoch = 0
        self.pull_done = torch.cuda.Event()
        self.free_event: torch.cuda.Event | None = None   # main stream finished with the occupant
        self.valid = True                                  # resident mode: holds the current parameters
        register_flag_source(self.source)


class FsdpRuntime:
    """Weight provider (see ``training.engine``) plus the sharded optimizer step."""

    def __init__(self, cfg: ModelConfig, tcfg, device: torch.device, group=None, full_cfg: ModelConfig | None = None,
                 tp_group=None, resident: str = "auto", frozen: tuple[str, ...] = (), trainable: bool = True):
        """``cfg`` describes what this rank stores: the whole model, or (with ``tp_group``) one
        tensor-parallel slice of ``full_cfg`` (see ``parallel.tp.tp_local_config``).  ``frozen``
        names components (``lm_head`` / ``embed`` / ``norm``) that get no update: their regions of
        the arena are skipped by AdamW (moments never touched, no weight decay) and their gradient
        slots stay zero, so they do not enter the global norm
        (src/causal_trainer/training/steps.py:213-375).  ``trainable=False`` is the frozen base of
        adapter training: the runtime only shards and serves the weights (all-gather -> GEMM); it
        allocates no gradient staging, no gradient shards and no moments, and ``grads_ready`` /
        ``apply_update`` have nothing to do (src/causal_trainer/modeling/lora.py:178-200)."""
        _lib.require_gpu_lib()
        self.trainable = trainable
        self.cfg, self.tcfg, self.device = cfg, tcfg, device
        self.full_cfg = full_cfg if full_cfg is not None else cfg
        self.tp_group = tp_group
        self.tp_world = dist.get_world_size(tp_group) if tp_group is not None else 1
        self.tp_rank = dist.get_rank(tp_group) if tp_group is not None else 0
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.fused = bool(getattr(tcfg, "fused_collectives", True))
        from ..models.freezing import frozen_segments

        self.frozen = tuple(frozen)
        self.frozen_segs = frozen_segments(self.full_cfg, self.frozen)
        self.grad_dtype = torch.bfloat16
        self.main = torch.cuda.current_stream(device)
        self.side = torch.cuda.Stream(device, priority=-1)       # all-gather pulls
        self.reduce_stream = torch.cuda.Stream(device, priority=-1)  # reduce-scatter kernels
        self.spin_budget = 4_000_000_000
        L = _lib.lib()
        if self.world > L.ctb_max_ranks():
            raise ValueError("too many ranks for the peer-pointer tables")

        # ---- unit geometry ----
        self.units: dict[str, _UnitState] = {}
        off = 0
        grain = self.world * CHUNK
        for lay in unit_layouts(cfg):
            padded = (lay.numel + grain - 1) // grain * grain
            covered = sum(s.numel for s in lay.segments)
            self.units[lay.name] = _UnitState(lay, padded, padded // self.world, off, covered != lay.numel)
            off += padded // self.world
        self.arena_elems = off
        self.max_padded = max(u.padded for u in self.units.values())
        self.order = list(self.units)

        # ---- symmetric memory: parameter shards, gradient staging, signal pads ----
        n_pads = 2 * N_SLOTS * self.world + 64
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem

            gname = self.group.group_name
            try:
                symm_mem.enable_symm_mem_for_group(gname)
            except Exception:  # newer torch enables groups lazily
                pass
            self.param_arena = symm_mem.empty(self.arena_elems, dtype=torch.bfloat16, device=device)
            self.h_params = symm_mem.rendezvous(self.param_arena, gname)
            self.staging = symm_mem.empty(N_SLOTS * self.max_padded if trainable else CHUNK, dtype=torch.bfloat16,
                                          device=device)
            self.h_staging = symm_mem.rendezvous(self.staging, gname)
            self.pads = symm_mem.empty(n_pads, dtype=torch.int32, device=device)
            self.pads.zero_()
            self.h_pads = symm_mem.rendezvous(self.pads, gname)
            self.param_arena.zero_()
            self.staging.zero_()
            torch.cuda.synchronize(device)
            dist.barrier(self.group)
            self.param_ptrs = [int(p) for p in self.h_params.buffer_ptrs]
            self.staging_ptrs = [int(p) for p in self.h_staging.buffer_ptrs]
            self.pad_ptrs = [int(p) for p in self.h_pads.buffer_ptrs]
        else:
            # a group of one (pure tensor parallelism): the same kernels run on ordinary memory
            self.param_arena = torch.zeros(self.arena_elems, dtype=torch.bfloat16, device=device)
            self.staging = torch.zeros(N_SLOTS * self.max_padded if trainable else CHUNK, dtype=torch.bfloat16,
                                       device=device)
            self.pads = torch.zeros(n_pads, dtype=torch.int32, device=device)
            self.param_ptrs = [self.param_arena.data_ptr()]
            self.staging_ptrs = [self.staging.data_ptr()]
            self.pad_ptrs = [self.pads.data_ptr()]
        self.ready_base = 0                       # pads[slot*world + rank]
        self.done_base = N_SLOTS * self.world     # pads[done_base + slot*world + rank]

        # ---- local state ----
        state_elems = self.arena_elems if trainable else 0
        self.m = torch.zeros(state_elems, dtype=torch.bfloat16, device=device)
        self.v = torch.zeros(state_elems, dtype=torch.bfloat16, device=device)
        self.grad_shards = torch.zeros(state_elems, dtype=torch.bfloat16, device=device)
        self.accum: torch.Tensor | None = None
        self.sumsq = torch.zeros((len(self.units), REDUCE_CTAS * 8), dtype=torch.float32, device=device)
        self.finish_counter = torch.zeros(1, dtype=torch.int32, device=device)
        # Gathered weights: with room to spare (180 GB parts) every unit keeps its own gathered
        # buffer for the whole optimizer step, so the forward pass of the first micro-batch is the
        # only all-gather; otherwise three buffers rotate and every use re-gathers.
        total_bytes = 2 * sum(u.padded for u in self.units.values())
        free, _ = torch.cuda.mem_get_info(device)
        fits = torch.tensor([int(total_bytes < free // 4)], dtype=torch.int32, device=device)
        if self.world > 1:
            # every rank must take the same branch (the number of pulls, hence the flag epochs,
            # depends on it): the most constrained GPU decides
            dist.all_reduce(fits, op=dist.ReduceOp.MIN, group=self.group)
        if self.tp_group is not None:
            dist.all_reduce(fits, op=dist.ReduceOp.MIN, group=self.tp_group)
        self.resident = resident == "always" or (resident == "auto" and bool(fits.item()))
        self.where: dict[str, _Gathered] = {}
        # resident mode allocates a unit's gathered buffer at its first pull (the embedding unit is
        # never pulled when its rows are fetched from the peers' shards directly)
        self.gathered = [] if self.resident else [_Gathered(self.max_padded, device) for _ in range(N_GATHER)]
        self._build_region_table()
        a = tcfg.adamw
        # AdamW inside the reduce kernel: possible when no global-norm clip has to be known first
        self.fuse_adam = self.fused and a.max_grad_norm <= 0 and not self.frozen_segs and self.tp_world == 1
        self.pending_lr = 0.0
        self.slot_of: dict[str, int] = {}
        self.slot_epoch = [0] * N_SLOTS          # epoch last published for each slot
        self.slot_counter = 0
        self.epoch = 0
        self.count = 0                           # optimizer steps taken
        self.mb_first = True
        self.mb_last = True
        self.trace: list[tuple[str, str, torch.cuda.Event, torch.cuda.Event]] | None = None   # see _traced
        self._init_parameters()

    def _traced(self, kind: str, name: str, stream):
        """Context manager: with ``self.trace`` set (``benchmarks/step_phases.py``) brackets the
        launches issued inside it with timing events on ``stream``; otherwise does nothing."""
        import contextlib

        if self.trace is None:
            return contextlib.nullcontext()

        @contextlib.contextmanager
        def bracket():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            yield
            b.record(stream)
            self.trace.append((kind, name, a, b))
        return bracket()

    # ------------------------------------------------------------------ parameters
    def shard_view(self, name: str, of: torch.Tensor | None = None) -> torch.Tensor:
        u = self.units[name]
        base = self.param_arena if of is None else of
        return base[u.arena_offset:u.arena_offset + u.shard_elems]

    def _init_parameters(self) -> None:
        """Random N(0, initializer_range) weights, identical to a single-replica initialisation:
        every rank draws the full unit from the same seeded generator and keeps its slice (its
        tensor-parallel slice of every segment first, then its FSDP shard of that)."""
        from .tp import slice_unit_tensor

        full_cfg = self.full_cfg
        full_layouts = {lay.name: lay for lay in unit_layouts(full_cfg)}
        gen = torch.Generator(device=self.device).manual_seed(self.tcfg.seed)
        scratch_full = torch.zeros(max(lay.numel for lay in full_layouts.values()), dtype=torch.bfloat16,
                                   device=self.device)
        scratch = torch.zeros(self.max_padded, dtype=torch.bfloat16, device=self.device) if self.tp_world > 1 else scratch_full
        if scratch.numel() < self.max_padded:
            scratch = scratch_full = torch.zeros(self.max_padded, dtype=torch.bfloat16, device=self.device)
        for name, u in self.units.items():
            scratch_full.zero_()
            full_unit = Unit(full_layouts[name], scratch_full)
            for seg in full_layouts[name].segments:
                t = full_unit.view(seg.name)
                if seg.name in ("ln1", "ln2", "norm"):
                    t.fill_(1.0)
                elif seg.name.endswith("_b"):
                    t.zero_()
                else:
                    t.normal_(0.0, full_cfg.initializer_range, generator=gen)
            if name == "embed":
                full_unit.view("embed")[full_cfg.pad_token_id].zero_()
            if self.tp_world > 1:
                scratch.zero_()
                unit = Unit(u.layout, scratch)
                for seg in u.layout.segments:
                    unit.view(seg.name).copy_(slice_unit_tensor(seg.name, full_unit.view(seg.name), full_cfg,
                                                                self.tp_world, self.tp_rank))
            lo = self.rank * u.shard_elems
            self.shard_view(name).copy_(scratch[lo:lo + u.shard_elems])
        del scratch, scratch_full
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def load_full_unit(self, name: str, full: torch.Tensor) -> None:
        """Stores this rank's slice of a full (unpadded) unit buffer."""
        u = self.units[name]
        lo = self.rank * u.shard_elems
        hi = min(lo + u.shard_elems, full.numel())
        view = self.shard_view(name)
        view.zero_()
        if hi > lo:
            view[:hi - lo].copy_(full[lo:hi])

    def gather_full_unit(self, name: str) -> torch.Tensor:
        """Full unit on every rank through NCCL (checkpoint export, tests)."""
        u = self.units[name]
        out = torch.empty(u.padded, dtype=torch.bfloat16, device=self.device)
        dist.all_gather_into_tensor(out, self.shard_view(name).contiguous(), group=self.group)
        return out[:u.layout.numel]

    def set_grad_dtype(self, dtype: torch.dtype) -> None:
        if dtype == torch.float32 and self.accum is None and self.trainable:
            self.accum = torch.zeros(self.arena_elems, dtype=torch.float32, device=self.device)

    def _build_region_table(self) -> None:
        """Cuts this rank's arena into AdamW regions: for every unit the part of its shard that
        holds vectors (no decay), the part that holds matrices (decay), and inside both the
        frozen segments (skipped).  One device table serves the single AdamW launch per step."""
        cuts: list[tuple[int, int, int]] = []          # (arena start, arena stop, mode)
        for name, u in self.units.items():
            lo, hi = self.rank * u.shard_elems, (self.rank + 1) * u.shard_elems
            marks = {lo, hi, min(max(u.layout.vector_numel, lo), hi)}
            frozen_spans = []
            for seg in u.layout.segments:
                if (name, seg.name) in self.frozen_segs:
                    a, b = max(seg.offset, lo), min(seg.offset + seg.numel, hi)
                    if b > a:
                        frozen_spans.append((a, b))
                        marks.update((a, b))
            edges = sorted(marks)
            for a, b in zip(edges[:-1], edges[1:]):
                if b <= a:
                    continue
                if any(fa <= a and b <= fb for fa, fb in frozen_spans):
                    mode = -1
                else:
                    mode = 1 if a >= u.layout.vector_numel else 0
                cuts.append((u.arena_offset + a - lo, u.arena_offset + b - lo, mode))
        merged: list[list[int]] = []
        for a, b, mode in cuts:
            if merged and merged[-1][2] == mode and merged[-1][1] == a:
                merged[-1][1] = b
            else:
                merged.append([a, b, mode])
        self.adam_regions = [(a, b, mode) for a, b, mode in merged]
        self.region_bounds = torch.tensor([r[0] for r in merged] + [self.arena_elems], dtype=torch.int64,
                                          device=self.device)
        self.region_modes = torch.tensor([r[2] for r in merged], dtype=torch.int32, device=self.device)

    def _frozen_spans(self, name: str) -> list[tuple[int, int]]:
        """Unit-local element ranges of ``name`` whose gradients are never produced."""
        u = self.units[name]
        return [(seg.offset, seg.offset + seg.numel) for seg in u.layout.segments
                if (name, seg.name) in self.frozen_segs]

    # ------------------------------------------------------------------ all-gather (pull) + flags
    def _pick_buffer(self, keep: set[str]) -> _Gathered:
        for g in self.gathered:
            if g.unit is None:
                return g
        for g in self.gathered:
            if g.unit not in keep:
                return g
        raise RuntimeError("no gathered buffer free")

    def _start_pull(self, name: str, keep: set[str]) -> _Gathered:
        if self.resident:
            g = self.where.get(name)
            if g is None:
                g = _Gathered(self.units[name].padded, self.device)
                self.gathered.append(g)
                # the buffer and its flags were just cleared on the main stream: the pull (side
                # stream) must not start before that, or the clearing would land on top of it
                fresh = torch.cuda.Event()
                fresh.record(self.main)
                g.free_event = fresh
            g.valid = True
        else:
            g = self._pick_buffer(keep | {name})
            if g.unit is not None:
                self.where.pop(g.unit, None)
        u = self.units[name]
        self.epoch += 1
        g.unit, g.epoch = name, self.epoch
        g.source.epoch = self.epoch
        g.source.spin_budget = self.spin_budget
        g.source.complete = g.pull_done
        g.source.own_start = self.rank * u.shard_elems
        g.source.own_stop = (self.rank + 1) * u.shard_elems
        self.where[name] = g
        if g.free_event is not None:
            self.side.wait_event(g.free_event)
        with torch.cuda.stream(self.side), self._traced("pull", name, self.side):
            if self.fused:
                ptrs = _ptr_array([p + 2 * u.arena_offset for p in self.param_ptrs])
                code = _lib.lib().ctb_ag_pull(ptrs, _lib.ptr(g.buffer), ctypes.c_long(u.shard_elems), self.rank,
                                              self.world, CHUNK, _lib.ptr(g.flags), ctypes.c_uint(self.epoch),
                                              PULL_CTAS, ctypes.c_void_p(self.side.cuda_stream))
                _lib.check(code, "ctb_ag_pull")
            else:
                dist.all_gather_into_tensor(g.buffer[:u.padded], self.shard_view(name), group=self.group)
                g.flags.fill_(self.epoch)
            g.pull_done.record(self.side)
        return g

    def acquire(self, name: str, prefetch: str | None = None) -> Unit:
        keep = {name} | ({prefetch} if prefetch else set())
        g = self.where.get(name)
        if g is None or not g.valid:
            g = self._start_pull(name, keep)
        if prefetch is not None and (prefetch not in self.where or not self.where[prefetch].valid):
            self._start_pull(prefetch, keep)
        u = self.units[name]
        if g.pull_done.query():
            pass                                # already complete (resident weights of an earlier pass)
        elif self.fused and name.startswith("layer."):
            # vectors (norm scales, biases) are read by non-GEMM kernels: wait for their chunks only
            nvec = max(1, math.ceil(u.layout.vector_numel / CHUNK))
            with self._traced("wait", name, self.main):
                code = _lib.lib().ctb_wait_flags(_lib.ptr(g.flags), 0, 1, nvec, ctypes.c_uint(g.epoch),
                                                 ctypes.c_longlong(self.spin_budget), _lib.stream_ptr())
            _lib.check(code, "ctb_wait_flags")
        elif self.fused and name == "final":
            with self._traced("wait", name, self.main):
                code = _lib.lib().ctb_wait_flags(_lib.ptr(g.flags), 0, 1, 1, ctypes.c_uint(g.epoch),
                                                 ctypes.c_longlong(self.spin_budget), _lib.stream_ptr())
            _lib.check(code, "ctb_wait_flags")
        else:
            with self._traced("wait", name, self.main):
                self.main.wait_event(g.pull_done)   # embedding rows are gathered at random: whole unit
        return Unit(u.layout, g.buffer[:u.layout.numel])

    def release(self, name: str) -> None:
        g = self.where.get(name)
        if g is not None:
            ev = torch.cuda.Event()
            ev.record(self.main)
            g.free_event = ev

    def prefetch(self, name: str) -> None:
        """Starts the all-gather of ``name`` without waiting for any of it."""
        g = self.where.get(name)
        if g is None or not g.valid:
            self._start_pull(name, {name})

    def embedding_rows(self, ids: torch.Tensor) -> torch.Tensor | None:
        """``embed[ids]`` fetched row by row from the shards that own the rows (16-byte peer loads
        over NVLink): the all-gather and the gather as one kernel, moving ``tokens x d`` elements
        instead of the whole table.  None when this runtime gathers through NCCL."""
        if not self.fused:
            return None
        u = self.units["embed"]
        seg = u.layout.segment("embed")
        flat = ids.reshape(-1).to(torch.int32).contiguous()
        out = torch.empty((flat.numel(), seg.shape[1]), dtype=torch.bfloat16, device=self.device)
        ptrs = _ptr_array([p + 2 * u.arena_offset for p in self.param_ptrs])
        code = _lib.lib().ctb_embed_gather_peer(_lib.ptr(flat), ptrs, self.world, ctypes.c_long(u.shard_elems),
                                                ctypes.c_long(seg.offset), _lib.ptr(out), ctypes.c_long(flat.numel()),
                                                int(seg.shape[1]), int(seg.shape[0]), _lib.stream_ptr())
        _lib.check(code, "ctb_embed_gather_peer")
        return out

    # ------------------------------------------------------------------ gradients
    def grad_buffer(self, name: str) -> torch.Tensor:
        if not self.trainable:
            raise RuntimeError("this runtime serves frozen weights: it has no gradient buffers")
        if name in self.slot_of:
            slot = self.slot_of[name]
        else:
            slot = self.slot_counter % N_SLOTS
            self.slot_counter += 1
            self.slot_of[name] = slot
            prev = self.slot_epoch[slot]
            if prev > 0 and self.fused:
                # every peer must have finished reducing the previous occupant of this slot
                with self._traced("slot", name, self.main):
                    code = _lib.lib().ctb_wait_flags(_lib.ptr(self.pads), self.done_base + slot * self.world, 1,
                                                     self.world, ctypes.c_uint(prev),
                                                     ctypes.c_longlong(self.spin_budget), _lib.stream_ptr())
                _lib.check(code, "ctb_wait_flags")
            elif prev > 0:
                self.main.wait_stream(self.reduce_stream)
            u = self.units[name]
            view = self.staging[slot * self.max_padded:slot * self.max_padded + u.padded]
            if u.has_gaps:
                view.zero_()
            else:
                view[u.layout.numel:].zero_()
                for a, b in self._frozen_spans(name):     # nothing writes these: keep them out of the norm
                    view[a:b].zero_()
        return self.staging[slot * self.max_padded:slot * self.max_padded + self.units[name].padded]

    def grads_ready(self, name: str, last_microbatch: bool) -> None:
        if not self.trainable:
            return                          # frozen base: no gradient was produced for this unit
        u = self.units[name]
        slot = self.slot_of.pop(name)
        self.epoch += 1
        epoch = self.epoch
        self.slot_epoch[slot] = epoch
        idx = self.order.index(name)
        first, last = self.mb_first, self.mb_last
        L = _lib.lib()
        off = u.arena_offset
        if self.fused:
            code = L.ctb_signal_peers(_ptr_array(self.pad_ptrs), self.world, self.ready_base + slot * self.world + self.rank,
                                      ctypes.c_uint(epoch), _lib.stream_ptr())
            _lib.check(code, "ctb_signal_peers")
            ev = torch.cuda.Event()
            ev.record(self.main)
            self.reduce_stream.wait_event(ev)
            accum = self.accum[off:off + u.shard_elems] if self.accum is not None else None
            staging = _ptr_array([p + 2 * slot * self.max_padded for p in self.staging_ptrs])
            done = _ptr_array([p + 4 * (self.done_base + slot * self.world + self.rank) for p in self.pad_ptrs])
            with torch.cuda.stream(self.reduce_stream), self._traced("reduce", name, self.reduce_stream):
                adam = int(last and self.fuse_adam)
                sl = slice(off, off + u.shard_elems)
                a = self.tcfg.adamw
                step = self.count + 1
                lo = self.rank * u.shard_elems
                decay_from = min(max(u.layout.vector_numel, lo), lo + u.shard_elems) - lo
                hyper = [self.pending_lr, a.beta1, a.beta2, a.epsilon, a.weight_decay, 1 - a.beta1 ** step,
                         1 - a.beta2 ** step] if adam else [0.0] * 7
                code = L.ctb_rs_reduce(
                    staging, ctypes.c_long(self.rank * u.shard_elems), ctypes.c_long(u.shard_elems), self.world,
                    _lib.ptr(self.pads), self.ready_base + slot * self.world, ctypes.c_uint(epoch),
                    _lib.ptr(accum), int(not first), int(last),
                    None if adam else _lib.ptr(self.grad_shards[sl]), _lib.ptr(self.sumsq[idx]),
                    adam, _lib.ptr(self.param_arena[sl]) if adam else None, _lib.ptr(self.m[sl]) if adam else None,
                    _lib.ptr(self.v[sl]) if adam else None, ctypes.c_long(decay_from),
                    *(ctypes.c_float(x) for x in hyper),
                    done, 0, _lib.ptr(self.finish_counter), REDUCE_CTAS, ctypes.c_longlong(self.spin_budget),
                    ctypes.c_void_p(self.reduce_stream.cuda_stream),
                )
                _lib.check(code, "ctb_rs_reduce")
        else:
            ev = torch.cuda.Event()
            ev.record(self.main)
            self.reduce_stream.wait_event(ev)
            with torch.cuda.stream(self.reduce_stream), self._traced("reduce", name, self.reduce_stream):
                src = self.staging[slot * self.max_padded:slot * self.max_padded + u.padded]
                red = torch.empty(u.shard_elems, dtype=torch.bfloat16, device=self.device)
                dist.reduce_scatter_tensor(red, src, group=self.group)
                if self.accum is not None:
                    acc = self.accum[off:off + u.shard_elems]
                    if first:
                        acc.copy_(red)
                    else:
                        acc.add_(red)
                    final = acc
                else:
                    final = red
                if last:
                    g = self.grad_shards[off:off + u.shard_elems]
                    g.copy_(final)
                    self.sumsq[idx].zero_()
                    self.sumsq[idx, 0] = g.float().pow(2).sum()

    # ------------------------------------------------------------------ optimizer step
    def apply_update(self, lr: float) -> torch.Tensor:
        """Global norm (one 4-byte all-reduce per axis), clip, then ONE AdamW launch over the whole
        arena; with clipping off the update already happened inside the reduce kernels.  Ends with
        a fence so that no peer pulls a shard that is still being updated."""
        a = self.tcfg.adamw
        self.main.wait_stream(self.side)
        self.main.wait_stream(self.reduce_stream)
        if not self.trainable:
            # frozen base: the weights never change, so gathered copies stay valid from step to step
            self.count += 1
            return torch.zeros((), device=self.device)
        with self._traced("norm", "all", self.main):
            total = self.sumsq.sum().reshape(1)
            if self.tp_world > 1:
                # norm scales (and shared key/value heads) are replicated over tp ranks: every copy
                # holds the same, already summed, gradient, so its square counts once
                for index, copies in self._replicated_index():
                    total = total - (1.0 - 1.0 / copies) * self.grad_shards[index].float().pow(2).sum()
                dist.all_reduce(total, group=self.tp_group)
            dist.all_reduce(total, group=self.group)      # also orders every peer's pulls before the update
            grad_norm = torch.sqrt(total)
            clip = None
            if a.max_grad_norm > 0:
                clip = torch.clamp(a.max_grad_norm / torch.clamp(grad_norm, min=1e-16), max=1.0)
                clip = torch.where(torch.isfinite(grad_norm), clip, torch.ones_like(clip))
        self.count += 1
        if not self.fuse_adam:
            with self._traced("adamw", "all", self.main):
                ew.adamw_regions(self.param_arena, self.grad_shards, self.m, self.v, self.region_bounds,
                                 self.region_modes, lr=lr, b1=a.beta1, b2=a.beta2, eps=a.epsilon,
                                 decay=a.weight_decay, step=self.count, clip=clip)
        fence = torch.zeros(1, device=self.device)
        dist.all_reduce(fence, group=self.group)          # nobody pulls before every shard is updated
        if self.resident:
            for g in self.gathered:
                g.valid = False
        else:
            self.where.clear()
            for g in self.gathered:
                g.unit = None
        return grad_norm[0]

    def _replicated_index(self) -> list[tuple[torch.Tensor, int]]:
        """``(arena positions inside this rank's shards, copies)`` of parameters that several tp
        ranks hold copies of: norm scales (all ranks) and shared key/value heads."""
        if getattr(self, "_rep_index", None) is None:
            from .tp import REPLICATED_SEGMENTS, kv_replicas

            kv_rep = kv_replicas(self.full_cfg, self.tp_world)
            ql, kvl = self.cfg.query_width, self.cfg.key_value_width
            classes: dict[int, list[torch.Tensor]] = {}
            for name, u in self.units.items():
                lo, hi = self.rank * u.shard_elems, (self.rank + 1) * u.shard_elems
                for seg in u.layout.segments:
                    if seg.name in REPLICATED_SEGMENTS:
                        a, b, copies = seg.offset, seg.offset + seg.numel, self.tp_world
                    elif kv_rep > 1 and seg.name in ("qkv_w", "qkv_b"):
                        inner = seg.numel // seg.shape[0]
                        a, b, copies = seg.offset + ql * inner, seg.offset + (ql + 2 * kvl) * inner, kv_rep
                    else:
                        continue
                    a, b = max(a, lo), min(b, hi)
                    if b > a:
                        classes.setdefault(copies, []).append(
                            torch.arange(u.arena_offset + a - lo, u.arena_offset + b - lo, device=self.device))
            self._rep_index = [(torch.cat(v), k) for k, v in classes.items()]
        return self._rep_index

    # ------------------------------------------------------------------ step driver
    def make_step(self, engine) -> "FsdpStep":
        return FsdpStep(self, engine)


class FsdpStep:
    """Counterpart of ``training.steps.TrainStep`` for sharded state."""

    def __init__(self, runtime: FsdpRuntime, engine):
        self.rt = runtime
        self.engine = engine

    @property
    def optimizer_step(self) -> int:
        return self.rt.count

    def run(self, micro_batches: list[dict[str, torch.Tensor]], lr_position: int | None = None) -> StepMetrics:
        rt = self.rt
        self.engine.options.optimizer_step = rt.count      # MoBA's dense_after_step switch
        total = None
        for b in micro_batches:
            _, w = losses.aligned_targets_and_weights(b)
            s = self.engine.select_tokens(w).sum(dtype=torch.float32)
            total = s if total is None else total + s
        total = total.reshape(1).clone()
        dist.all_reduce(total, group=rt.group)
        denom = torch.clamp(total, min=1.0)
        scale = 1.0 / denom                                # stays on the device: no host round trip per step
        if len(micro_batches) > 1:
            rt.set_grad_dtype(torch.float32)
        step = rt.count if lr_position is None else lr_position
        lr = learning_rate_at(rt.tcfg.schedule, step)
        rt.pending_lr = lr                                 # for reduce kernels that apply AdamW themselves
        nll_sum = None
        for i, batch in enumerate(micro_batches):
            rt.mb_first, rt.mb_last = i == 0, i == len(micro_batches) - 1
            nll, _ = self.engine(batch, scale, True, rt.mb_last)
            nll_sum = nll if nll_sum is None else nll_sum + nll
        nll_sum = nll_sum.reshape(1).clone()
        dist.all_reduce(nll_sum, group=rt.group)
        grad_norm = rt.apply_update(lr)
        return StepMetrics((nll_sum / denom)[0], nll_sum[0], total[0], grad_norm, lr)
