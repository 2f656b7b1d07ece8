"""Layerwise sm_100a training engine: explicit forward, recompute and backward schedule.

The reference traces one XLA program per step and lets ``jax.checkpoint(nothing_saveable)``
recompute each layer in the backward pass (src/causal_trainer/modeling/architecture.py:
777-786).  On B200 the same schedule is written out by hand, with no autograd graph and no
tracing compiler:

* forward keeps only each layer's input (residual stream + pending branch), bf16;
* backward walks the layers in reverse, re-runs the layer forward saving its internals,
  then runs the hand-derived layer backward;
* every matmul is the tcgen05 GEMM (forward, dgrad reading ``W`` in place as an MN-major
  operand, wgrad reading ``dY`` and ``X`` in place, optionally accumulating in fp32
  through TMA reduce-add), attention is the tcgen05 flash kernels, the loss is the
  projection-fused cut cross-entropy and everything else the fused memory-bound kernels;
* weights come from a *provider*: plain local buffers on one GPU, or the FSDP runtime,
  which hands out gathered unit buffers and takes gradients back for reduce-scatter.

The residual add of a layer's MLP output is fused into the next layer's input RMSNorm
(``h = resid + branch`` is produced by the norm kernel), so the residual stream is written
once per half-layer.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..models.config import ModelConfig
from ..models.params import ModelParams, Unit, embed_layout
from ..ops import attention as attn_ops
from ..ops import cross_entropy as ce
from ..ops import elementwise as ew
from ..ops import lib as _lib
from ..ops.gemm import gemm
from . import losses


class LocalProvider:
    """Weight provider for a single replica: units are used where they live."""

    def __init__(self, params: ModelParams, grad_dtype: torch.dtype):
        self.params = params
        self.grad_dtype = grad_dtype

    def acquire(self, name: str, prefetch: str | None = None) -> Unit:
        return self.params.units[name]

    def grad_buffer(self, name: str) -> torch.Tensor:
        u = self.params.units[name]
        if u.grad is None or u.grad.dtype != self.grad_dtype:
            u.grad = torch.zeros(u.layout.numel, dtype=self.grad_dtype, device=u.data.device)
        return u.grad

    def release(self, name: str) -> None:
        pass

    def prefetch(self, name: str) -> None:
        pass

    def embedding_rows(self, ids: torch.Tensor) -> torch.Tensor | None:
        return None

    def grads_ready(self, name: str, last_microbatch: bool) -> None:
        pass


@dataclass
class EngineOptions:
    cut_chunk_rows: int = 4096
    attention_options: object | None = None
    optimizer_step: int | None = None
    train_lm_head: bool = True
    train_embed: bool = True
    train_norm: bool = True
    remat: str = "auto"                      # "auto" | "full" | "none"
    overlap_wgrad: bool = False              # issue weight-gradient GEMMs on a second stream (measured: no gain)
    compact_loss_rows: bool = True           # run the LM head only on rows with non-zero loss weight
    loss_backend: str = "cut"                # "cut": projection-fused; "logits": materialised bf16 logits slab per chunk
    memory_reserve_bytes: int = 8 << 30
    remat_group_size: int = 1                # recomputed layers keep their input only at every G-th layer; the
                                             # others' inputs are rebuilt group by group in the backward pass
    mlp_chunk_rows: int = 0                  # > 0: the MLP runs in tiles of this many token rows and its [T, 2F]
                                             # intermediate is never held whole (rebuilt per tile in backward)
    moba_implementation: str = "grouped"     # "grouped": rows gathered by selected block, cost ~ top_k * block;
                                             # "lists": one masked flash pass over the union of a tile's selections
    moba_dense_shortcut: bool = True         # batches whose longest document has at most top_k blocks (a host-side
                                             # fact the batch carries) run the dense kernel: the same function


class LayerwiseEngine:
    """Gradient producer (see ``training.steps.GradientProducer``) running on the CUDA kernels."""

    def __init__(self, cfg: ModelConfig, provider, options: EngineOptions | None = None):
        _lib.require_gpu_lib()
        self.cfg = cfg
        self.provider = provider
        self.options = options or EngineOptions()
        self.launches = 0
        self.kept_layers = 0
        self.train_base = True                   # False: base weights frozen, no gradient buffers (LoRA)
        self.marks: list[tuple[str, torch.cuda.Event]] | None = None   # phase boundaries (benchmarks/step_phases.py)
        self._inv_freq: torch.Tensor | None = None
        import os

        overlap = self.options.overlap_wgrad and os.environ.get("CTB_OVERLAP_WGRAD", "1") != "0"
        self._wgrad_stream = torch.cuda.Stream() if overlap else None

    # ------------------------------------------------------------------ helpers
    def _views(self, unit: Unit, base: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
        return {seg.name: unit.view(seg.name, of=base) for seg in unit.layout.segments}

    def _count(self, n: int = 1) -> None:
        self.launches += n

    def _mark(self, name: str) -> None:
        if self.marks is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self.marks.append((name, ev))

    def select_tokens(self, t: torch.Tensor) -> torch.Tensor:
        """The part of a ``[B, S, ...]`` batch tensor this rank computes on (everything, unless the
        sequence is split over ranks)."""
        return t

    def _local_seq(self, s: int) -> int:
        """Tokens of a row of ``s`` tokens that this rank computes on."""
        return s

    def _project(self, li: int, name: str, x: torch.Tensor, w: dict[str, torch.Tensor]) -> torch.Tensor:
        """Projection ``name`` ("qkv" | "o" | "gu" | "down") of layer ``li``: ``x @ W^T (+ bias)``."""
        self._count()
        return gemm(x, w[name + "_w"], bias=w.get(name + "_b"))

    def _project_backward(self, li: int, name: str, dy: torch.Tensor, x: torch.Tensor, w: dict[str, torch.Tensor],
                          g: dict[str, torch.Tensor], accumulate: bool) -> torch.Tensor:
        """Input gradient of projection ``name``; its weight (and bias) gradients go into ``g``."""
        dx = gemm(dy, w[name + "_w"], b_mn=True)
        self._count()
        self._wgrad(dy, x, g[name + "_w"], accumulate)
        if name + "_b" in w:
            self._bias_grad(dy, g[name + "_b"], accumulate)
        return dx

    def _wgrad(self, dy: torch.Tensor, x: torch.Tensor, gview: torch.Tensor | None, accumulate: bool) -> None:
        """Weight gradient ``dy^T x`` (skipped when the weight is frozen: ``gview`` is None).  With
        ``overlap_wgrad`` it is issued on a second stream: nothing in the layer waits for it, so the
        partly filled last wave of one persistent GEMM is filled by the first CTAs of the next kernel
        instead of leaving SMs idle."""
        if gview is None:
            return
        side = self._wgrad_stream
        if side is None:
            gemm(dy, x, a_mn=True, b_mn=True, out=gview, accumulate=accumulate)
        else:
            ev = torch.cuda.Event()
            ev.record()
            side.wait_event(ev)
            with torch.cuda.stream(side):
                gemm(dy, x, a_mn=True, b_mn=True, out=gview, accumulate=accumulate)
            dy.record_stream(side)
            x.record_stream(side)
        self._count()

    def _join_wgrads(self) -> None:
        if self._wgrad_stream is not None:
            torch.cuda.current_stream().wait_stream(self._wgrad_stream)

    def _bias_grad(self, dy: torch.Tensor, gview: torch.Tensor | None, accumulate: bool) -> None:
        if gview is None:
            return
        s = dy.float().sum(0)
        if accumulate:
            gview.add_(s.to(gview.dtype))
        else:
            gview.copy_(s.to(gview.dtype))
        self._count(2)

    # ------------------------------------------------------------------ attention (dense or MoBA)
    def _uses_moba(self, li: int, seq: int, longest: int | None = None) -> bool:
        ao = self.options.attention_options
        if ao is None or not ao.applies_to_layer(li, self.cfg.num_hidden_layers, self.options.optimizer_step):
            return False
        # a document of at most top_k blocks leaves the router nothing to drop (blocks are counted from
        # the document's first token, and the current block is one of the top_k): exactly dense
        span = seq if longest is None or not self.options.moba_dense_shortcut else min(seq, max(int(longest), 1))
        return ao.moba_top_k * min(ao.moba_block_size, seq) < span

    def _attention_forward(self, q, k, v, ctx: dict, li: int):
        """Returns (O, LSE, routing); routing is None for dense layers."""
        if not self._uses_moba(li, ctx["seq"], ctx.get("longest")):
            o, lse = attn_ops.flash_attention_forward(q, k, v, ctx["meta"])
            return o, lse, None
        from ..ops import moba as moba_ops

        ao = self.options.attention_options
        block = min(ao.moba_block_size, ctx["seq"])
        if self.options.moba_implementation == "grouped" and block % 128 == 0 and ao.moba_top_k >= 2:
            routing = moba_ops.build_groups(q, k, ctx["meta"], block, ao.moba_top_k)
            o, lse = moba_ops.moba_grouped_forward(q, k, v, ctx["meta"], routing)
            self._count(11)
            return o, lse, routing
        routing = moba_ops.build_routing(q, k, ctx["meta"], block, ao.moba_top_k)
        o, lse = moba_ops.moba_forward(q, k, v, ctx["meta"], routing)
        self._count(40)
        return o, lse, routing

    def _attention_backward(self, q, k, v, o, do, lse, routing, ctx: dict, dq, dk, dv) -> None:
        if routing is None:
            attn_ops.flash_attention_backward(q, k, v, o, do, lse, ctx["meta"], dq=dq, dk=dk, dv=dv)
        else:
            from ..ops import moba as moba_ops

            if isinstance(routing, moba_ops.MobaGroups):
                moba_ops.moba_grouped_backward(q, k, v, o, do, lse, ctx["meta"], routing, dq=dq, dk=dk, dv=dv)
            else:
                moba_ops.moba_backward(q, k, v, o, do, lse, ctx["meta"], routing, dq=dq, dk=dk, dv=dv)

    def _embed(self, local_ids: torch.Tensor, first_layer: str) -> torch.Tensor:
        """Token embeddings of this rank's tokens.  A sharded provider fetches just the rows it
        needs from the shards that own them; otherwise the table is acquired like any unit."""
        prov = self.provider
        rows = prov.embedding_rows(local_ids) if hasattr(prov, "embedding_rows") else None
        if rows is not None:
            prov.prefetch(first_layer)
        else:
            embed = prov.acquire("embed", prefetch=first_layer)
            rows = ew.embedding_gather(local_ids, embed.view("embed"))
            prov.release("embed")
        self._count()
        return rows

    def _norm_grad(self, g: dict[str, torch.Tensor], name: str) -> torch.Tensor | None:
        return g[name] if self.options.train_norm else None

    # ------------------------------------------------------------------ layer forward
    def _layer_forward(self, w: dict[str, torch.Tensor], resid: torch.Tensor, branch: torch.Tensor | None, ctx: dict,
                       li: int, save: str | None) -> tuple[torch.Tensor, torch.Tensor, dict | None]:
        cfg = self.cfg
        t = resid.shape[0]
        qw, kvw, d_head = cfg.query_width, cfg.key_value_width, cfg.head_dim
        n1, rstd1, x = ew.rmsnorm_forward(resid, w["ln1"], cfg.rms_norm_eps, residual=branch)
        qkv = self._project(li, "qkv", n1, w)
        ew.rope_inplace(qkv, ctx["cos"], ctx["sin"], cfg.num_attention_heads + cfg.num_key_value_heads, d_head,
                        cfg.rotary_dim, cfg.rope_style)
        b, s = ctx["batch"], ctx["seq"]
        q = qkv[:, :qw].view(b, s, cfg.num_attention_heads, d_head)
        k = qkv[:, qw:qw + kvw].view(b, s, cfg.num_key_value_heads, d_head)
        v = qkv[:, qw + kvw:].view(b, s, cfg.num_key_value_heads, d_head)
        o, lse, routing = self._attention_forward(q, k, v, ctx, li)
        attn_out = self._project(li, "o", o.view(t, qw), w)
        n2, rstd2, h = ew.rmsnorm_forward(x, w["ln2"], cfg.rms_norm_eps, residual=attn_out)
        chunk = self.options.mlp_chunk_rows
        if chunk > 0 and t > chunk:
            # tiled MLP (src/causal_trainer/modeling/architecture.py:509-534): bounded [chunk, 2F] intermediates
            gu = act = None
            mlp = torch.empty((t, cfg.hidden_size), dtype=n2.dtype, device=n2.device)
            for r0 in range(0, t, chunk):
                gu_c = self._project(li, "gu", n2[r0:r0 + chunk], w)
                gemm(ew.swiglu_forward(gu_c), w["down_w"], bias=w.get("down_b"), out=mlp[r0:r0 + chunk])
                self._count(2)
        else:
            gu = self._project(li, "gu", n2, w)
            act = ew.swiglu_forward(gu)
            mlp = self._project(li, "down", act, w)
        self._count(6)
        saved = None
        if save == "all":      # transient: consumed by the backward pass that follows at once
            saved = dict(x=x, n1=n1, rstd1=rstd1, qkv=qkv, o=o, lse=lse, h=h, n2=n2, rstd2=rstd2, gu=gu, act=act,
                         routing=routing)
        elif save == "keep":   # kept from the forward pass: the three cheap tensors are rebuilt in backward
            saved = dict(x=x, rstd1=rstd1, qkv=qkv, o=o, lse=lse, h=h, rstd2=rstd2, gu=gu, routing=routing)
        return h, mlp, saved

    # ------------------------------------------------------------------ layer backward
    def _layer_backward(self, w: dict[str, torch.Tensor], g: dict[str, torch.Tensor], sv: dict, dout: torch.Tensor,
                        ctx: dict, accumulate: bool, li: int = 0) -> torch.Tensor:
        """``dout`` is the gradient of the layer output (h + mlp); returns the gradient of its input x."""
        cfg = self.cfg
        t = dout.shape[0]
        qw, kvw, d_head = cfg.query_width, cfg.key_value_width, cfg.head_dim
        b, s = ctx["batch"], ctx["seq"]
        if "act" not in sv:
            # kept activations: the memory-bound intermediates are cheaper to rebuild than to hold
            sv = dict(sv)
            sv["act"] = ew.swiglu_forward(sv["gu"]) if sv["gu"] is not None else None
            sv["n2"] = ew.rmsnorm_forward(sv["h"], w["ln2"], cfg.rms_norm_eps)[0]
            sv["n1"] = ew.rmsnorm_forward(sv["x"], w["ln1"], cfg.rms_norm_eps)[0]
            self._count(3)
        # MLP branch
        if sv["gu"] is None:
            # tiled MLP: every tile rebuilds its gate/up product, then runs the usual backward on it
            chunk = self.options.mlp_chunk_rows
            dn2 = torch.empty_like(sv["n2"])
            for r0 in range(0, t, chunk):
                rows = slice(r0, r0 + chunk)
                later = accumulate or r0 > 0
                gu_c = self._project(li, "gu", sv["n2"][rows], w)
                dact = self._project_backward(li, "down", dout[rows], ew.swiglu_forward(gu_c), w, g, later)
                dgu = ew.swiglu_backward(gu_c, dact)
                dn2[rows] = self._project_backward(li, "gu", dgu, sv["n2"][rows], w, g, later)
                del gu_c, dact, dgu
        else:
            dact = self._project_backward(li, "down", dout, sv["act"], w, g, accumulate)
            dgu = ew.swiglu_backward(sv["gu"], dact)
            del dact
            dn2 = self._project_backward(li, "gu", dgu, sv["n2"], w, g, accumulate)
            del dgu
        dh, _ = ew.rmsnorm_backward(dn2, sv["h"], w["ln2"], sv["rstd2"], dres=dout, dw_out=self._norm_grad(g, "ln2"),
                                    dw_accumulate=accumulate)
        del dn2
        # attention branch: dh is the gradient of h = x + attn_out
        do = self._project_backward(li, "o", dh, sv["o"].view(t, qw), w, g, accumulate)
        qkv = sv["qkv"]
        q = qkv[:, :qw].view(b, s, cfg.num_attention_heads, d_head)
        k = qkv[:, qw:qw + kvw].view(b, s, cfg.num_key_value_heads, d_head)
        v = qkv[:, qw + kvw:].view(b, s, cfg.num_key_value_heads, d_head)
        dqkv = torch.empty_like(qkv)
        dq = dqkv[:, :qw].view(b, s, cfg.num_attention_heads, d_head)
        dk = dqkv[:, qw:qw + kvw].view(b, s, cfg.num_key_value_heads, d_head)
        dv = dqkv[:, qw + kvw:].view(b, s, cfg.num_key_value_heads, d_head)
        self._attention_backward(q, k, v, sv["o"], do.view(b, s, cfg.num_attention_heads, d_head), sv["lse"],
                                 sv.get("routing"), ctx, dq, dk, dv)
        ew.rope_inplace(dqkv, ctx["cos"], ctx["sin"], cfg.num_attention_heads + cfg.num_key_value_heads, d_head,
                        cfg.rotary_dim, cfg.rope_style, inverse=True)
        dn1 = self._project_backward(li, "qkv", dqkv, sv["n1"], w, g, accumulate)
        dx, _ = ew.rmsnorm_backward(dn1, sv["x"], w["ln1"], sv["rstd1"], dres=dh, dw_out=self._norm_grad(g, "ln1"),
                                    dw_accumulate=accumulate)
        self._count(8)
        return dx

    # ------------------------------------------------------------------ activation policy
    def _layers_to_keep(self, tokens: int) -> int:
        """How many layers keep their activations instead of being recomputed in backward.

        ``remat="full"`` recomputes every layer (the reference's ``nothing_saveable``), ``"none"``
        keeps all, ``"auto"`` keeps as many as fit in the memory that is free right now, after a
        reserve for the backward working set: on a 180 GB part an 8B model usually keeps all.
        """
        cfg, mode = self.cfg, self.options.remat
        if mode == "full":
            return 0
        if mode == "none":
            return cfg.num_hidden_layers
        from .memory_plan import backward_working_set_bytes, layer_activation_bytes

        per_layer = layer_activation_bytes(cfg, tokens)
        free, _ = torch.cuda.mem_get_info()
        cached = torch.cuda.memory_reserved() - torch.cuda.memory_allocated()
        working_set = backward_working_set_bytes(cfg, tokens, self.options.cut_chunk_rows)
        budget = free + cached - working_set - self.options.memory_reserve_bytes
        return max(0, min(cfg.num_hidden_layers, int(budget // per_layer)))

    # ------------------------------------------------------------------ step context
    def _context(self, batch: dict[str, torch.Tensor]) -> dict:
        cfg = self.cfg
        ids = batch["input_ids"]
        mask = batch["attention_mask"]
        end = batch.get("attention_end")
        seg, restart_pos, meta = attn_ops.attention_metadata(mask, batch.get("segment_ids"), end)
        pos = batch.get("position_ids")
        if pos is None:
            pos = restart_pos
        if self._inv_freq is None or self._inv_freq.device != ids.device:
            self._inv_freq = ew.inverse_frequencies(cfg.rotary_dim, cfg.rope_theta, device=ids.device)
        cos, sin = ew.rope_table(pos, self._inv_freq)
        self._count(1)   # segments, positions and block summaries: one launch per micro-batch
        return dict(batch=ids.shape[0], seq=ids.shape[1], cos=cos, sin=sin, meta=meta, seg=seg,
                    longest=batch.get("longest_document"))

    # ------------------------------------------------------------------ forward only
    @torch.no_grad()
    def forward_hidden(self, batch: dict[str, torch.Tensor]) -> torch.Tensor:
        """Final-norm hidden states [B*S, d] (evaluation / tests)."""
        ctx = self._context(batch)
        cfg = self.cfg
        resid = self._embed(self.select_tokens(batch["input_ids"]), "layer.0")
        branch = None
        for li in range(cfg.num_hidden_layers):
            unit = self.provider.acquire(f"layer.{li}", prefetch=f"layer.{li + 1}" if li + 1 < cfg.num_hidden_layers else "final")
            resid, branch, _ = self._layer_forward(self._views(unit), resid, branch, ctx, li, save=None)
            self.provider.release(f"layer.{li}")
        final = self.provider.acquire("final")
        y, _, _ = ew.rmsnorm_forward(resid, final.view("norm"), cfg.rms_norm_eps, residual=branch)
        self.provider.release("final")
        return y

    # ------------------------------------------------------------------ gradient producer
    @torch.no_grad()
    def __call__(self, batch: dict[str, torch.Tensor], grad_scale: float, first: bool, last: bool = True):
        cfg = self.cfg
        prov = self.provider
        accumulate = not first
        self._mark("begin")
        ctx = self._context(batch)
        nl = cfg.num_hidden_layers
        # ---------------- forward: keep (resid, branch) per layer ----------------
        local_ids = self.select_tokens(batch["input_ids"])
        resid = self._embed(local_ids, "layer.0")
        self._mark("embedding")
        branch = None
        inputs: list[tuple[torch.Tensor, torch.Tensor | None]] = []
        kept: list[dict | None] = []
        keep_layers = self._layers_to_keep(resid.shape[0])
        self.kept_layers = keep_layers
        group = max(1, self.options.remat_group_size)
        for li in range(nl):
            unit = prov.acquire(f"layer.{li}", prefetch=f"layer.{li + 1}" if li + 1 < nl else "final")
            # the last layers are kept first: their activations are consumed soonest
            keep = li >= nl - keep_layers
            # a recomputed layer keeps its input; with remat groups only the first layer of a group does
            inputs.append((resid, branch) if (not keep and li % group == 0) else None)
            resid, branch, sv = self._layer_forward(self._views(unit), resid, branch, ctx, li,
                                                    save="keep" if keep else None)
            kept.append(sv)
            prov.release(f"layer.{li}")
        self._mark("layers forward")
        # ---------------- head: final norm + cut cross-entropy ----------------
        final = prov.acquire("final", prefetch=f"layer.{nl - 1}")
        fw = self._views(final)
        fg = self._views(final, prov.grad_buffer("final")) if self.train_base else dict.fromkeys(fw)
        y, rstd_f, xf = ew.rmsnorm_forward(resid, fw["norm"], cfg.rms_norm_eps, residual=branch)
        targets, weights = losses.aligned_targets_and_weights(batch)
        targets, weights = self.select_tokens(targets).reshape(-1), self.select_tokens(weights).reshape(-1)
        train_head = self.options.train_lm_head and self.train_base
        # Active-row compaction: with sparse supervision (assistant-only loss, MaskGIT targets) only
        # the rows that carry weight go through the LM head; their gradients are scattered back.
        # (src/causal_trainer/kernels/cut_cross_entropy.py:673-694; stable order, so results do not
        # depend on it.)
        full_rows = y.shape[0]
        active = None
        # (only batches that carry explicit weights can be sparse; asking costs one read back, which a
        # plain next-token batch is spared)
        if self.options.compact_loss_rows and ("loss_weights" in batch or "prediction_weights" in batch):
            idx_p, n_active_dev, n_active = ew.active_rows(weights)     # whole 128-row tiles, row 0 repeated as padding
            if n_active < 0.9 * full_rows:
                active = idx_p
                y_all = y
                y = ew.gather_rows(y_all, idx_p)
                targets = targets.index_select(0, idx_p.long())
                weights = weights.index_select(0, idx_p.long())
                weights[n_active:] = 0                                   # padding slots carry no loss
                self._count(5)
        if self.options.loss_backend == "logits":
            nll, wsum, dy, _ = ce.logits_ce_forward_backward(
                y, fw["lm_head"], targets, weights, grad_scale, chunk_rows=self.options.cut_chunk_rows,
                need_dhead=train_head, dhead_out=fg["lm_head"] if train_head else None, dhead_accumulate=accumulate)
        else:
            nll, wsum, lse, coef = ce.cut_ce_forward(y, fw["lm_head"], targets, weights, grad_scale)
            dy, _ = ce.cut_ce_backward(y, fw["lm_head"], targets, lse, coef, chunk_rows=self.options.cut_chunk_rows,
                                       need_dhead=train_head, dhead_out=fg["lm_head"] if train_head else None,
                                       dhead_accumulate=accumulate)
        self._count(4 + 3 * ((y.shape[0] + self.options.cut_chunk_rows - 1) // self.options.cut_chunk_rows))
        if active is not None:
            dy, y = ew.scatter_rows(dy, active, n_active_dev, full_rows), y_all     # rows without loss get zero gradient
        dout, _ = ew.rmsnorm_backward(dy, xf, fw["norm"], rstd_f, dw_out=self._norm_grad(fg, "norm"),
                                      dw_accumulate=accumulate)
        del y, dy, xf
        prov.release("final")
        prov.grads_ready("final", last)
        self._mark("head forward+backward")
        # ---------------- backward: recompute + hand-written layer backward ----------------
        for li in reversed(range(nl)):
            saved = kept.pop()
            if saved is None and inputs[li] is None:
                # remat group (src/causal_trainer/modeling/architecture.py:777-786): rebuild the inputs of
                # the group's later layers from the one input the forward pass kept
                first = li - li % group
                x = inputs[first]
                for j in range(first, li):
                    uj = prov.acquire(f"layer.{j}")
                    r, br, _ = self._layer_forward(self._views(uj), x[0], x[1], ctx, j, save=None)
                    prov.release(f"layer.{j}")
                    x = inputs[j + 1] = (r, br)
            # the embedding table is not read in the backward pass: nothing to prefetch for layer 0
            unit = prov.acquire(f"layer.{li}", prefetch=f"layer.{li - 1}" if li > 0 else None)
            w = self._views(unit)
            g = self._views(unit, prov.grad_buffer(f"layer.{li}")) if self.train_base else dict.fromkeys(w)
            layer_in = inputs.pop()
            if saved is None:
                _, _, saved = self._layer_forward(w, layer_in[0], layer_in[1], ctx, li, save="all")
            dout = self._layer_backward(w, g, saved, dout, ctx, accumulate, li)
            del saved, layer_in
            self._join_wgrads()
            prov.release(f"layer.{li}")
            prov.grads_ready(f"layer.{li}", last)
        self._mark("layers backward")
        # ---------------- embedding ----------------
        if self.options.train_embed and self.train_base:
            lay = embed_layout(cfg)
            seg = lay.segment("embed")
            gbuf = prov.grad_buffer("embed")[seg.offset:seg.offset + seg.numel].view(seg.shape)
            if first:
                gbuf.zero_()
            ew.embedding_backward(local_ids, dout, gbuf, cfg.pad_token_id)
            self._count(5)
            prov.grads_ready("embed", last)
        self._mark("embedding backward")
        return nll, wsum
