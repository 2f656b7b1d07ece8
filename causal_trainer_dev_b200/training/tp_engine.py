"""Tensor-parallel layerwise engine: the explicit schedule of ``training.engine`` with the
activations sharded by token rows over the tp ranks and the collectives fused into the GEMMs.

Per layer (forward):  RMSNorm(own rows) -> all-gather -> QKV GEMM (local heads) -> RoPE ->
attention (local heads, all tokens) -> O GEMM -> reduce-scatter -> RMSNorm(own rows) -> all-gather
-> gate/up GEMM (local FFN columns) -> SwiGLU -> down GEMM -> reduce-scatter.  The backward pass
mirrors it: every dgrad of a column-parallel weight is a GEMM -> reduce-scatter, every dgrad of a
row-parallel weight reads an all-gathered gradient, and the weight gradients read the re-gathered
normalised activations.  The LM head is vocabulary-parallel (cut cross-entropy statistics are
combined across ranks in one kernel) and so is the embedding.

The reference reaches the same partitioning through GSPMD shardings and, for long contexts,
``shard_map`` bodies with explicit ``all_gather`` / ``psum_scatter`` over ``tp``
(src/causal_trainer/distributed/runtime.py:334-338; src/causal_trainer/modeling/token_tiling.py:
59-64,120-128,241-246; src/causal_trainer/kernels/cut_cross_entropy.py:474-521).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.config import ModelConfig
from ..models.params import embed_layout
from ..ops import cross_entropy as ce
from ..ops import elementwise as ew
from ..ops.gemm import gemm
from ..parallel.tp import Gathered, TpContext, kv_replicas, tp_local_config
from . import losses
from .engine import EngineOptions, LayerwiseEngine


class TpLayerwiseEngine(LayerwiseEngine):
    """Gradient producer for one tensor-parallel rank; ``provider`` hands out tp-local units."""

    def __init__(self, full_cfg: ModelConfig, tp_group, provider, options: EngineOptions | None = None,
                 fused: bool = True):
        self.full_cfg = full_cfg
        self.tp_group = tp_group
        self.tp_world = dist.get_world_size(tp_group)
        self.tp_rank = dist.get_rank(tp_group)
        self.fused = fused
        self._contexts: dict[int, TpContext] = {}
        super().__init__(tp_local_config(full_cfg, self.tp_world), provider, options)
        self._wgrad_stream = None      # weight gradients read ring buffers that later all-gathers reuse
        # fewer key/value heads than ranks: the ranks that share a head sum its weight gradients
        self.kv_rep = kv_replicas(full_cfg, self.tp_world)
        self.kv_group = None
        if self.kv_rep > 1:
            ranks = dist.get_process_group_ranks(tp_group)
            first = self.tp_rank // self.kv_rep * self.kv_rep
            self.kv_group = dist.new_group(ranks[first:first + self.kv_rep], use_local_synchronization=True)

    # ------------------------------------------------------------------ context
    def _tp(self, rows: int) -> TpContext:
        ctx = self._contexts.get(rows)
        if ctx is None:
            ctx = TpContext(self.tp_group, torch.device("cuda", torch.cuda.current_device()), rows,
                            self.cfg.hidden_size, fused=self.fused)
            self._contexts[rows] = ctx
        return ctx

    def _context(self, batch):
        ctx = super()._context(batch)
        ctx["tp"] = self._tp(ctx["batch"] * self._local_seq(ctx["seq"]))
        return ctx

    def _layers_to_keep(self, tokens: int) -> int:
        # `tokens` counts this rank's rows; the kept tensors are mostly full-row, local-width
        return super()._layers_to_keep(tokens * self.tp_world)

    # ------------------------------------------------------------------ layer forward
    def _layer_forward(self, w, resid, branch, ctx, li, save):
        cfg = self.cfg
        tp: TpContext = ctx["tp"]
        t = tp.rows
        qw, kvw, d_head = cfg.query_width, cfg.key_value_width, cfg.head_dim
        g1 = tp.next_slot()
        _, rstd1, x = ew.rmsnorm_forward(resid, w["ln1"], cfg.rms_norm_eps, residual=branch, out=g1.mine)
        n1 = tp.all_gather(g1)
        qkv = gemm(n1, w["qkv_w"], bias=w.get("qkv_b"))
        ew.rope_inplace(qkv, ctx["cos"], ctx["sin"], cfg.num_attention_heads + cfg.num_key_value_heads, d_head,
                        cfg.rotary_dim, cfg.rope_style)
        b, s = ctx["batch"], ctx["seq"]
        q = qkv[:, :qw].view(b, s, cfg.num_attention_heads, d_head)
        k = qkv[:, qw:qw + kvw].view(b, s, cfg.num_key_value_heads, d_head)
        v = qkv[:, qw + kvw:].view(b, s, cfg.num_key_value_heads, d_head)
        o, lse, routing = self._attention_forward(q, k, v, ctx, li)
        attn_out = tp.gemm_reduce_scatter(o.view(t, qw), w["o_w"])
        g2 = tp.next_slot()
        _, rstd2, h = ew.rmsnorm_forward(x, w["ln2"], cfg.rms_norm_eps, residual=attn_out, out=g2.mine)
        n2 = tp.all_gather(g2)
        gu = gemm(n2, w["gu_w"])
        act = ew.swiglu_forward(gu)
        mlp = tp.gemm_reduce_scatter(act, w["down_w"])
        self._count(16)
        saved = None
        if save == "all":
            saved = dict(x=x, rstd1=rstd1, qkv=qkv, o=o, lse=lse, h=h, rstd2=rstd2, gu=gu, act=act, routing=routing)
        elif save == "keep":
            saved = dict(x=x, rstd1=rstd1, qkv=qkv, o=o, lse=lse, h=h, rstd2=rstd2, gu=gu, routing=routing)
        return h, mlp, saved

    # ------------------------------------------------------------------ layer backward
    def _regather_norm(self, tp: TpContext, x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
        g = tp.next_slot()
        ew.rmsnorm_forward(x, scale, self.cfg.rms_norm_eps, out=g.mine)
        return tp.all_gather(g)

    def _layer_backward(self, w, g, sv, dout: Gathered, ctx, accumulate) -> Gathered:
        """``dout.mine`` holds this rank's rows of the gradient of the layer output; returns the
        (not yet gathered) gradient of the layer input in the same form."""
        cfg = self.cfg
        tp: TpContext = ctx["tp"]
        t = tp.rows
        qw, kvw, d_head = cfg.query_width, cfg.key_value_width, cfg.head_dim
        b, s = ctx["batch"], ctx["seq"]
        act = sv["act"] if "act" in sv else ew.swiglu_forward(sv["gu"])
        # MLP branch
        dout_full = tp.all_gather(dout)
        dact = gemm(dout_full, w["down_w"], b_mn=True)
        self._wgrad(dout_full, act, g["down_w"], accumulate)
        dgu = ew.swiglu_backward(sv["gu"], dact)
        del dact, act
        n2 = self._regather_norm(tp, sv["h"], w["ln2"])
        dn2 = tp.gemm_reduce_scatter(dgu, w["gu_w"], b_mn=True)
        self._wgrad(dgu, n2, g["gu_w"], accumulate)
        del dgu
        gh = tp.next_slot()
        ew.rmsnorm_backward(dn2, sv["h"], w["ln2"], sv["rstd2"], dres=dout.mine, dw_out=g["ln2"],
                            dw_accumulate=accumulate, dx_out=gh.mine)
        # attention branch
        dh_full = tp.all_gather(gh)
        do = gemm(dh_full, w["o_w"], b_mn=True)
        self._wgrad(dh_full, sv["o"].view(t, qw), g["o_w"], accumulate)
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
        n1 = self._regather_norm(tp, sv["x"], w["ln1"])
        dn1 = tp.gemm_reduce_scatter(dqkv, w["qkv_w"], b_mn=True)
        self._wgrad(dqkv, n1, g["qkv_w"], accumulate)
        if "qkv_b" in w:
            self._bias_grad(dqkv, g["qkv_b"], accumulate)
        gx = tp.next_slot()
        ew.rmsnorm_backward(dn1, sv["x"], w["ln1"], sv["rstd1"], dres=gh.mine, dw_out=g["ln1"],
                            dw_accumulate=accumulate, dx_out=gx.mine)
        self._count(24)
        return gx

    # ------------------------------------------------------------------ forward only
    @torch.no_grad()
    def forward_hidden(self, batch):
        """Final-norm hidden states of this rank's rows ``[B*S/tp, d]``."""
        ctx = self._context(batch)
        cfg, tp = self.cfg, ctx["tp"]
        embed = self.provider.acquire("embed")
        resid = tp.embed_lookup(self.select_tokens(batch["input_ids"]), embed.view("embed"), self.full_cfg.vocab_size)
        self.provider.release("embed")
        branch = None
        for li in range(cfg.num_hidden_layers):
            nxt = f"layer.{li + 1}" if li + 1 < cfg.num_hidden_layers else "final"
            unit = self.provider.acquire(f"layer.{li}", prefetch=nxt)
            resid, branch, _ = self._layer_forward(self._views(unit), resid, branch, ctx, li, save=None)
            self.provider.release(f"layer.{li}")
        final = self.provider.acquire("final")
        y, _, _ = ew.rmsnorm_forward(resid, final.view("norm"), cfg.rms_norm_eps, residual=branch)
        self.provider.release("final")
        return y

    # ------------------------------------------------------------------ gradient producer
    @torch.no_grad()
    def __call__(self, batch, grad_scale: float, first: bool, last: bool = True):
        cfg, full = self.cfg, self.full_cfg
        prov = self.provider
        accumulate = not first
        ctx = self._context(batch)
        tp: TpContext = ctx["tp"]
        nl = cfg.num_hidden_layers
        vocab_local = cfg.vocab_size
        vocab_lo = self.tp_rank * vocab_local
        # ---------------- forward ----------------
        embed = prov.acquire("embed", prefetch="layer.0")
        local_ids = self.select_tokens(batch["input_ids"])
        resid = tp.embed_lookup(local_ids, embed.view("embed"), full.vocab_size)
        self._count(3)
        prov.release("embed")
        branch = None
        inputs, kept = [], []
        keep_layers = self._layers_to_keep(resid.shape[0])
        self.kept_layers = keep_layers
        for li in range(nl):
            unit = prov.acquire(f"layer.{li}", prefetch=f"layer.{li + 1}" if li + 1 < nl else "final")
            keep = li >= nl - keep_layers
            inputs.append(None if keep else (resid, branch))
            resid, branch, sv = self._layer_forward(self._views(unit), resid, branch, ctx, li,
                                                    save="keep" if keep else None)
            kept.append(sv)
            prov.release(f"layer.{li}")
        # ---------------- head: final norm + vocabulary-parallel cut cross-entropy ----------------
        final = prov.acquire("final", prefetch=f"layer.{nl - 1}")
        fw = self._views(final)
        fg = self._views(final, prov.grad_buffer("final"))
        gy = tp.next_slot()
        _, rstd_f, xf = ew.rmsnorm_forward(resid, fw["norm"], cfg.rms_norm_eps, residual=branch, out=gy.mine)
        y = tp.all_gather(gy)
        targets, weights = losses.aligned_targets_and_weights(batch)
        targets, weights = self.select_tokens(targets).reshape(-1), self.select_tokens(weights).reshape(-1)
        local_t = targets.to(torch.int32) - vocab_lo
        local_t = torch.where((local_t >= 0) & (local_t < vocab_local), local_t, torch.full_like(local_t, -1))
        nll, wsum, lse, coef = ce.cut_ce_forward(y, fw["lm_head"], local_t, weights, grad_scale, exchange=tp)
        train_head = self.options.train_lm_head
        if tp.fused:
            push = tp.begin_push()
            ce.cut_ce_backward(y, fw["lm_head"], local_t, lse, coef, chunk_rows=self.options.cut_chunk_rows,
                               need_dhead=train_head, dhead_out=fg["lm_head"] if train_head else None,
                               dhead_accumulate=accumulate, push=push)
            dy = tp.finish_push(push)
        else:
            tp.wait_gathered(gy)
            dy_partial, _ = ce.cut_ce_backward(y, fw["lm_head"], local_t, lse, coef,
                                               chunk_rows=self.options.cut_chunk_rows, need_dhead=train_head,
                                               dhead_out=fg["lm_head"] if train_head else None,
                                               dhead_accumulate=accumulate)
            dy = torch.empty((tp.rows_per_rank, cfg.hidden_size), dtype=torch.bfloat16, device=dy_partial.device)
            dist.reduce_scatter_tensor(dy, dy_partial, group=self.tp_group)
        self._count(8 + 3 * ((y.shape[0] + self.options.cut_chunk_rows - 1) // self.options.cut_chunk_rows))
        dout = tp.next_slot()
        ew.rmsnorm_backward(dy, xf, fw["norm"], rstd_f, dw_out=fg["norm"], dw_accumulate=accumulate, dx_out=dout.mine)
        tp.all_reduce_replicated([fg["norm"]])
        del y, dy, xf
        prov.release("final")
        prov.grads_ready("final", last)
        # ---------------- backward ----------------
        for li in reversed(range(nl)):
            unit = prov.acquire(f"layer.{li}", prefetch=f"layer.{li - 1}" if li > 0 else "embed")
            w = self._views(unit)
            gbuf = prov.grad_buffer(f"layer.{li}")
            g = self._views(unit, gbuf)
            layer_in = inputs.pop()
            saved = kept.pop()
            if saved is None:
                _, _, saved = self._layer_forward(w, layer_in[0], layer_in[1], ctx, li, save="all")
            dout = self._layer_backward(w, g, saved, dout, ctx, accumulate)
            del saved, layer_in
            # norm scales are replicated over tp and saw only this rank's rows: sum the pair at once
            ln = unit.layout.segment("ln1")
            ln2 = unit.layout.segment("ln2")
            tp.all_reduce_replicated([gbuf[ln.offset:ln2.offset + ln2.numel]])
            if self.kv_group is not None:
                ql = cfg.query_width
                dist.all_reduce(g["qkv_w"][ql:], group=self.kv_group)
                if "qkv_b" in g:
                    dist.all_reduce(g["qkv_b"][ql:], group=self.kv_group)
            prov.release(f"layer.{li}")
            prov.grads_ready(f"layer.{li}", last)
        # ---------------- embedding (vocabulary-parallel) ----------------
        if self.options.train_embed:
            lay = embed_layout(cfg)
            seg = lay.segment("embed")
            gtab = prov.grad_buffer("embed")[seg.offset:seg.offset + seg.numel].view(seg.shape)
            if first:
                gtab.zero_()
            dx_full = tp.all_gather(dout)
            tp.wait_gathered(dout)
            ew.embedding_backward(local_ids, dx_full, gtab, full.pad_token_id, vocab_lo)
            self._count(8)
            prov.grads_ready("embed", last)
        return nll, wsum
