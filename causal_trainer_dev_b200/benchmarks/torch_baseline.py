"""Library baseline of the headline benchmark: the same Llama-shape training step written with
stock libraries only — cuBLAS matmuls, library flash attention, ``F.cross_entropy`` in row chunks,
autograd, fused ``torch.optim.AdamW`` and, on several GPUs, ``fully_shard`` (FSDP2) over NCCL.
None of this repository's kernels run here.  It exists to give the product path a same-box,
same-shape number to stand against (``bench.py --impl torch``).

Attention does the same work as the product path: the packed documents are attended separately
(``flash_attn_varlen_func`` with the documents' cumulative lengths) when the ``flash_attn`` package
is importable; otherwise ``scaled_dot_product_attention`` with a plain causal mask over the whole
row, which is more attention FLOPs for the baseline (``attention`` in the result says which ran).
"""
from __future__ import annotations


import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class Block(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        d, q, kv, f = cfg.hidden_size, cfg.query_width, cfg.key_value_width, cfg.intermediate_size
        self.cfg = cfg
        self.ln1 = nn.RMSNorm(d, eps=cfg.rms_norm_eps)
        self.ln2 = nn.RMSNorm(d, eps=cfg.rms_norm_eps)
        self.qkv = nn.Linear(d, q + 2 * kv, bias=cfg.attention_bias)
        self.o = nn.Linear(q, d, bias=False)
        self.gu = nn.Linear(d, 2 * f, bias=False)
        self.down = nn.Linear(f, d, bias=False)

    def forward(self, h, cos, sin, varlen=None):
        cfg = self.cfg
        b, s, _ = h.shape
        q, kv = cfg.query_width, cfg.key_value_width
        x = self.qkv(self.ln1(h))
        qh = x[..., :q].view(b, s, cfg.num_attention_heads, cfg.head_dim)
        kh = x[..., q:q + kv].view(b, s, cfg.num_key_value_heads, cfg.head_dim)
        vh = x[..., q + kv:].view(b, s, cfg.num_key_value_heads, cfg.head_dim)
        qh, kh = _rope(qh, cos[:, :, None, :], sin[:, :, None, :]), _rope(kh, cos[:, :, None, :], sin[:, :, None, :])
        if varlen is not None:
            # documents attended separately, like the product path: tokens flattened, cumulative lengths
            fn, cu, longest = varlen
            a = fn(qh.reshape(b * s, -1, cfg.head_dim), kh.reshape(b * s, -1, cfg.head_dim),
                   vh.reshape(b * s, -1, cfg.head_dim), cu, cu, longest, longest, causal=True).reshape(b, s, q)
        else:
            a = F.scaled_dot_product_attention(qh.transpose(1, 2), kh.transpose(1, 2), vh.transpose(1, 2),
                                               is_causal=True, enable_gqa=True).transpose(1, 2).reshape(b, s, q)
        h = h + self.o(a)
        g, u = self.gu(self.ln2(h)).chunk(2, dim=-1)
        return h + self.down(F.silu(g) * u)


class Model(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([Block(cfg) for _ in range(cfg.num_hidden_layers)])
        self.norm = nn.RMSNorm(cfg.hidden_size, eps=cfg.rms_norm_eps)
        self.head = nn.Linear(cfg.hidden_size, cfg.vocab_size, bias=False)

    def forward(self, ids, targets, weights, denom: float, chunk_rows: int = 4096, positions=None, varlen=None):
        cfg = self.cfg
        b, s = ids.shape
        pos = (torch.arange(s, device=ids.device).expand(b, s) if positions is None else positions).float()
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=ids.device).float() / cfg.head_dim))
        ang = pos[:, :, None] * inv[None, None, :]
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)         # [b, s, half]
        h = self.embed(ids)
        for layer in self.layers:
            h = layer(h, cos, sin, varlen)
        h = self.norm(h).view(b * s, -1)
        total = h.new_zeros((), dtype=torch.float32)
        t, w = targets.reshape(-1), weights.reshape(-1)
        for r0 in range(0, b * s, chunk_rows):     # bounded logits memory, like every trainer does
            logits = self.head(h[r0:r0 + chunk_rows]).float()
            nll = F.cross_entropy(logits, t[r0:r0 + chunk_rows], reduction="none")
            total = total + (nll * w[r0:r0 + chunk_rows]).sum()
        return total / denom


class TorchBaseline:
    """Same call surface as ``api.Trainer`` for the parts ``bench.py`` uses."""

    def __init__(self, cfg, micro_batch_rows: int, lr: float = 2e-5, seed: int = 0):
        self.cfg = cfg
        self.micro = micro_batch_rows
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        torch.manual_seed(seed)
        with torch.device("meta"):
            model = Model(cfg)
        model = model.to(torch.bfloat16)
        if self.world > 1:
            from torch.distributed.fsdp import fully_shard

            for layer in model.layers:
                fully_shard(layer)
            fully_shard(model)
        model.to_empty(device=self.device)
        with torch.no_grad():
            for name, p in model.named_parameters():
                if p.dim() > 1:
                    p.normal_(0.0, cfg.initializer_range)
                elif "ln" in name or "norm" in name:
                    p.fill_(1.0)
                else:
                    p.zero_()
        self.model = model
        decay = [p for p in model.parameters() if p.dim() > 1]
        plain = [p for p in model.parameters() if p.dim() <= 1]
        self.opt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": plain, "weight_decay": 0.0}],
                                     lr=lr, betas=(0.9, 0.95), eps=1e-8, fused=True)
        self._h2d = self._d2h = 0
        try:
            from flash_attn import flash_attn_varlen_func

            self.varlen_fn = flash_attn_varlen_func
        except ImportError:
            self.varlen_fn = None
        self.attention = ("flash_attn varlen (documents attended separately)" if self.varlen_fn is not None
                          else "SDPA causal over whole rows (no segment mask)")

    @staticmethod
    def _document_bounds(segments: torch.Tensor):
        """Cumulative lengths of the runs of equal segment id over the flattened ``[rows * seq]`` tokens
        (padding runs included: they attend among themselves, at zero loss weight)."""
        flat = segments.reshape(-1)
        rows, seq = segments.shape
        change = torch.ones_like(flat, dtype=torch.bool)
        change[1:] = flat[1:] != flat[:-1]
        change[::seq] = True                              # a row boundary always starts a run
        starts = torch.nonzero(change).reshape(-1).to(torch.int32)
        cu = torch.cat([starts, torch.tensor([flat.numel()], dtype=torch.int32, device=flat.device)])
        return cu, int((cu[1:] - cu[:-1]).max())

    def upload(self, host_batch):
        out = {}
        if self.varlen_fn is not None:
            # document bounds of every micro-batch, found on the host copy (no device read back)
            seg = host_batch["segment_ids"]
            out["_varlen"] = []
            for r0 in range(0, seg.shape[0], self.micro):
                cu, longest = self._document_bounds(seg[r0:r0 + self.micro])
                out["_varlen"].append((cu.to(self.device, non_blocking=True), longest))
        for k in ("input_ids", "attention_mask", "segment_ids", "position_ids"):
            v = host_batch[k]
            self._h2d += v.numel() * v.element_size()
            out[k] = v.to(self.device, non_blocking=True)
        return out

    def train_step_device(self, batch):
        from ..training import losses

        rows = batch["input_ids"].shape[0]
        targets, weights = losses.aligned_targets_and_weights(batch)
        total = weights.sum(dtype=torch.float32)
        if self.world > 1:
            dist.all_reduce(total)
        denom = float(total.clamp(min=1.0))
        loss_sum = None
        for r0 in range(0, rows, self.micro):
            sl = slice(r0, r0 + self.micro)
            varlen = positions = None
            if self.varlen_fn is not None:
                cu, longest = batch["_varlen"][r0 // self.micro]
                varlen = (self.varlen_fn, cu, longest)
                positions = batch["position_ids"][sl] if "position_ids" in batch else None
            loss = self.model(batch["input_ids"][sl].long(), targets[sl].long().clamp(min=0), weights[sl].float(), denom,
                              positions=positions, varlen=varlen)
            loss.backward()
            loss_sum = loss.detach() if loss_sum is None else loss_sum + loss.detach()
        norm = torch.nn.utils.clip_grad_norm_(self.model.parameters(), 1.0)
        self.opt.step()
        self.opt.zero_grad(set_to_none=True)
        return loss_sum, norm

    def train_step(self, host_batch):
        loss, norm = self.train_step_device(self.upload(host_batch))
        if self.world > 1:
            loss = loss.clone()
            dist.all_reduce(loss)
        norm = norm.full_tensor() if hasattr(norm, "full_tensor") else norm
        packed = torch.stack([loss.float(), norm.float()]).cpu()
        self._d2h += 8
        return {"loss": float(packed[0]), "grad_norm": float(packed[1])}

    def transfer_counters(self):
        return self._h2d, self._d2h
