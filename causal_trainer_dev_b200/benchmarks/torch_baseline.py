"""Library baseline of the headline benchmark: the same Llama-shape training step written with
stock PyTorch only — cuBLAS matmuls, ``scaled_dot_product_attention`` (flash backend, plain causal
mask: segment isolation is dropped, which only helps the baseline), ``F.cross_entropy`` in row
chunks, autograd, fused ``torch.optim.AdamW`` and, on several GPUs, ``fully_shard`` (FSDP2) over
NCCL.  None of this repository's kernels run here.  It exists to give the product path a
same-box, same-shape number to stand against (``bench.py --impl torch``).
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

    def forward(self, h, cos, sin):
        cfg = self.cfg
        b, s, _ = h.shape
        q, kv = cfg.query_width, cfg.key_value_width
        x = self.qkv(self.ln1(h))
        qh = x[..., :q].view(b, s, cfg.num_attention_heads, cfg.head_dim).transpose(1, 2)
        kh = x[..., q:q + kv].view(b, s, cfg.num_key_value_heads, cfg.head_dim).transpose(1, 2)
        vh = x[..., q + kv:].view(b, s, cfg.num_key_value_heads, cfg.head_dim).transpose(1, 2)
        qh, kh = _rope(qh, cos, sin), _rope(kh, cos, sin)
        a = F.scaled_dot_product_attention(qh, kh, vh, is_causal=True, enable_gqa=True)
        h = h + self.o(a.transpose(1, 2).reshape(b, s, q))
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

    def forward(self, ids, targets, weights, denom: float, chunk_rows: int = 4096):
        cfg = self.cfg
        b, s = ids.shape
        pos = torch.arange(s, device=ids.device, dtype=torch.float32)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=ids.device).float() / cfg.head_dim))
        ang = pos[:, None] * inv[None, :]
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        h = self.embed(ids)
        for layer in self.layers:
            h = layer(h, cos, sin)
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

    def upload(self, host_batch):
        out = {}
        for k in ("input_ids", "attention_mask", "segment_ids"):
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
            loss = self.model(batch["input_ids"][sl].long(), targets[sl].long().clamp(min=0), weights[sl].float(), denom)
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
