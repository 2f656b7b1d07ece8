"""LoRA fine-tuning on the layerwise CUDA engine.

The base model is frozen: every projection still runs on the tcgen05 GEMM (forward and input
gradient), but no base weight gradient is computed and no gradient or optimizer memory exists for
the base weights.  Each adapted projection adds the rank-``r`` path ``(x @ A) @ B`` (no alpha
multiplier; src/causal_trainer/modeling/lora.py:1-9,218-242) to the slice of the fused output that
belongs to it (``q | k | v`` inside ``qkv``, ``gate | up`` inside ``gu``) and its backward

    t  = x @ A            dB += t^T @ dy
    dt = dy @ B^T         dA += x^T @ dt          dx += dt @ A^T

The rank-``r`` products (a fraction ``r / d`` of the projection's FLOPs) run on the same tcgen05
GEMM as the projections whenever ``r`` is a multiple of 8 (16-byte rows): the adapter output is
accumulated straight into the projection's output slice and the input gradient into ``dx`` through
the GEMM's reduce-add epilogue, the adapter gradients into fp32 buffers.  Adapter gradients are
handed to the optimizer step as extra regions (``training.steps.TrainStep``), which also
all-reduces them over data-parallel replicas.

The weight provider may be the sharded runtime in its weights-only mode
(``FsdpRuntime(trainable=False)``): the frozen base is then sharded over the data ranks and
all-gathered into the consuming GEMMs like any trained model, with no gradient or optimizer memory
behind it (src/causal_trainer/modeling/lora.py:178-242, src/causal_trainer/training/steps.py:378-552).
"""
from __future__ import annotations

import torch

from ..models.config import ModelConfig
from ..models.lora import LoraState
from ..ops.gemm import gemm
from .engine import EngineOptions, LayerwiseEngine


def _column_ranges(cfg: ModelConfig) -> dict[str, list[tuple[str, int, int]]]:
    """Fused projection -> [(adapter name, first output column, one past the last)]."""
    q, kv, f, d = cfg.query_width, cfg.key_value_width, cfg.intermediate_size, cfg.hidden_size
    return {
        "qkv": [("q_proj", 0, q), ("k_proj", q, q + kv), ("v_proj", q + kv, q + 2 * kv)],
        "o": [("o_proj", 0, d)],
        "gu": [("gate_proj", 0, f), ("up_proj", f, 2 * f)],
        "down": [("down_proj", 0, d)],
    }


class LoraLayerwiseEngine(LayerwiseEngine):
    """Gradient producer for adapters only; ``grads[(layer, name)] = (dA, dB)`` in fp32."""

    def __init__(self, cfg: ModelConfig, provider, lora: LoraState, options: EngineOptions | None = None):
        super().__init__(cfg, provider, options)
        if lora.train_embed_and_lm_head:
            raise ValueError("the LoRA engine trains adapters only; trainable embedding / LM head copies run on "
                             "the autograd path")
        self.lora = lora
        self.train_base = False
        self._ranges = _column_ranges(cfg)
        self.grads = {key: (torch.zeros_like(lora.a[key], dtype=torch.float32),
                            torch.zeros_like(lora.b[key], dtype=torch.float32)) for key in lora.a}

    def extra_regions(self) -> list[tuple[torch.Tensor, bool, object]]:
        """``(parameter, decays, gradient getter)`` per adapter leaf, in the adapter's stable order."""
        out = []
        for name, t in self.lora.trainable():
            _, layer, proj, leaf = name.split("/")
            ga, gb = self.grads[(int(layer), proj)]
            g = ga if leaf == "lora_a" else gb
            out.append((t.detach(), t.dim() > 1, (lambda g=g: g)))
        return out

    @staticmethod
    def _on_tensor_cores(a: torch.Tensor, x: torch.Tensor) -> bool:
        return a.shape[1] % 8 == 0 and a.dtype == torch.bfloat16 and x.dtype == torch.bfloat16

    def _project(self, li, name, x, w):
        y = super()._project(li, name, x, w)
        for proj, lo, hi in self._ranges[name]:
            a, b = self.lora.pair(li, proj)            # a [in, r], b [r, out]
            if self._on_tensor_cores(a, x):
                t = gemm(x, a, b_mn=True)                                   # x @ a
                gemm(t, b, b_mn=True, out=y[:, lo:hi], accumulate=True)     # y += t @ b
            else:
                y[:, lo:hi].addmm_(x @ a, b)
            self._count(2)
        return y

    def _project_backward(self, li, name, dy, x, w, g, accumulate):
        dx = super()._project_backward(li, name, dy, x, w, g, accumulate)
        for proj, lo, hi in self._ranges[name]:
            a, b = self.lora.pair(li, proj)
            ga, gb = self.grads[(li, proj)]
            dys = dy[:, lo:hi]
            if self._on_tensor_cores(a, x):
                t = gemm(x, a, b_mn=True)                                             # x @ a           [T, r]
                dt = gemm(dys, b)                                                     # dy @ b^T        [T, r]
                gemm(t, dys, a_mn=True, b_mn=True, out=gb, accumulate=accumulate)     # dB (+)= t^T dy  [r, out]
                gemm(x, dt, a_mn=True, b_mn=True, out=ga, accumulate=accumulate)      # dA (+)= x^T dt  [in, r]
                gemm(dt, a, out=dx, accumulate=True)                                  # dx += dt @ a^T
            else:
                t = x @ a
                dt = dys @ b.t()
                d_b = t.t() @ dys
                d_a = x.t() @ dt
                if accumulate:
                    ga.add_(d_a)
                    gb.add_(d_b)
                else:
                    ga.copy_(d_a)
                    gb.copy_(d_b)
                dx.addmm_(dt, a.t())
            self._count(7)
        return dx
