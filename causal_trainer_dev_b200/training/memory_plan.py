"""Per-GPU memory plan of a training configuration, computed from shapes alone.

``plan(...)`` lists the buffers a rank allocates for a model, a row length and a rank lattice --
parameter shards, AdamW moments, gradient accumulators, gathered-unit and staging buffers, the
activations a layer keeps for its backward pass, attention metadata, the rotary table, the
sequence-parallel K / V ring, the tensor-parallel rings, MoBA's grouping and gather buffers, the
loss chunk -- and how many layers can keep their activations in what is left of the HBM.  The
figures are estimates from shapes (ring depths and capacities as the runtime sizes them, no
allocator slack); nothing is allocated, so the plan can be asked about a million-token row on a
laptop; the engine's own activation policy (``LayerwiseEngine._layers_to_keep``) uses the same
per-layer figures.

The reference checks the same property -- no buffer grows with the square of the row length, from
4 K to 1 M tokens -- by capturing kernel call shapes without running them
(tests/kernels/test_efficient_attention.py:88-110); ``tests/test_memory_plan_cpu.py`` does it on
this plan.

    python -m causal_trainer_dev_b200.training.memory_plan --model llama3-8b --seq_len 131072 \
        --rows 1 --sharding 1,1,1,4,1 --moba 4096,4
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass

from ..models.config import ModelConfig, preset
from ..models.params import unit_layouts

HBM_BYTES = 183_359 * (1 << 20)      # what a B200 reports
FLAG_CHUNK = 65536                   # elements per all-gather flag: units are padded to ranks x this
GATHERED_UNITS = 3                   # gathered parameter buffers in rotation when not all can stay resident
STAGING_SLOTS = 3                    # gradient staging slots
RING_SLOTS = 8                       # symmetric activation / K-V buffers in rotation


@dataclass(frozen=True)
class Lattice:
    fsdp: int = 1      # data ranks that shard parameters (dp x fsdp of the command line)
    tp: int = 1
    sp: int = 1

    @property
    def shard_ranks(self) -> int:
        return self.fsdp * self.sp           # the sp ranks are further FSDP ranks


def layer_activation_bytes(cfg: ModelConfig, tokens: int) -> int:
    """What one layer keeps for its backward pass: the residual input, both norm outputs, Q | K | V
    and the attention output, the gate / up product and the SwiGLU output (bf16), the log-sum-exp
    and the two inverse norms (fp32)."""
    return (tokens * 2 * (3 * cfg.hidden_size + 2 * cfg.query_width + 2 * cfg.key_value_width + 2 * cfg.intermediate_size)
            + tokens * 12 * cfg.num_attention_heads)


def backward_working_set_bytes(cfg: ModelConfig, tokens: int, cut_chunk_rows: int) -> int:
    """Transient buffers of one layer's backward pass plus the loss chunk (bf16 logits slab)."""
    return tokens * 2 * (6 * cfg.intermediate_size + 8 * cfg.hidden_size) + cut_chunk_rows * cfg.vocab_size * 2


def _local_config(cfg: ModelConfig, tp: int) -> ModelConfig:
    if tp == 1:
        return cfg
    from ..parallel.tp import tp_local_config

    return tp_local_config(cfg, tp)


def plan(cfg: ModelConfig, *, seq_len: int, micro_rows: int, lattice: Lattice = Lattice(), micro_batches: int = 1,
         moba: tuple[int, int] | None = None, cut_chunk_rows: int = 4096, reserve_bytes: int = 8 << 30,
         hbm_bytes: int = HBM_BYTES) -> dict:
    """Bytes per GPU, by buffer, and the number of layers whose activations fit (``layers_kept``)."""
    if seq_len % (128 * lattice.sp):
        raise ValueError("seq_len must be a multiple of 128 x sp")
    local = _local_config(cfg, lattice.tp)
    ranks = lattice.shard_ranks
    grain = ranks * FLAG_CHUNK
    padded = [-(-u.numel // grain) * grain for u in unit_layouts(local)]
    shard_elems = sum(padded) // ranks
    sharded = ranks > 1 or lattice.tp > 1
    out: dict[str, int] = {}
    out["parameter_shards"] = 2 * shard_elems
    out["adam_moments"] = 4 * shard_elems                                   # bf16 first and second moments
    out["gradient_shards"] = (4 if micro_batches > 1 else 2) * shard_elems  # fp32 when micro-batches accumulate
    if sharded:
        all_units, rotating = 2 * sum(padded), 2 * GATHERED_UNITS * max(padded)
        out["gradient_staging"] = 2 * STAGING_SLOTS * max(padded)
    else:
        all_units = rotating = 0                                            # one rank trains in place
        out["gradient_staging"] = 0
    # tokens: what a rank holds between projections / inside attention and the MLP
    seq_local = seq_len // lattice.sp
    tokens_full = micro_rows * seq_local                                    # all tokens of the rank's rows (its sp slice)
    tokens_rows = tokens_full // lattice.tp                                 # row-sharded over tp between projections
    per_layer = layer_activation_bytes(local, tokens_full)
    working = backward_working_set_bytes(local, tokens_full, cut_chunk_rows)
    out["attention_metadata"] = micro_rows * seq_len * 4 * 9 + micro_rows * (seq_len // 128) * 4 * 8
    out["rotary_table"] = 2 * micro_rows * seq_local * local.rotary_dim * 4 // 2
    if lattice.sp > 1:
        out["sp_kv_ring"] = RING_SLOTS * seq_len * 2 * local.key_value_width * 2
        out["sp_kv_in_sequence_order"] = 2 * seq_len * 2 * local.key_value_width * 2
    if lattice.tp > 1:
        widest = max(local.hidden_size, local.query_width)                  # gathered hidden rows, pushed partial sums
        out["tp_rings"] = 2 * RING_SLOTS * tokens_rows * lattice.tp * widest * 2
    if moba is not None:
        block, top_k = moba
        picks = max(top_k - 1, 1)
        hq, hkv, d = local.num_attention_heads, local.num_key_value_heads, local.head_dim
        rows = micro_rows * hq * seq_len
        slot_cap = micro_rows * hkv * -(-seq_len // block)
        rows_cap = -(-rows * picks // 256) * 256 + 256 * slot_cap
        words = -(-(-(-seq_len // block)) // 32)
        out["moba_selection_bits"] = rows * words * 4
        out["moba_grouping"] = 2 * rows * picks * 4 + rows_cap * 4 + slot_cap * 4 * (6 + block // 128 * 4) + rows_cap // 128 * 16
        # gathered Q, the grouped output and its statistics (forward); dO, dQ per gathered row (backward)
        out["moba_gathered_rows"] = rows_cap * (2 * d * 2 + 8) + rows_cap * (2 * d * 2)
        out["moba_pooled_keys"] = micro_rows * hkv * (seq_len // 128) * d * 4
    fixed = sum(out.values()) + working + reserve_bytes
    resident = sharded and fixed + all_units + per_layer <= hbm_bytes       # every unit's gathered copy stays
    out["gathered_units"] = all_units if resident else rotating
    fixed += out["gathered_units"]
    budget = hbm_bytes - fixed
    kept = max(0, min(cfg.num_hidden_layers, budget // per_layer))
    out.update(backward_working_set=working, reserve=reserve_bytes, activations_per_layer=per_layer,
               activations_kept=kept * per_layer, layers_kept=int(kept), layers=cfg.num_hidden_layers,
               gathered_units_resident=bool(resident), tokens_per_micro_batch=tokens_full,
               total=fixed + kept * per_layer, hbm=hbm_bytes, fits=bool(budget >= per_layer))
    return out


def main(argv: list[str] | None = None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    p.add_argument("--model", default="llama3-8b", help="a preset name (models.config.preset)")
    p.add_argument("--seq_len", type=int, default=4096)
    p.add_argument("--rows", type=int, default=4, help="rows per micro-batch on one data rank")
    p.add_argument("--micro_batches", type=int, default=1)
    p.add_argument("--sharding", default="1,1,1,1,1", help="dp,fsdp,ep,tp,sp as on the training command line")
    p.add_argument("--moba", default="", help="block,top_k for MoBA layers")
    a = p.parse_args(argv)
    dp, fsdp, _, tp, sp = (int(x) for x in a.sharding.split(","))
    moba = tuple(int(x) for x in a.moba.split(",")) if a.moba else None
    result = plan(preset(a.model), seq_len=a.seq_len, micro_rows=a.rows, lattice=Lattice(dp * fsdp, tp, sp),
                  micro_batches=a.micro_batches, moba=moba)
    width = max(len(k) for k in result)
    counts = ("layers_kept", "layers", "tokens_per_micro_batch", "gathered_units_resident", "fits")
    for k, v in result.items():
        shown = f"{v!s:>10}" if k in counts else f"{v / 2**30:10.2f} GiB"
        print(f"{k:<{width}}  {shown}")
    print(json.dumps(result))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
