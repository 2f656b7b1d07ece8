"""Shape-only checks of the per-GPU memory plan: nothing is allocated, so rows of a million tokens
can be asked about on any machine (the reference does the same by capturing kernel call shapes,
tests/kernels/test_efficient_attention.py:88-110)."""
import pytest

from causal_trainer_dev_b200.models.config import preset
from causal_trainer_dev_b200.training.memory_plan import (Lattice, backward_working_set_bytes, layer_activation_bytes,
                                                          main, plan)

SIZED_BY_THE_ROW = ("activations_per_layer", "attention_metadata", "rotary_table", "sp_kv_ring", "sp_kv_in_sequence_order",
                    "tp_rings", "moba_grouping", "moba_gathered_rows", "moba_pooled_keys")


def test_headline_configuration_keeps_every_layer_on_one_gpu_and_on_eight():
    cfg = preset("llama3-8b")
    one = plan(cfg, seq_len=4096, micro_rows=4, micro_batches=8)
    assert one["layers_kept"] == 32 and one["fits"] and one["gathered_units"] == 0
    # 8.03 B parameters: bf16 weights + two bf16 moments + fp32 gradient accumulators
    assert 8.0e9 * 10 < one["parameter_shards"] + one["adam_moments"] + one["gradient_shards"] < 8.1e9 * 10
    eight = plan(cfg, seq_len=4096, micro_rows=4, lattice=Lattice(fsdp=8))
    assert eight["layers_kept"] == 32 and eight["gathered_units_resident"]
    assert eight["parameter_shards"] * 8 == pytest.approx(one["parameter_shards"], rel=0.01)
    assert eight["total"] < one["total"]


@pytest.mark.parametrize("lattice,moba", [(Lattice(tp=8), (4096, 4)), (Lattice(tp=4, sp=2), None), (Lattice(fsdp=2, tp=4), (4096, 12))])
def test_no_buffer_grows_faster_than_the_row_from_4k_to_1m_tokens(lattice, moba):
    cfg = preset("llama3-8b")
    short = plan(cfg, seq_len=4096, micro_rows=1, lattice=lattice, moba=moba)
    for seq in (32768, 131072, 1 << 20):
        long = plan(cfg, seq_len=seq, micro_rows=1, lattice=lattice, moba=moba)
        ratio = seq / 4096
        for key in SIZED_BY_THE_ROW:
            if key in short:
                assert long[key] <= short[key] * ratio * 1.05 + (1 << 20), (key, seq)
        for key in ("parameter_shards", "adam_moments", "gradient_shards", "gradient_staging"):
            assert long[key] == short[key]
        if moba is not None:
            # the router's selection is one bit per (query row, key block): the one buffer that grows with
            # the square of the row, with a constant that keeps it under a hundredth of a layer's activations
            assert long["moba_selection_bits"] * 100 < long["activations_per_layer"]


def test_a_million_token_row_needs_recomputation_and_says_so():
    cfg = preset("llama3-8b")
    huge = plan(cfg, seq_len=1 << 20, micro_rows=1, lattice=Lattice(tp=8), moba=(4096, 12))
    assert huge["layers_kept"] < cfg.num_hidden_layers            # tens of GB per layer: most layers are recomputed
    assert huge["activations_kept"] == huge["layers_kept"] * huge["activations_per_layer"]
    modest = plan(cfg, seq_len=131072, micro_rows=1, lattice=Lattice(tp=4), moba=(4096, 4))
    assert modest["fits"] and modest["total"] <= modest["hbm"]


def test_per_layer_figures_are_the_ones_the_engine_uses():
    cfg = preset("llama3-8b")
    t = 16384
    assert layer_activation_bytes(cfg, t) == t * 2 * (3 * 4096 + 2 * 4096 + 2 * 1024 + 2 * 14336) + t * 12 * 32
    assert backward_working_set_bytes(cfg, t, 4096) == t * 2 * (6 * 14336 + 8 * 4096) + 4096 * 128256 * 2


def test_command_line_prints_the_plan(capsys):
    assert main(["--model", "llama3-8b", "--seq_len", "32768", "--rows", "1", "--sharding", "1,2,1,4,1", "--moba", "4096,4"]) == 0
    text = capsys.readouterr().out
    assert "layers_kept" in text and "moba_gathered_rows" in text and "GiB" in text
    with pytest.raises(ValueError):
        plan(preset("llama3-8b"), seq_len=4096 + 64, micro_rows=1)


def test_engine_policy_counts_layers_from_the_same_figures(monkeypatch):
    import torch

    from causal_trainer_dev_b200.training.engine import EngineOptions, LayerwiseEngine

    cfg = preset("llama3-8b")
    engine = LayerwiseEngine.__new__(LayerwiseEngine)
    engine.cfg, engine.options = cfg, EngineOptions()
    tokens = 16384
    per_layer = layer_activation_bytes(cfg, tokens)
    working = backward_working_set_bytes(cfg, tokens, engine.options.cut_chunk_rows)
    free = working + engine.options.memory_reserve_bytes + 5 * per_layer + per_layer // 2
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda: (free, 0))
    monkeypatch.setattr(torch.cuda, "memory_reserved", lambda: 0)
    monkeypatch.setattr(torch.cuda, "memory_allocated", lambda: 0)
    assert engine._layers_to_keep(tokens) == 5
    engine.options = EngineOptions(remat="full")
    assert engine._layers_to_keep(tokens) == 0
    engine.options = EngineOptions(remat="none")
    assert engine._layers_to_keep(tokens) == cfg.num_hidden_layers
