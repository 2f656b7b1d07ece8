"""Small public helpers that the main paths do not exercise directly."""
import pytest
import torch

from causal_trainer_dev_b200.models.config import preset
from causal_trainer_dev_b200.models.freezing import split_trainable
from causal_trainer_dev_b200.models.params import ModelParams
from causal_trainer_dev_b200.parallel import runtime as rt
from causal_trainer_dev_b200.parallel.tp import kv_replicas, merge_unit_tensor, slice_unit_tensor
from causal_trainer_dev_b200.training.losses import mean_loss


@pytest.mark.parametrize("kv_heads,tp", [(2, 2), (1, 2), (4, 4), (2, 4)])
def test_tensor_parallel_slices_merge_back(kv_heads, tp):
    """slice_unit_tensor / merge_unit_tensor are inverses, also when key/value heads are shared."""
    cfg = preset("tiny", num_attention_heads=4, num_key_value_heads=kv_heads, intermediate_size=512)
    q, kv, f, d = cfg.query_width, cfg.key_value_width, cfg.intermediate_size, cfg.hidden_size
    gen = torch.Generator().manual_seed(0)
    shapes = {"qkv_w": (q + 2 * kv, d), "qkv_b": (q + 2 * kv,), "o_w": (d, q), "gu_w": (2 * f, d), "down_w": (d, f),
              "embed": (cfg.vocab_size, d), "lm_head": (cfg.vocab_size, d), "ln1": (d,)}
    for name, shape in shapes.items():
        full = torch.randn(shape, generator=gen)
        parts = [slice_unit_tensor(name, full, cfg, tp, r) for r in range(tp)]
        assert torch.equal(merge_unit_tensor(name, parts, cfg), full), name
    rep = kv_replicas(cfg, tp)
    assert rep == max(1, tp // kv_heads)
    if rep > 1:     # ranks that share a key/value head hold identical K/V rows
        full = torch.randn(shapes["qkv_w"], generator=gen)
        a, b = slice_unit_tensor("qkv_w", full, cfg, tp, 0), slice_unit_tensor("qkv_w", full, cfg, tp, 1)
        assert torch.equal(a[q // tp:], b[q // tp:]) and not torch.equal(a[:q // tp], b[:q // tp])


def test_split_trainable_reports_frozen_components():
    cfg = preset("tiny")
    names = ModelParams(cfg, torch.float32, "cpu").hf_names()
    frozen, trainable = split_trainable(cfg, ("embed", "norm"), names)
    assert "model.embed_tokens.weight" in frozen and "model.norm.weight" in frozen
    assert "model.layers.0.input_layernorm.weight" in frozen and "lm_head.weight" in trainable
    assert sorted(frozen + trainable) == sorted(names)


def test_single_process_host_collectives_are_identities():
    assert rt.broadcast_object({"a": 1}) == {"a": 1}
    assert rt.allgather_object(3) == [3]
    assert rt.pickle_digest([1, 2]) == rt.pickle_digest([1, 2]) != rt.pickle_digest([2, 1])


def test_mean_loss_guards_empty_batches():
    assert float(mean_loss(torch.tensor(6.0), torch.tensor(3.0))) == 2.0
    assert float(mean_loss(torch.tensor(0.0), torch.tensor(0.0))) == 0.0


def test_loss_backend_resolution():
    from causal_trainer_dev_b200.training.arguments import parse_args
    from causal_trainer_dev_b200.training.runner import resolve_loss_implementation

    base = ["--repo-id", "local-model", "--dataset-name", "local-data"]
    for mode in ([], ["--lora", "True"], ["--lora", "True", "--lora-train-embed-and-lm-head", "True"]):
        args = parse_args(base + mode)
        assert resolve_loss_implementation(args) == "cut"
        assert resolve_loss_implementation(args, cut_supported=False) == "pallas"
    for explicit in ("cut", "pallas", "xla"):
        args = parse_args(base + ["--loss-implementation", explicit])
        assert resolve_loss_implementation(args, cut_supported=explicit != "cut") == explicit
    chunked = parse_args(base + ["--cut-chunk-size", "4"])
    assert resolve_loss_implementation(chunked) == "cut"
    with pytest.raises(ValueError, match="cut_chunk_size"):
        resolve_loss_implementation(chunked, cut_supported=False)
    with pytest.raises(ValueError, match="CUDA"):
        resolve_loss_implementation(chunked, "tpu")


def test_schedule_builder_and_tensor_level_loss_entry_points():
    from causal_trainer_dev_b200.training.losses import causal_lm_loss, chunked_causal_lm_loss, shifted_loss_mask
    from causal_trainer_dev_b200.training.optimizer import build_learning_rate_schedule

    sched = build_learning_rate_schedule("cosine", 1e-3, 1e-4, total_steps=10, warmup_steps=2)
    assert sched(0) == 0.0 and sched(1) == pytest.approx(5e-4) and sched(2) == pytest.approx(1e-3)
    assert sched(10) == pytest.approx(1e-4) and sched(6) == pytest.approx(1e-4 + 9e-4 * 0.5)
    assert build_learning_rate_schedule("linear", 1.0, 0.0, 4)(2) == pytest.approx(0.5)
    assert build_learning_rate_schedule("constant", 1.0, 0.0, 1, warmup_steps=1)(0) == 1.0
    for bad in (dict(total_steps=0), dict(total_steps=4, warmup_steps=4), dict(total_steps=4, warmup_steps=-1)):
        with pytest.raises(ValueError):
            build_learning_rate_schedule("cosine", 1.0, 0.0, **bad)
    with pytest.raises(ValueError, match="unsupported scheduler"):
        build_learning_rate_schedule("exponential", 1.0, 0.0, 4)

    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(1, 50, (2, 8), generator=gen)
    mask = torch.tensor([[1] * 8, [1] * 6 + [0] * 2])
    seg = torch.tensor([[1] * 4 + [2] * 4, [1] * 6 + [0] * 2])
    frac = torch.rand(2, 8, generator=gen) * mask
    hidden = torch.randn(2, 8, 16, generator=gen)
    head = torch.randn(50, 16, generator=gen)
    targets, supervised = shifted_loss_mask(ids, mask, seg)
    assert supervised.dtype == torch.bool and not supervised[0, 3] and not supervised[1, 5:].any()
    got = chunked_causal_lm_loss(hidden, head, ids, mask, seg, loss_weights=frac, token_budget=5)
    want = causal_lm_loss(hidden, head, {"input_ids": ids, "attention_mask": mask, "segment_ids": seg,
                                         "loss_weights": frac}, implementation="xla", token_budget=4096)
    assert torch.allclose(got[0], want[0], rtol=1e-5) and torch.allclose(got[1], want[1])
    logp = torch.log_softmax(hidden.reshape(-1, 16) @ head.t(), dim=-1)
    pt = torch.randint(0, 50, (2, 8), generator=gen)
    pw = torch.rand(2, 8, generator=gen)
    nll, count = chunked_causal_lm_loss(hidden, head, ids, mask, prediction_targets=pt, prediction_weights=pw)
    assert torch.allclose(nll, -(logp.gather(1, pt.reshape(-1, 1)).squeeze(1) * pw.reshape(-1)).sum(), rtol=1e-5)
    assert torch.allclose(count, pw.sum())
    with pytest.raises(ValueError, match="together"):
        chunked_causal_lm_loss(hidden, head, ids, mask, prediction_targets=pt)


def test_experiment_logger_without_and_with_a_fake_wandb(monkeypatch):
    import sys
    import types

    from causal_trainer_dev_b200.training import logging as tlog

    quiet = tlog.ExperimentLogger(False, "p", None, {})
    quiet.log({"loss": 1.0}, 3)
    quiet.finish()
    assert not quiet.active and tlog.init_wandb(types.SimpleNamespace(use_wandb=False)) is None
    events = []
    run = types.SimpleNamespace(log=lambda values, step: events.append(("log", values, step)),
                                finish=lambda: events.append(("finish",)))
    fake = types.ModuleType("wandb")
    fake.init = lambda **kwargs: events.append(("init", kwargs)) or run
    monkeypatch.setitem(sys.modules, "wandb", fake)
    logger = tlog.init_wandb(types.SimpleNamespace(use_wandb=True, wandb_project="proj", wandb_run_name="r"))
    logger.log({"loss": 2.0}, 7)
    logger.finish()
    assert events[0][0] == "init" and events[0][1]["project"] == "proj" and events[0][1]["name"] == "r"
    assert events[1:] == [("log", {"loss": 2.0}, 7), ("finish",)]
    monkeypatch.setitem(sys.modules, "wandb", None)      # import wandb now fails
    with pytest.raises(RuntimeError, match="wandb"):
        tlog.ExperimentLogger(True, "p", None, {})
    assert tlog.memory_metrics() == {} or all(k.startswith("device_") for k in tlog.memory_metrics())


def test_partition_rules_match_the_tensor_parallel_windows():
    from causal_trainer_dev_b200.checkpointing.huggingface import tp_window

    cfg = preset("tiny", num_attention_heads=4, num_key_value_heads=2, intermediate_size=512)
    p = "model.layers.0."
    for name in (p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "mlp.gate_proj.weight",
                 p + "self_attn.o_proj.weight", p + "mlp.down_proj.weight", "model.embed_tokens.weight", "lm_head.weight",
                 p + "self_attn.q_proj.bias", p + "input_layernorm.weight", "model.norm.weight"):
        spec = rt.parameter_partition_spec(name)
        kind = tp_window(name, cfg, 2, 1)[4]
        expected = {"rows": "tp" in spec[:1], "cols": spec[1:2] == ("tp",), "rep": spec == ()}[kind]
        assert expected, (name, spec, kind)
    assert rt.parameter_partition_spec("layers/0/attention/q_proj/kernel") == ("fsdp", "tp")
    assert rt.parameter_partition_spec("layers/0/attention/o_proj/kernel") == ("tp", "fsdp")
    assert rt.parameter_partition_spec("layers/0/input_layernorm/scale") == ()
    assert rt.resolve_axis_dims("-1, 1, 1, 4, 1", 32) == (8, 1, 1, 4, 1)
    assert rt.parse_local_device_ids(" 2, 3 ") == (2, 3) and rt.parse_local_device_ids("") is None
    assert rt.parse_local_device_ids([1]) == (1,) and rt.parse_local_device_ids(None) is None
    for bad in ("1,1", "-1", []):
        with pytest.raises(ValueError):
            rt.parse_local_device_ids(bad)
    env = rt.detect_environment("127.0.0.1:1", 2, 1, "5,6", env={})
    assert env.local_rank == 5


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the message of a box without CUDA")
def test_trainer_without_cuda_names_the_cpu_path():
    from causal_trainer_dev_b200.api import Trainer

    with pytest.raises(RuntimeError, match="make_train_step"):
        Trainer(preset("tiny"))
