"""causal-train end to end on a B200: the command-line path through the sm_100a engine
(raw JSONL -> tokenise -> pack -> train on the CUDA kernels -> checkpoint bundle -> resume)."""
import json

import pytest
import torch

from helpers import write_model_dir

pytestmark = pytest.mark.gpu


def _argv(tmp_path, *extra):
    from test_runner_cpu import _data

    model = tmp_path / "model"
    if not model.exists():
        write_model_dir(model, hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=64, torch_dtype="bfloat16")
    data = _data(tmp_path / "train.jsonl", n=600)
    return ["--repo_id", str(model), "--dataset_name", str(data), "--output_dir", str(tmp_path / "out"),
            "--max_sequence_length", "256", "--packing", "--total_batch_size", "2", "--sharding_axis", "1,1,1,1,1",
            "--param_dtype", "bfloat16", "--dtype", "bfloat16", "--attn_mechanism", "efficient",
            "--loss_implementation", "cut", "--learning_rate", "3e-3", "--scheduler", "constant", "--logging_steps", "1",
            "--no-distributed", *extra]


def test_cli_trains_on_the_cuda_engine_and_resumes(cuda_lib, tmp_path):
    from causal_trainer_dev_b200.checkpointing import bundles, safetensors_io as st
    from causal_trainer_dev_b200.training import runner
    from causal_trainer_dev_b200.training.arguments import parse_args

    before = cuda_lib.launch_count()
    argv = _argv(tmp_path, "--max_steps", "6", "--save_steps", "3", "--save_optimizer_state")
    run = runner.TrainingRun(parse_args(argv))
    assert run.use_engine
    run.resolve_model(); run.load_data(); run.discover_resume(); run.build_model(); run.train()
    assert cuda_lib.launch_count() > before + 100          # the step ran on this library's kernels
    out = tmp_path / "out"
    manifest = json.loads((out / bundles.MANIFEST_NAME).read_text())
    assert manifest["global_step"] == 6 and manifest["total_steps"] == 6 and manifest["has_optimizer_state"]
    tensors, _, _ = st.read_header(out / "model.safetensors")
    assert tensors["lm_head.weight"].dtype == "BF16" and (out / "checkpoint-3").is_dir()
    # relaunch: the finished run is recognised and left untouched
    before_bytes = (out / "model.safetensors").read_bytes()
    assert runner.main(argv) == 0 and (out / "model.safetensors").read_bytes() == before_bytes
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_cli_pallas_loss_backend_and_frozen_embeddings(cuda_lib, tmp_path):
    from causal_trainer_dev_b200.training import runner

    argv = _argv(tmp_path, "--max_steps", "3", "--loss_implementation", "pallas")
    assert runner.main(argv) == 0
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_cli_profiles_steps_with_cuda_events_and_honours_the_memory_flags(cuda_lib, tmp_path):
    """``--profile_steps`` on a GPU (CUDA events, not the host clock), with every layer recomputed in
    groups of two, the MLP tiled and the norm scales frozen."""
    from causal_trainer_dev_b200.training import runner
    from causal_trainer_dev_b200.training.arguments import parse_args

    argv = _argv(tmp_path, "--max_steps", "5", "--profile_steps", "2", "--activation_memory", "recompute",
                 "--mlp_chunk_size", "128", "--frozen_parameters", "norm")
    run = runner.TrainingRun(parse_args(argv))
    run.resolve_model(); run.load_data(); run.discover_resume(); run.build_model()
    engine = run.step_fn.producer
    assert engine.options.remat == "full" and engine.options.mlp_chunk_rows == 128 and not engine.options.train_norm
    run.train()
    assert engine.kept_layers == 0
    profile = json.loads((tmp_path / "out" / "profile_steps.json").read_text())
    assert profile["profiled_steps"] == 2 and profile["ms_per_step"] > 0 and "event" in profile["clock"].lower()
    assert cuda_lib.device_status() == (0, 0, 0, 0)


def test_cli_lora_runs_on_the_cuda_engine_and_writes_a_peft_adapter(cuda_lib, tmp_path):
    from causal_trainer_dev_b200.checkpointing import safetensors_io as st
    from causal_trainer_dev_b200.training import runner
    from causal_trainer_dev_b200.training.arguments import parse_args
    from causal_trainer_dev_b200.training.lora_engine import LoraLayerwiseEngine

    argv = _argv(tmp_path, "--max_steps", "3", "--lora", "--lora_rank", "8", "--lora_save_adapter_only")
    run = runner.TrainingRun(parse_args(argv))
    assert run.use_lora_engine and not run.use_engine
    run.resolve_model(); run.load_data(); run.discover_resume(); run.build_model()
    assert isinstance(run.step_fn.producer, LoraLayerwiseEngine)
    run.train()
    out = tmp_path / "out"
    cfg = json.loads((out / "adapter_config.json").read_text())
    assert cfg["r"] == 8 and cfg["lora_alpha"] == 8
    tensors = st.load_file(out / "adapter_model.safetensors")
    b = tensors["base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight"]
    assert b.shape == (256, 8) and float(b.float().abs().max()) > 0.0       # B left zero: the adapter trained
    assert cuda_lib.device_status() == (0, 0, 0, 0)
