"""causal-train end to end on CPU: raw JSONL -> tokenise -> pack -> train -> bundle -> resume."""
import json

import pytest
import torch

from causal_trainer_dev_b200.checkpointing import bundles, safetensors_io as st
from causal_trainer_dev_b200.training import runner
from causal_trainer_dev_b200.training.arguments import parse_args
from helpers import write_model_dir


def _data(path, n=40):
    rows = [{"text": " ".join(f"w{(i * 3 + j) % 40}" for j in range(4 + i % 11))} for i in range(n)]
    path.write_text("\n".join(json.dumps(r) for r in rows))
    return path


def _argv(tmp_path, *extra):
    model = write_model_dir(tmp_path / "model") if not (tmp_path / "model").exists() else tmp_path / "model"
    data = _data(tmp_path / "train.jsonl")
    return ["--repo_id", str(model), "--dataset_name", str(data), "--output_dir", str(tmp_path / "out"),
            "--max_sequence_length", "32", "--packing", "--total_batch_size", "2", "--sharding_axis", "1,1,1,1,1",
            "--param_dtype", "float32", "--dtype", "float32", "--attn_mechanism", "vanilla", "--loss_implementation", "xla",
            "--learning_rate", "1e-2", "--scheduler", "constant", "--logging_steps", "1", "--no-distributed", *extra]


def test_train_save_resume_complete(tmp_path):
    argv = _argv(tmp_path, "--max_steps", "4", "--save_steps", "2", "--save_optimizer_state", "--save_total_limit", "1")
    assert runner.main(argv) == 0
    out = tmp_path / "out"
    manifest = json.loads((out / bundles.MANIFEST_NAME).read_text())
    assert manifest["global_step"] == 4 and manifest["total_steps"] == 4 and manifest["has_optimizer_state"]
    assert manifest["format_version"] == 4 and manifest["artifact_kind"] == "merged"
    assert (out / "model.safetensors").is_file() and (out / "tokenizer.json").is_file() and (out / "training_args.json").is_file()
    assert (out / "checkpoint-2").is_dir()                     # the only periodic bundle (limit 1, step 4 is the final one)
    tensors, meta, _ = st.read_header(out / "model.safetensors")
    assert meta["checkpoint_id"] == manifest["checkpoint_id"] and tensors["lm_head.weight"].dtype == "F32"
    # a second launch finds the finished run and does nothing
    before = (out / "model.safetensors").read_bytes()
    assert runner.main(argv) == 0 and (out / "model.safetensors").read_bytes() == before


def test_interrupted_run_continues_bit_exactly(tmp_path):
    full = _argv(tmp_path, "--max_steps", "4", "--save_optimizer_state")
    run = runner.TrainingRun(parse_args(full))
    run.resolve_model(); run.load_data(); run.discover_resume(); run.build_model(); run.train()
    reference = st.load_file(tmp_path / "out" / "model.safetensors")
    # same run, interrupted after step 2 (a periodic bundle exists), then relaunched
    import shutil

    shutil.rmtree(tmp_path / "out")
    argv = _argv(tmp_path, "--max_steps", "4", "--save_optimizer_state", "--save_steps", "2")
    run = runner.TrainingRun(parse_args(argv))
    run.resolve_model(); run.load_data(); run.discover_resume(); run.build_model()
    run.plan = type(run.plan)(**{**run.plan.__dict__, "total_steps": 4})
    it = iter(run.global_batches())
    for step in (1, 2):
        raw = next(it)
        run.step_fn.run(run.to_device(raw))
    run.save_bundle(tmp_path / "out" / "checkpoint-2", 2)
    resumed = runner.TrainingRun(parse_args(argv))
    resumed.resolve_model(); resumed.load_data(); resumed.discover_resume()
    assert resumed.action == "continue" and resumed.start_step == 2
    resumed.build_model(); resumed.train()
    again = st.load_file(tmp_path / "out" / "model.safetensors")
    assert all(torch.equal(again[k], reference[k]) for k in reference)


def test_changed_flags_make_old_checkpoints_incompatible(tmp_path):
    assert runner.main(_argv(tmp_path, "--max_steps", "2")) == 0
    with pytest.raises(ValueError, match="incompatible"):
        runner.main(_argv(tmp_path, "--max_steps", "2", "--learning_rate", "3e-3"))


def test_streaming_and_lora_adapter_modes(tmp_path):
    argv = _argv(tmp_path, "--dataset_streaming", "--num_train_epochs", "1", "--no-shuffle")
    assert runner.main(argv) == 0
    m = json.loads((tmp_path / "out" / bundles.MANIFEST_NAME).read_text())
    assert m["training_complete"] and m["source_examples_seen"] == 40 and len(m["streaming_data_digest"]) == 64
    out2 = tmp_path / "lora"
    argv = _argv(tmp_path, "--max_steps", "2", "--lora", "--lora_rank", "4", "--lora_save_adapter_only")
    argv[argv.index("--output_dir") + 1] = str(out2)
    assert runner.main(argv) == 0
    cfg = json.loads((out2 / "adapter_config.json").read_text())
    assert cfg["r"] == 4 and cfg["lora_alpha"] == 4 and cfg["peft_type"] == "LORA"
    keys = st.read_header(out2 / "adapter_model.safetensors")[0]
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.weight" in keys
    assert json.loads((out2 / bundles.MANIFEST_NAME).read_text())["artifact_kind"] == "peft-adapter"


def test_pure_helpers():
    assert runner.prepared_streaming_limits(10, 4, 1.5, -1) == (4, 2)
    assert runner.prepared_streaming_limits(2, 8, 0.25, -1) == (1, 1)
    assert runner.prepared_streaming_limits(10, 4, 0, 7) == (7, None)
    assert [runner.buffered_streaming_schedule_total(n) for n in (0, 1, 19, 20, 100, 101)] == [1, 2, 20, 21, 105, 107]
    pos = [runner.streaming_schedule_position(s, e, 3) for e, s in ((0, 0), (0, 2), (0, 3), (0, 5), (1, 0), (2, 0), (2, 9))]
    assert pos == [0, 2, 3, 3, 3, 6, 9]
    assert runner.project_streaming_progress_total(5, 1, 3) == 15 and runner.project_streaming_progress_total(10, 2, 3) == 15
    assert runner.project_streaming_progress_total(14, 3, 3) == 14


def test_profile_steps_times_steps_after_the_warm_up_ones(tmp_path):
    from causal_trainer_dev_b200.training.logging import StepProfiler

    assert runner.main(_argv(tmp_path, "--max_steps", "5", "--profile_steps", "2")) == 0
    report = json.loads((tmp_path / "out" / "profile_steps.json").read_text())
    assert report["profiled_steps"] == 2 and report["skipped_steps"] == 2 and report["clock"].startswith("host clock")
    assert report["ms_per_step_min"] <= report["ms_per_step"] <= report["ms_per_step_max"]
    assert report["tokens_per_second"] > 0 and report["mfu"] > 0
    assert bundles.find_latest_checkpoint(tmp_path / "out", json.loads(
        (tmp_path / "out" / bundles.MANIFEST_NAME).read_text())["training_signature"]) is not None
    idle = StepProfiler(0, None, tokens_per_step=1, flops_per_token=1.0, n_gpus=1)
    idle.begin(); idle.end()
    assert idle.finish() is None
    short = StepProfiler(3, None, tokens_per_step=8, flops_per_token=1.0, n_gpus=1, skip=1)
    for _ in range(2):
        short.begin(); short.end()
    assert short.finish()["profiled_steps"] == 1


def test_training_from_a_prepared_artifact_materialised_and_streamed(tmp_path):
    from causal_trainer_dev_b200 import prepare

    base = _argv(tmp_path)
    model, data = base[1], base[3]
    prepared_dir = tmp_path / "prepared"
    manifest = prepare.prepare_dataset(prepare.parse_args([
        "--dataset_name", data, "--tokenizer_name_or_path", model, "--output_dir", str(prepared_dir),
        "--max_sequence_length", "32", "--packing", "--num_shards", "2"]))
    assert manifest.total_rows > 4

    def argv(out, *extra):
        args = list(base)
        args[3] = str(prepared_dir)
        args[5] = str(tmp_path / out)
        return [*args, "--dataset_format", "prepared", *extra]

    assert runner.main(argv("out_prepared", "--max_steps", "3")) == 0
    done = json.loads((tmp_path / "out_prepared" / bundles.MANIFEST_NAME).read_text())
    assert done["global_step"] == done["total_steps"] == 3
    assert runner.main(argv("out_streamed", "--dataset_streaming", "--num_train_epochs", "1", "--no-shuffle")) == 0
    streamed = json.loads((tmp_path / "out_streamed" / bundles.MANIFEST_NAME).read_text())
    assert streamed["global_step"] == streamed["total_steps"] == manifest.total_rows // 2
    assert streamed["source_examples_seen"] == manifest.total_rows and len(streamed["streaming_data_digest"]) == 64
    # a shard that no longer matches its manifest stops the run before any step
    shard = prepared_dir / manifest.shards[0].path
    blob = bytearray(shard.read_bytes())
    blob[len(blob) // 2] ^= 0xFF
    shard.write_bytes(blob)
    with pytest.raises(RuntimeError, match="checksum mismatch"):
        runner.main(argv("out_corrupt", "--max_steps", "1"))


def _chat_data(path, n=24):
    grid = "<|image_1|><|image_2|><|image_3|>\n<|image_4|><|image_5|><|image_6|>"
    rows = []
    for i in range(n):
        reply = f"w{i % 40} {grid} w{(i + 3) % 40}" if i % 2 else f"w{i % 40} w{(i + 1) % 40}"
        rows.append({"messages": [{"role": "user", "content": f"w{(i * 5) % 40} w{(i * 7) % 40}"},
                                  {"role": "assistant", "content": reply}]})
    path.write_text("\n".join(json.dumps(r) for r in rows))
    return path


def test_chat_modes_assistant_only_with_frozen_components_and_maskgit(tmp_path):
    base = _argv(tmp_path)
    base[3] = str(_chat_data(tmp_path / "chat.jsonl"))
    base[base.index("--max_sequence_length") + 1] = "64"
    chat = [*base, "--dataset_text_field", "messages", "--assistant_only_loss", "--max_steps", "3"]

    frozen = list(chat)
    frozen[5] = str(tmp_path / "out_frozen")
    run = runner.TrainingRun(parse_args([*frozen, "--frozen_parameters", "embed|norm"]))
    run.resolve_model(); run.load_data(); run.discover_resume(); run.build_model()
    before = {n: run.params.tensor(n).clone() for n in run.params.hf_names()}
    run.train()
    changed = {n for n in before if not torch.equal(before[n], run.params.tensor(n))}
    assert "model.embed_tokens.weight" not in changed and not any("norm" in n for n in changed)
    assert "lm_head.weight" in changed and "model.layers.0.mlp.up_proj.weight" in changed
    saved = st.load_file(tmp_path / "out_frozen" / "model.safetensors")
    assert torch.equal(saved["model.embed_tokens.weight"], before["model.embed_tokens.weight"])

    mixed = list(chat)
    mixed[5] = str(tmp_path / "out_maskgit")
    assert runner.main([*mixed, "--maskgit_probability", "1.0"]) == 0
    done = json.loads((tmp_path / "out_maskgit" / bundles.MANIFEST_NAME).read_text())
    assert done["global_step"] == 3
    # the MaskGIT probability is part of the run's identity: the plain run cannot resume from it
    plain = list(chat)
    plain[5] = str(tmp_path / "out_maskgit")
    with pytest.raises(ValueError, match="incompatible"):
        runner.main(plain)


def test_two_gloo_ranks_train_the_same_model_as_one_process(tmp_path):
    """Data parallel on CPU ranks: the global batch is split over two processes, the result is the
    single-process model up to summation order."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    # replicated preprocessing: every process packs the whole source, so both runs see the same rows
    # (sharded preprocessing packs per process shard, which legitimately gives other rows)
    single = _argv(tmp_path, "--max_steps", "3", "--preprocessing_mode", "replicated")
    single[single.index("--total_batch_size") + 1] = "4"
    assert runner.main(single) == 0
    want = st.load_file(tmp_path / "out" / "model.safetensors")

    multi = [a for a in single if a != "--no-distributed"]
    multi[5] = str(tmp_path / "out2")
    multi[multi.index("--sharding_axis") + 1] = "2,1,1,1,1"
    import socket

    with socket.socket() as probe:
        probe.bind(("127.0.0.1", 0))
        port = probe.getsockname()[1]
    env = dict(os.environ, PYTHONPATH=f"{root}{os.pathsep}{os.environ.get('PYTHONPATH', '')}", CUDA_VISIBLE_DEVICES="")
    done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "causal_trainer_dev_b200.train",
                           *multi], env=env, capture_output=True, text=True, timeout=600, cwd=str(tmp_path))
    assert done.returncode == 0, done.stderr[-3000:]
    got = st.load_file(tmp_path / "out2" / "model.safetensors")
    assert set(got) == set(want)
    for name in want:
        assert torch.allclose(got[name], want[name], atol=2e-5, rtol=1e-4), name
    manifest = json.loads((tmp_path / "out2" / bundles.MANIFEST_NAME).read_text())
    assert manifest["global_step"] == 3
