"""Host-side pieces of the headline benchmark script: the reference arm's line and the clock sampler."""
import importlib.util
import json
import os
import stat
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_reference_arm_prints_one_json_line_and_exits_zero():
    done = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                           "--warmup", "3"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    record = json.loads(lines[0])
    assert record["impl"] == "reference" and record["unavailable"].startswith("unavailable on this box")


def test_clock_sampler_reads_median_clock_and_active_reasons(tmp_path, monkeypatch):
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/sh\n"
                    "echo '0, 1500, 1965, 990.1, 0x4, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1410, 1965, 1001.5, 0x4, Not Active, Not Active, Not Active, Active'\n"
                    "echo '0, 1605, 1965, 870.0, 0x0, Not Active, Not Active, Not Active, Not Active'\n"
                    "echo 'garbage line'\n"
                    "exec sleep 30\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}{os.pathsep}{os.environ['PATH']}")
    sampler = _bench().ClockSampler(0)
    sampler.start()
    deadline = time.time() + 10
    while time.time() < deadline and Path(sampler.path).read_text().count("\n") < 4:
        time.sleep(0.05)
    clocks = sampler.stop()
    assert clocks["sm_mhz"] == 1500 and clocks["sm_max_mhz"] == 1965 and clocks["samples"] == 3
    assert clocks["reasons"] == ["sw_power_cap"]


def test_clock_sampler_without_nvidia_smi_reports_nothing(tmp_path, monkeypatch):
    monkeypatch.setenv("PATH", str(tmp_path))
    sampler = _bench().ClockSampler(0)
    sampler.start()
    assert sampler.stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}


def test_named_configurations_generate_rows_of_the_named_shape():
    import numpy as np

    from causal_trainer_dev_b200.benchmarks import configs

    assert set(configs.CONFIGS) == {"llama8b-pretrain", "qwen7b-sft-fsdp4tp2", "llama8b-moba32k-fsdp2tp4",
                                    "qwen1.5b-maskgit-fsdp8", "llama8b-moba32k-one-document",
                                    "llama8b-moba128k-one-document"}
    for name, rows, seq in (("llama8b-pretrain", 2, 1024), ("qwen7b-sft-fsdp4tp2", 2, 1024),
                            ("llama8b-moba32k-fsdp2tp4", 1, 4096), ("qwen1.5b-maskgit-fsdp8", 2, 4096),
                            ("llama8b-moba32k-one-document", 1, 4096)):
        bc = configs.CONFIGS[name]
        cfg = configs.model_of(bc)
        data = bc.make_rows(cfg, rows, seq, 3)
        assert data["input_ids"].shape == (rows, seq) and int(data["input_ids"].max()) < cfg.vocab_size
        executed = configs.executed_flops_per_token(cfg, data, seq)
        assert 0 < executed <= cfg.flops_per_token(seq) * 1.001      # segment isolation never adds work
        if name == "qwen7b-sft-fsdp4tp2":
            assert 0 < data["loss_weights"].mean() < 0.8              # assistant spans only
        if name == "llama8b-moba32k-fsdp2tp4":
            assert sorted(set(data["segment_ids"][0].tolist())) == [1, 2, 3, 4]
        if name == "llama8b-moba32k-one-document":
            assert set(data["segment_ids"][0].tolist()) == {1}
        if name == "qwen1.5b-maskgit-fsdp8":
            mask_id = 151936 + 16384
            masked = data["input_ids"] == mask_id
            assert masked.any() and (data["prediction_weights"][masked] == 1).all()
            assert (data["attention_end"] >= np.arange(seq)[None, :]).all()
            grid = data["attention_end"] > np.arange(seq)[None, :]
            # no next-token target inside a bidirectional grid: only the masked codes carry weight there
            assert (data["prediction_weights"][grid & ~masked] == 0).all()


def test_data_path_benchmark_reports_both_arms_and_checks_their_outputs():
    from causal_trainer_dev_b200.benchmarks import data_bench

    docs, tokens = data_bench._documents(300, 512, seed=2)
    for case in (data_bench.packing_case, data_bench.streaming_case, data_bench.batching_case):
        result = case(docs, tokens, 512)
        assert result["mtokens_per_s"] > 0 and result["rows"] > 0
        if "reference" in result:                    # the reference package is not installed beside the repository
            assert result["reference"].startswith("unavailable")
        else:                                        # same input through the reference's own functions
            assert result.get("identical_rows", True) and result.get("identical_last_batch_digest", True)
            assert result.get("identical_first_batch", True)
            assert result["reference_mtokens_per_s"] > 0
