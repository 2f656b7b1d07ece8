"""FSDP over NVLink peer memory (fused pull collectives) against the single-GPU step and the NCCL variant."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _launch(mode: str, nproc: int, tmp_path: Path, port: int) -> dict:
    out = tmp_path / f"{mode}.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "_fsdp_worker.py"), mode,
           str(out), "3"]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return json.loads(out.read_text())


def _single_gpu_history(steps: int) -> list[dict]:
    from causal_trainer_dev_b200.api import Trainer, TrainerConfig
    from causal_trainer_dev_b200.data.synthetic import pretraining_rows
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig

    cfg = preset("tiny", vocab_size=4096, num_hidden_layers=3)
    tcfg = TrainerConfig(micro_batch_rows=2, adamw=AdamWConfig(weight_decay=0.1, max_grad_norm=1.0),
                         schedule=ScheduleConfig(1e-3, 0.0, "constant", 0, 10), seed=3)
    trainer = Trainer(cfg, tcfg)
    data = pretraining_rows(8, 256, cfg.vocab_size, eos_token_id=2, pad_token_id=0, median_len=80, min_len=8, seed=5)
    batch = {k: torch.from_numpy(v).pin_memory() for k, v in data.items()}
    return [trainer.train_step(batch) for _ in range(steps)]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_fsdp_matches_nccl_and_single_gpu(cuda_lib, tmp_path):
    fused = _launch("fused", 2, tmp_path, 29611)
    nccl = _launch("nccl", 2, tmp_path, 29612)
    assert fused["status"] == [0, 0, 0, 0]
    single = _single_gpu_history(3)
    for a, b, c in zip(fused["history"], nccl["history"], single):
        assert a["token_count"] == b["token_count"] == c["token_count"]
        assert abs(a["loss"] - b["loss"]) < 2e-2 and abs(a["loss"] - c["loss"]) < 5e-2
        assert abs(a["grad_norm"] - b["grad_norm"]) / b["grad_norm"] < 5e-2
    assert fused["history"][-1]["loss"] < fused["history"][0]["loss"]
    assert abs(fused["checksum"] - nccl["checksum"]) / nccl["checksum"] < 1e-2
