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


def _launch(mode: str, nproc: int, tmp_path: Path, port: int, *extra: str) -> dict:
    out = tmp_path / f"{mode}-{port}.json"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "_fsdp_worker.py"), mode,
           str(out), "3", *extra]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    return json.loads(out.read_text())


def _single_gpu_history(steps: int, clip: float = 1.0, frozen: tuple = ()) -> list[dict]:
    from causal_trainer_dev_b200.api import Trainer, TrainerConfig
    from causal_trainer_dev_b200.data.synthetic import pretraining_rows
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig

    cfg = preset("tiny", vocab_size=4096, num_hidden_layers=3)
    tcfg = TrainerConfig(micro_batch_rows=2, adamw=AdamWConfig(weight_decay=0.1, max_grad_norm=clip),
                         schedule=ScheduleConfig(1e-3, 0.0, "constant", 0, 10), seed=3, frozen=frozen)
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


N = min(2, torch.cuda.device_count())      # the same checks on one GPU (a group of one) and on two


def test_sharded_runtime_matches_the_plain_step(cuda_lib, tmp_path):
    fused = _launch("fused", N, tmp_path, 29613)
    nccl = _launch("nccl", N, tmp_path, 29614)
    single = _single_gpu_history(3)
    assert fused["status"] == [0, 0, 0, 0] and not fused["fuse_adam"]
    for a, b, c in zip(fused["history"], nccl["history"], single):
        assert a["token_count"] == b["token_count"] == c["token_count"]
        assert abs(a["loss"] - b["loss"]) < 2e-2 and abs(a["loss"] - c["loss"]) < 5e-2
        assert abs(a["grad_norm"] - b["grad_norm"]) / b["grad_norm"] < 5e-2
    assert abs(fused["checksum"] - nccl["checksum"]) / nccl["checksum"] < 1e-2
    # every matrix was trained (a norm scale of 1.0 does not move in bf16 under updates this small)
    assert not any(same for key, same in fused["unchanged"].items() if key.split("/")[1] not in ("ln1", "ln2", "norm"))


def test_adamw_inside_the_reduce_kernel_when_clipping_is_off(cuda_lib, tmp_path):
    """``max_grad_norm = 0``: the fused path updates parameters and moments in the reduce-scatter
    kernel; the NCCL variant of the same schedule reduces first and sweeps afterwards."""
    for port, micro in ((29615, "micro=8"), (29625, "micro=2")):      # one micro-batch per step; fp32 accumulation
        fused = _launch("fused", N, tmp_path, port, "clip=0", micro)
        nccl = _launch("nccl", N, tmp_path, port + 1, "clip=0", micro)
        assert fused["fuse_adam"] and not nccl["fuse_adam"] and fused["status"] == [0, 0, 0, 0]
        for a, b in zip(fused["history"], nccl["history"]):
            assert abs(a["loss"] - b["loss"]) < 2e-2 and abs(a["grad_norm"] - b["grad_norm"]) / b["grad_norm"] < 5e-2
        assert fused["history"][-1]["loss"] < fused["history"][0]["loss"]
        assert abs(fused["checksum"] - nccl["checksum"]) / nccl["checksum"] < 1e-2
        assert abs(fused["moments"] - nccl["moments"]) / nccl["moments"] < 2e-2


def test_frozen_components_on_the_sharded_runtime(cuda_lib, tmp_path):
    got = _launch("fused", N, tmp_path, 29617, "frozen=lm_head,norm")
    single = _single_gpu_history(3, frozen=("lm_head", "norm"))
    assert got["status"] == [0, 0, 0, 0]
    for key, same in got["unchanged"].items():
        # bit-identical where frozen (no weight decay either), trained elsewhere
        assert same == (key.split("/")[1] in ("lm_head", "norm", "ln1", "ln2")), key
    for a, c in zip(got["history"], single):
        assert abs(a["loss"] - c["loss"]) < 5e-2 and abs(a["grad_norm"] - c["grad_norm"]) / c["grad_norm"] < 5e-2


def test_adapter_training_over_a_sharded_frozen_base(cuda_lib, tmp_path):
    got = _launch("lora", N, tmp_path, 29618)
    assert got["status"] == [0, 0, 0, 0]
    assert got["worst"] < 2e-2                            # same adapter gradients as over a local base
    assert abs(got["nll"][0] - got["nll"][1]) < 1e-3 * abs(got["nll"][1]) and got["nll"][0] == got["nll"][2]
