"""Worker of the multi-GPU FSDP test (launched by torch.distributed.run)."""
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def lora_over_sharded_base(out_path: str) -> None:
    """Adapter gradients with the frozen base served by the sharded runtime (weights-only mode)
    against the same engine over a local copy of the base."""
    from causal_trainer_dev_b200.api import TrainerConfig
    from causal_trainer_dev_b200.data.synthetic import pretraining_rows
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.lora import LoraState
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.ops import lib
    from causal_trainer_dev_b200.parallel.fsdp import FsdpRuntime
    from causal_trainer_dev_b200.training.engine import LocalProvider
    from causal_trainer_dev_b200.training.lora_engine import LoraLayerwiseEngine
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig

    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = preset("tiny", vocab_size=4096, num_hidden_layers=2)
    tcfg = TrainerConfig(adamw=AdamWConfig(), schedule=ScheduleConfig(1e-3, 0.0, "constant", 0, 10), seed=3)
    runtime = FsdpRuntime(cfg, tcfg, dev, trainable=False)
    assert runtime.m.numel() == 0 and runtime.grad_shards.numel() == 0      # no optimizer or gradient memory
    local = ModelParams(cfg, torch.bfloat16, dev)
    for name, unit in local.units.items():
        unit.data.copy_(runtime.gather_full_unit(name))
    lora = LoraState.init(cfg, 16, seed=4, dtype=torch.bfloat16, device=dev)
    with torch.no_grad():
        gen = torch.Generator(device=dev).manual_seed(9)
        for b in lora.b.values():
            b.normal_(0, 0.05, generator=gen)
    data = pretraining_rows(2 * world, 256, cfg.vocab_size, eos_token_id=2, pad_token_id=0, median_len=80, min_len=8, seed=5)
    mine = {k: torch.from_numpy(v[2 * rank:2 * rank + 2].copy()).to(dev) for k, v in data.items()}
    sharded = LoraLayerwiseEngine(cfg, runtime, lora)
    plain = LoraLayerwiseEngine(cfg, LocalProvider(local, torch.bfloat16), lora)
    nll_s, _ = sharded(mine, 1.0 / 300, True)
    nll_p, _ = plain(mine, 1.0 / 300, True)
    worst = 0.0
    for key in lora.a:
        for gs, gp in zip(sharded.grads[key], plain.grads[key]):
            worst = max(worst, float((gs - gp).norm() / gp.norm().clamp_min(1e-12)))
    again, _ = sharded(mine, 1.0 / 300, True)         # second pass: the gathered weights are still valid
    status = lib.device_status(raise_on_error=False)
    if rank == 0:
        Path(out_path).write_text(json.dumps({"worst": worst, "nll": [float(nll_s), float(nll_p), float(again)],
                                              "status": status}))
    dist.destroy_process_group()


def main() -> None:
    if sys.argv[1] == "lora":
        local = int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        lora_over_sharded_base(sys.argv[2])
        return
    fused = sys.argv[1] == "fused"
    out_path = sys.argv[2]
    steps = int(sys.argv[3]) if len(sys.argv) > 3 else 2
    extra = dict(kv.split("=", 1) for kv in sys.argv[4:])          # clip=0  frozen=lm_head,norm  micro=1
    clip = float(extra.get("clip", "1.0"))
    frozen = tuple(x for x in extra.get("frozen", "").split(",") if x)
    micro = int(extra.get("micro", "2"))
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from causal_trainer_dev_b200.api import Trainer, TrainerConfig
    from causal_trainer_dev_b200.data.synthetic import pretraining_rows
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.ops import lib
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig

    world, rank = dist.get_world_size(), dist.get_rank()
    cfg = preset("tiny", vocab_size=4096, num_hidden_layers=3)
    tcfg = TrainerConfig(micro_batch_rows=micro, adamw=AdamWConfig(weight_decay=0.1, max_grad_norm=clip),
                         schedule=ScheduleConfig(1e-3, 0.0, "constant", 0, 10), fused_collectives=fused, seed=3,
                         force_sharded_runtime=True, frozen=frozen)
    trainer = Trainer(cfg, tcfg)
    before = {name: trainer.runtime.gather_full_unit(name).clone() for name in ("embed", "final", "layer.0")}
    rows = 8
    data = pretraining_rows(rows, 256, cfg.vocab_size, eos_token_id=2, pad_token_id=0, median_len=80, min_len=8, seed=5)
    per = rows // world
    mine = {k: torch.from_numpy(v[rank * per:(rank + 1) * per].copy()).pin_memory() for k, v in data.items()}
    history = [trainer.train_step(mine) for _ in range(steps)]
    status = lib.device_status(raise_on_error=False)
    checksum = float(trainer.runtime.gather_full_unit("layer.1").float().abs().sum())
    from causal_trainer_dev_b200.models.params import unit_layouts

    unchanged = {}
    for lay in unit_layouts(cfg):
        if lay.name in before:
            now = trainer.runtime.gather_full_unit(lay.name)
            for seg in lay.segments:
                sl = slice(seg.offset, seg.offset + seg.numel)
                unchanged[f"{lay.name}/{seg.name}"] = bool(torch.equal(now[sl], before[lay.name][sl]))
    moments = float(trainer.runtime.m.float().abs().sum())
    if rank == 0:
        Path(out_path).write_text(json.dumps({"history": history, "status": status, "checksum": checksum,
                                              "unchanged": unchanged, "moments": moments,
                                              "fuse_adam": bool(trainer.runtime.fuse_adam)}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
