"""Worker of the multi-GPU tensor-parallel tests (launched by torch.distributed.run).

    _tp_worker.py ops   <out.json>                 primitive checks on a tp group of all ranks
    _tp_worker.py train <out.json> <tp> <fused> <steps>
"""
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def run_ops(out_path: str) -> None:
    from causal_trainer_dev_b200.ops import cross_entropy as ce
    from causal_trainer_dev_b200.ops import lib
    from causal_trainer_dev_b200.ops.gemm import gemm
    from causal_trainer_dev_b200.parallel.tp import TpContext

    world, rank = dist.get_world_size(), dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    rows, d, n_out, vocab = 1024 * world, 512, 768, 2048 * world
    tp = TpContext(dist.group.WORLD, dev, rows, d, fused=True)
    gen = torch.Generator(device=dev).manual_seed(17)          # same on every rank
    x_full = (torch.randn((rows, d), generator=gen, device=dev) * 0.5).bfloat16()
    w_col = (torch.randn((world, n_out, d), generator=gen, device=dev) * 0.05).bfloat16()    # per-rank column blocks
    w_row = (torch.randn((d, world * 256), generator=gen, device=dev) * 0.05).bfloat16()     # [d, K_total]
    a_full = (torch.randn((rows, world * 256), generator=gen, device=dev) * 0.5).bfloat16()
    result = {}
    for it in range(3):       # several rounds: ring slots, receive buffers and epochs are reused
        # ---- all-gather -> GEMM
        g = tp.next_slot()
        g.mine.copy_(x_full[tp.rows_slice()])
        full = tp.all_gather(g)
        y = gemm(full, w_col[rank])
        ref = x_full.float() @ w_col[rank].float().t()
        result[f"ag_gemm_{it}"] = _rel(y, ref)
        # transposed consumer (weight gradient shape): waits for the whole operand
        g2 = tp.next_slot()
        g2.mine.copy_(x_full[tp.rows_slice()])
        full2 = tp.all_gather(g2)
        dw = gemm(y, full2, a_mn=True, b_mn=True)
        result[f"ag_wgrad_{it}"] = _rel(dw, y.float().t() @ x_full.float())
        # ---- GEMM -> reduce-scatter by push
        a_loc = a_full[:, rank * 256:(rank + 1) * 256].contiguous()
        w_loc = w_row[:, rank * 256:(rank + 1) * 256].contiguous()
        out = tp.gemm_reduce_scatter(a_loc, w_loc)
        ref_rs = (a_full.float() @ w_row.float().t())[tp.rows_slice()]
        result[f"gemm_rs_{it}"] = _rel(out, ref_rs)
    # ---- vocabulary-parallel cut cross-entropy (forward exchange + pushed dhidden)
    head = (torch.randn((vocab, d), generator=gen, device=dev) * 0.05).bfloat16()
    targets = torch.randint(0, vocab, (rows,), generator=gen, device=dev)
    weights = (torch.rand((rows,), generator=gen, device=dev) > 0.3).float()
    vl = vocab // world
    local_t = targets.to(torch.int32) - rank * vl
    local_t = torch.where((local_t >= 0) & (local_t < vl), local_t, torch.full_like(local_t, -1))
    g = tp.next_slot()
    g.mine.copy_(x_full[tp.rows_slice()])
    hidden = tp.all_gather(g)
    head_loc = head[rank * vl:(rank + 1) * vl].contiguous()
    nll, wsum, lse, coef = ce.cut_ce_forward(hidden, head_loc, local_t, weights, 0.01, exchange=tp)
    logits = x_full.float() @ head.float().t()
    ref_lse = torch.logsumexp(logits, dim=1)
    ref_nll = ((ref_lse - logits.gather(1, targets[:, None])[:, 0]) * weights).sum()
    result["ce_lse"] = float((lse - ref_lse).abs().max())
    result["ce_nll"] = abs(float(nll) - float(ref_nll)) / float(ref_nll)
    push = tp.begin_push()
    _, dhead = ce.cut_ce_backward(hidden, head_loc, local_t, lse, coef, chunk_rows=512, push=push)
    dh = tp.finish_push(push)
    p = torch.softmax(logits, dim=1)
    p[torch.arange(rows, device=dev), targets] -= 1.0
    dlog = p * (weights * 0.01)[:, None]
    result["ce_dhidden"] = _rel(dh, (dlog @ head.float())[tp.rows_slice()])
    result["ce_dhead"] = _rel(dhead, (dlog.t() @ x_full.float())[rank * vl:(rank + 1) * vl])
    # ---- vocabulary-parallel embedding
    ids = torch.randint(0, vocab, (rows,), generator=gen, device=dev)
    emb = tp.embed_lookup(ids, head_loc, vocab)
    result["embed"] = float((emb.float() - head[ids][tp.rows_slice()].float()).abs().max())
    torch.cuda.synchronize()
    result["status"] = lib.device_status(raise_on_error=False)
    gathered = [None] * world
    dist.all_gather_object(gathered, result)
    if rank == 0:
        Path(out_path).write_text(json.dumps(gathered))


def run_train(out_path: str, tp: int, fused: bool, steps: int, kv_heads: int = 2, sp: int = 1,
              seq: int = 256, layouts: tuple[str, ...] = ("contiguous",)) -> None:
    from causal_trainer_dev_b200.api import Trainer, TrainerConfig
    from causal_trainer_dev_b200.data.synthetic import pretraining_rows
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.ops import lib
    from causal_trainer_dev_b200.training.optimizer import AdamWConfig, ScheduleConfig

    rank = dist.get_rank()
    cfg = preset("tiny", vocab_size=4096, num_hidden_layers=3, intermediate_size=512, num_key_value_heads=kv_heads)
    result = {}
    for layout in layouts:
        tcfg = TrainerConfig(micro_batch_rows=2, adamw=AdamWConfig(weight_decay=0.1, max_grad_norm=1.0),
                             schedule=ScheduleConfig(1e-3, 0.0, "constant", 0, 10), fused_collectives=fused, seed=3, tp=tp,
                             sp=sp, sp_layout=layout)
        trainer = Trainer(cfg, tcfg)
        rows = 8
        data = pretraining_rows(rows, seq, cfg.vocab_size, eos_token_id=2, pad_token_id=0, median_len=80 if seq == 256 else seq // 3, min_len=8,
                                seed=5)
        per = rows // trainer.data_world
        lo = trainer.data_rank * per
        mine = {k: torch.from_numpy(v[lo:lo + per].copy()).pin_memory() for k, v in data.items()}
        history = [trainer.train_step(mine) for _ in range(steps)]
        key = "history" if layout == layouts[0] else f"history_{layout}"
        result[key] = history
        del trainer
    result["status"] = lib.device_status(raise_on_error=False)
    if rank == 0:
        Path(out_path).write_text(json.dumps(result))


def main() -> None:
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if sys.argv[1] == "ops":
        run_ops(sys.argv[2])
    else:
        run_train(sys.argv[2], int(sys.argv[3]), sys.argv[4] == "fused", int(sys.argv[5]),
                  int(sys.argv[6]) if len(sys.argv) > 6 else 2, int(sys.argv[7]) if len(sys.argv) > 7 else 1,
                  int(sys.argv[8]) if len(sys.argv) > 8 else 256,
                  tuple(sys.argv[9].split(",")) if len(sys.argv) > 9 else ("contiguous",))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
