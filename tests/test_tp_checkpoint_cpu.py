"""Checkpoint load and export of tensor-parallel x FSDP sharded parameters, on Gloo ranks.

Four CPU processes (fsdp=2 x tp=2) each fill their shards from a full checkpoint, reading only
their windows, and export the model again through bounded gather rounds; the exported file must
equal the original bit for bit.  Also checks the slicing helpers against each other.
"""
import os
import subprocess
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[1]

WORKER = r'''
import sys
from pathlib import Path
import torch
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from causal_trainer_dev_b200.checkpointing import huggingface as hfio
from causal_trainer_dev_b200.models.config import preset
from causal_trainer_dev_b200.models.params import unit_layouts
from causal_trainer_dev_b200.parallel import runtime as rt
from causal_trainer_dev_b200.parallel.tp import tp_local_config

src, dst = Path(sys.argv[2]), Path(sys.argv[3])
dist.init_process_group("gloo")
rank = dist.get_rank()
tp, fsdp = 2, 2
full = preset("tiny", vocab_size=512, num_hidden_layers=2, intermediate_size=384, attention_bias=True,
              num_key_value_heads=int(sys.argv[4]))
local = tp_local_config(full, tp)


class Unit:
    def __init__(self, layout, padded, shard, off):
        self.layout, self.padded, self.shard_elems, self.arena_offset = layout, padded, shard, off


class FakeRuntime:
    """The geometry of parallel.fsdp.FsdpRuntime on CPU tensors."""
    def __init__(self):
        self.cfg, self.full_cfg = local, full
        self.tp_world, self.tp_rank = tp, rank % tp
        self.world, self.rank = fsdp, rank // tp
        self.units, off, grain = {}, 0, fsdp * 64
        for lay in unit_layouts(local):
            padded = (lay.numel + grain - 1) // grain * grain
            self.units[lay.name] = Unit(lay, padded, padded // fsdp, off)
            off += padded // fsdp
        self.arena = torch.zeros(off, dtype=torch.bfloat16)

    def shard_view(self, name, of=None):
        u = self.units[name]
        return (self.arena if of is None else of)[u.arena_offset:u.arena_offset + u.shard_elems]


r = FakeRuntime()
hfio.load_sharded_parameters(src, r)
hfio.export_hf_checkpoint(dst, hfio.TensorSource(full, runtime=r), checkpoint_id="00000000-0000-4000-8000-000000000000")
rt.sync_processes("exported")
print("DONE", rank)
dist.destroy_process_group()
'''


import pytest


@pytest.mark.parametrize("kv_heads", [2, 1])
def test_tp_fsdp_load_and_export_roundtrip(tmp_path, kv_heads):
    from causal_trainer_dev_b200.checkpointing import huggingface as hfio
    from causal_trainer_dev_b200.checkpointing import safetensors_io as st
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.params import ModelParams

    cfg = preset("tiny", vocab_size=512, num_hidden_layers=2, intermediate_size=384, attention_bias=True,
                 num_key_value_heads=kv_heads)
    params = ModelParams.init_random(cfg, seed=4)
    for name, t in params.named_tensors():      # biases and norm scales that are not constant
        if t.dim() == 1:
            t.copy_(torch.randn(t.shape).bfloat16())
    src, dst = tmp_path / "src", tmp_path / "dst"
    hfio.export_hf_checkpoint(src, hfio.TensorSource(cfg, params=params),
                              checkpoint_id="00000000-0000-4000-8000-000000000000")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4",
                          "--master-addr", "127.0.0.1", "--master-port", str(29877 + kv_heads), str(script), str(ROOT),
                          str(src), str(dst), str(kv_heads)], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-3000:]
    a, b = st.load_file(src / "model.safetensors"), st.load_file(dst / "model.safetensors")
    assert list(a) == list(b)
    for name in a:
        assert torch.equal(a[name], b[name]), name
    assert (src / "model.safetensors").read_bytes() == (dst / "model.safetensors").read_bytes()


def test_tp_window_agrees_with_unit_slicing():
    from causal_trainer_dev_b200.checkpointing.huggingface import tp_window
    from causal_trainer_dev_b200.models.config import preset
    from causal_trainer_dev_b200.models.params import ModelParams
    from causal_trainer_dev_b200.parallel.tp import slice_unit_tensor, tp_local_config

    cfg = preset("tiny", vocab_size=512, num_hidden_layers=1, intermediate_size=384, attention_bias=True,
                 num_key_value_heads=1)
    full = ModelParams.init_random(cfg, seed=1, dtype=torch.float32)
    tp = 2
    local_cfg = tp_local_config(cfg, tp)
    for r in range(tp):
        local = ModelParams(local_cfg, torch.float32)
        for uname, unit in local.units.items():
            for seg in unit.layout.segments:
                unit.view(seg.name).copy_(slice_unit_tensor(seg.name, full.units[uname].view(seg.name), cfg, tp, r))
        for name, t in local.named_tensors():
            row0, rows, col0, cols, kind = tp_window(name, cfg, tp, r)
            want = full.tensor(name)
            want = want[row0:row0 + rows] if want.dim() == 1 else want[row0:row0 + rows, col0:col0 + cols]
            if kind == "rep":
                want = full.tensor(name)
            assert torch.equal(t, want), (name, r)
