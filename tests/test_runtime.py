import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from causal_trainer_dev_b200.parallel import runtime as rt

ROOT = Path(__file__).resolve().parents[1]


def test_mesh_inference_and_lattice_geometry():
    assert rt.resolve_mesh_shape("-1,1,1,4,1", 8) == (2, 1, 1, 4, 1)
    assert rt.resolve_mesh_shape("1,4,1,2,1", 8) == (1, 4, 1, 2, 1)
    for spec, world in (("-1,-1,1,1,1", 8), ("3,1,1,1,1", 8), ("1,1,1,1", 1), ("-1,1,1,3,1", 8)):
        with pytest.raises(ValueError):
            rt.resolve_mesh_shape(spec, world)
    lat = rt.RankLattice((1, 2, 1, 2, 2), rank=5)
    assert lat.coords() == {"dp": 0, "fsdp": 1, "ep": 0, "tp": 0, "sp": 1}
    assert lat.peers(("tp",)) == [5, 7] and lat.peers(("sp",)) == [4, 5] and lat.peers(("fsdp",)) == [1, 5]
    assert lat.peers(("dp", "fsdp")) == [1, 5] and lat.rank_of(lat.coords(6)) == 6
    with pytest.raises(ValueError, match="ep axis"):
        rt.RankLattice((1, 1, 2, 1, 1), 0).validate()


def test_environment_detection_order():
    d = rt.detect_environment
    assert d(env={}).num_processes == 1
    e = d(env={"RANK": "3", "WORLD_SIZE": "8", "LOCAL_RANK": "3", "MASTER_ADDR": "10.0.0.1", "MASTER_PORT": "1234"})
    assert (e.process_id, e.num_processes, e.coordinator, e.source) == (3, 8, "10.0.0.1:1234", "torchrun")
    assert d(env={"SLURM_PROCID": "2", "SLURM_NTASKS": "4", "SLURM_LOCALID": "2"}).source == "slurm"
    assert d(env={"OMPI_COMM_WORLD_RANK": "1", "OMPI_COMM_WORLD_SIZE": "2"}).source == "openmpi"
    f = d("host:1", 4, 2, "6,7", env={"RANK": "0", "WORLD_SIZE": "1"})
    assert (f.process_id, f.num_processes, f.local_rank, f.source) == (2, 4, 6, "flags")
    with pytest.raises(ValueError):
        d(None, 4, None, env={})


def test_single_process_collectives_are_identities():
    rt.assert_equal(bytes(32), "x")
    rt.raise_if_any_process_error(None, "stage")
    with pytest.raises(KeyError):
        rt.raise_if_any_process_error(KeyError("mine"), "stage")
    cols = {"a": np.arange(6).reshape(3, 2)}
    assert rt.merge_packed_host_arrays(cols) is cols


WORKER = r'''
import os as _os
def say(*parts):
    # one write() per line: lines of different ranks never interleave inside the shared pipe
    _os.write(1, (" ".join(str(p) for p in parts) + "\n").encode())

import sys, numpy as np, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from causal_trainer_dev_b200.parallel import runtime as rt
rt.initialize_distributed()
rank, world = rt.process_index(), rt.process_count()
scenario = sys.argv[2]
if scenario == "merge":
    rows = rank + 1                                  # uneven, rank 0 has 1 row
    local = {"input_ids": np.full((rows, 4), rank, dtype=np.int32), "loss_weights": np.full((rows, 4), rank + 0.1, dtype=np.float32)}
    out = rt.merge_packed_host_arrays(local)
    assert out["input_ids"].shape == (sum(range(1, world + 1)), 4), out["input_ids"].shape
    assert out["input_ids"][:, 0].tolist() == [r for r in range(world) for _ in range(r + 1)]
    assert out["loss_weights"].dtype == np.float32 and np.float32(1.1) == out["loss_weights"][1, 0]   # bit-exact floats
    rt.assert_equal(rt.digest_of({"same": 1}), "flags")
    rt.sync_processes("done")
    say("MERGE-OK", rank)
elif scenario == "error":
    err = ValueError("rank one broke") if rank == 1 else None
    try:
        rt.raise_if_any_process_error(err, "load dataset")
        say("NO-ERROR", rank)
    except ValueError as e:
        say("OWN-ERROR", rank, e)
    except RuntimeError as e:
        say("PEER-ERROR", rank, e)
elif scenario == "mismatch":
    try:
        rt.assert_equal(rt.digest_of({"rank": rank if rank == 2 else 0}), "command-line arguments")
        say("AGREE", rank)
    except RuntimeError as e:
        say("MISMATCH", rank, e)
elif scenario == "zero":
    try:
        rt.raise_if_process_zero_error(OSError("disk full") if rank == 0 else None, "write manifest")
    except OSError as e:
        say("ZERO-OWN", rank)
    except RuntimeError as e:
        say("ZERO-PEER", rank, e)
dist.destroy_process_group()
'''


def _launch(tmp_path, scenario, nproc=3):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, OMP_NUM_THREADS="1")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
                          "--master-addr", "127.0.0.1", "--master-port", str(29700 + hash(scenario) % 200),
                          str(script), str(ROOT), scenario], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    return res.stdout


def test_gloo_ranks_merge_datasets_in_rank_order(tmp_path):
    out = _launch(tmp_path, "merge")
    assert out.count("MERGE-OK") == 3


def test_error_bus_raises_on_every_rank(tmp_path):
    out = _launch(tmp_path, "error")
    assert "OWN-ERROR 1" in out and out.count("PEER-ERROR") == 2 and "NO-ERROR" not in out   # output may interleave
    assert "load dataset failed on process 1" in out and "rank one broke" in out


def test_disagreeing_flags_and_rank_zero_failures_are_seen_everywhere(tmp_path):
    assert _launch(tmp_path, "mismatch").count("MISMATCH") == 3
    out = _launch(tmp_path, "zero")
    assert out.count("ZERO-OWN") == 1 and out.count("ZERO-PEER") == 2 and "disk full" in out   # output may interleave
