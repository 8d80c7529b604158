"""Host-side logic of the multi-GPU path on CPU: two gloo ranks shard the batch the way bench.py
does (contiguous slices, replicated weights, no collective on the data path), each rank computes
its slice with the CPU oracle standing in for the kernel, and the pieces are checked against the
unsharded result.  Also covers the max-over-ranks reduction of the timing."""
import os
import socket
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np
import torch
import torch.distributed as dist
from bench import shard, algorithmic_bytes
from oracle import oracle_c, oracle_np

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:" + os.environ["MASTER_PORT"], rank=rank, world_size=world)
bs, K, N, DY = 13, 8, 64, 128                      # 13 does not divide evenly
x, w = oracle_np.make_inputs_1d(bs, K, N, DY, seed=5)     # same seed on every rank: replicated weights, global x
lo, hi = shard(bs, world, rank)
y_local = oracle_c.spectral_conv_1d(x[lo:hi], w, double=False)       # the rank's own slice only
# gather for verification only (the timed path has no exchange)
sizes = [None] * world
dist.all_gather_object(sizes, (lo, hi))
pieces = [None] * world
dist.all_gather_object(pieces, y_local)
t = torch.tensor([float(rank + 1)], dtype=torch.float64)
dist.all_reduce(t, op=dist.ReduceOp.MAX)
if rank == 0:
    assert sizes[0][0] == 0 and sizes[-1][1] == bs and all(sizes[i][1] == sizes[i + 1][0] for i in range(world - 1)), sizes
    full = np.concatenate(pieces, axis=0)
    ref = oracle_c.spectral_conv_1d(x, w, double=True)
    mr, l2 = oracle_np.errors(full, ref)
    assert mr < 1e-5 and l2 < 1e-5, (mr, l2)
    assert float(t.item()) == world
    assert sum(algorithmic_bytes(h - l, 1, DY, K, N) for l, h in sizes) == algorithmic_bytes(bs, 1, DY, K, N)
    print("SHARDING_OK", sizes)
dist.barrier()
dist.destroy_process_group()
"""


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_two_rank_batch_sharding_on_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    port = str(_free_port())
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=port, OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), outs
    assert "SHARDING_OK" in outs[0]


def test_shard_partitions_every_batch():
    sys.path.insert(0, ROOT)
    from bench import shard

    for bs in (1, 7, 8, 8192, 8191):
        for world in (1, 2, 3, 4, 8):
            cuts = [shard(bs, world, r) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == bs
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
            sizes = [h - l for l, h in cuts]
            assert max(sizes) - min(sizes) <= 1
