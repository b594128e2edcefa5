"""The multi-GPU layer's host logic on CPU ranks (gloo, world size 2): row shards with a
global row offset reproduce the unsharded masked softmax, and column/row-sharded MLP
partials summed by all-reduce reproduce the unsharded MLP.  The per-rank arithmetic is the
CPU oracle here; on GPUs the same shard boundaries feed the native kernels."""
import os
import socket

import numpy as np
import pytest

from compiler_b200 import shard
from oracle import oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(7)           # same stream on every rank: replicated inputs
    hidden, ffn, m = 32, 96, 10
    x = oracle.bf16_round(rng.standard_normal((m, hidden)).astype(np.float32))
    wg = oracle.bf16_round(rng.normal(0, 0.2, (hidden, ffn)).astype(np.float32))
    wu = oracle.bf16_round(rng.normal(0, 0.2, (hidden, ffn)).astype(np.float32))
    wd = oracle.bf16_round(rng.normal(0, 0.2, (ffn, hidden)).astype(np.float32))
    lo, hi = shard.column_range(ffn, rank, world)
    partial = oracle.swiglu_mlp_ref(x, wg[:, lo:hi], wu[:, lo:hi], wd[lo:hi])
    t = torch.from_numpy(partial.copy())
    for clo, chi in shard.row_chunks(m, 3):  # chunked all-reduce, like the GPU path
        dist.all_reduce(t[clo:chi])
    # row-sharded masked softmax with the global row offset
    rows, cols = 12, 7
    xs = rng.standard_normal((rows, cols))
    rlo, rhi = shard.block_range(rows, rank, world)
    mine = oracle.masked_softmax_ref(xs[rlo:rhi], row_offset=rlo)
    gathered = [torch.zeros((shard.block_range(rows, r, world)[1]
                             - shard.block_range(rows, r, world)[0], cols), dtype=torch.float64)
                for r in range(world)]
    dist.all_gather(gathered, torch.from_numpy(mine.copy()))
    if rank == 0:
        np.save(os.path.join(out_dir, "mlp.npy"), t.numpy())
        np.save(os.path.join(out_dir, "softmax.npy"), torch.cat(gathered).numpy())
        np.save(os.path.join(out_dir, "mlp_ref.npy"), oracle.swiglu_mlp_ref(x, wg, wu, wd))
        np.save(os.path.join(out_dir, "softmax_ref.npy"), oracle.masked_softmax_ref(xs, 0))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_world_size_2_shards_reproduce_the_unsharded_oracle(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    np.testing.assert_allclose(np.load(tmp_path / "mlp.npy"), np.load(tmp_path / "mlp_ref.npy"),
                               rtol=1e-12, atol=1e-12)
    np.testing.assert_array_equal(np.load(tmp_path / "softmax.npy"),
                                  np.load(tmp_path / "softmax_ref.npy"))
