"""Multi-GPU paths on real devices (skipped below 2 GPUs): the tensor-parallel SwiGLU MLP
against the unsharded oracle, and row-sharded masked softmax with global row offsets.
Each rank is a child process (torch.distributed, NCCL), launched the way bench.py is."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r'''
import os, sys, traceback
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["B200_REPO"])
from compiler_b200 import ops, shard, tp_mlp
from compiler_b200.runtime import abi
from oracle import oracle

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
def _report(kind, value, tb):
    sys.stderr.write(f"[rank {rank}] " + "".join(traceback.format_exception(kind, value, tb))[-1500:] + "\n")
    sys.stderr.flush()
sys.excepthook = _report
torch.cuda.set_device(rank)
abi.check(abi.lib().b200_set_device(rank))
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))

def bf16(a):
    return torch.from_numpy(oracle.bf16_round(a.astype(np.float32))).to(torch.bfloat16).cuda()

rng = np.random.default_rng(5)                      # same stream on every rank
hidden, ffn, m = 512, 1792, 300
x = oracle.bf16_round(rng.standard_normal((m, hidden)).astype(np.float32))
wg = oracle.bf16_round(rng.normal(0, 0.05, (hidden, ffn)).astype(np.float32))
wu = oracle.bf16_round(rng.normal(0, 0.05, (hidden, ffn)).astype(np.float32))
wd = oracle.bf16_round(rng.normal(0, 0.05, (ffn, hidden)).astype(np.float32))
lo, hi = shard.column_range(ffn, rank, world)
mlp = tp_mlp.TensorParallelMLP(bf16(wg[:, lo:hi]).contiguous(), bf16(wu[:, lo:hi]).contiguous(),
                               bf16(wd[lo:hi]).contiguous(), chunks=3)
y = torch.empty((m, hidden), device="cuda", dtype=torch.bfloat16)
for _ in range(2):                                   # second call reuses the scratch buffer
    mlp.forward(bf16(x), y)
torch.cuda.synchronize()
ops.device_status(torch.cuda.current_stream().cuda_stream)
ref = oracle.swiglu_mlp_ref(x, wg, wu, wd)
oracle.compare(y.float().cpu().numpy().astype(np.float64), ref, 2e-2, 2e-2, name="tp mlp")

# the same MLP with the reduce-scatter fused into the down-projection's epilogue (peer stores)
mp = 256 * world
xp = oracle.bf16_round(rng.standard_normal((mp, hidden)).astype(np.float32))
peer = tp_mlp.TensorParallelMLP(bf16(wg[:, lo:hi]).contiguous(), bf16(wu[:, lo:hi]).contiguous(),
                                bf16(wd[lo:hi]).contiguous(), collective="peer")
yp = torch.empty((mp, hidden), device="cuda", dtype=torch.bfloat16)
for _ in range(3):
    peer.forward(bf16(xp), yp)
torch.cuda.synchronize()
ops.device_status(torch.cuda.current_stream().cuda_stream)
oracle.compare(yp.float().cpu().numpy().astype(np.float64), oracle.swiglu_mlp_ref(xp, wg, wu, wd),
               2e-2, 2e-2, name="tp mlp (peer)")

# the benchmark's shape (CTA-pair GEMMs, 256-row tiles, every collective): a spread of rows of
# each rank's own output against the float64 oracle of the unsharded MLP
hidden, ffn, m = 4096, 14336, 4096
rng_b = np.random.default_rng(6)
xb = oracle.bf16_round(rng_b.standard_normal((m, hidden), dtype=np.float32))
wgb = oracle.bf16_round(rng_b.standard_normal((hidden, ffn), dtype=np.float32) * np.float32(0.02))
wub = oracle.bf16_round(rng_b.standard_normal((hidden, ffn), dtype=np.float32) * np.float32(0.02))
wdb = oracle.bf16_round(rng_b.standard_normal((ffn, hidden), dtype=np.float32) * np.float32(0.02))
lo, hi = shard.column_range(ffn, rank, world)
block = m // world
sel = sorted({r for k in range(world) for r in (k * block, (k + 1) * block - 1)} | {127, 128, 255, 256})
expected = np.zeros((len(sel), hidden))
for c0 in range(0, ffn, 2048):                       # column blocks bound the float64 copies
    cols_ = slice(c0, c0 + 2048)
    expected += oracle.swiglu_mlp_ref(xb[sel], wgb[:, cols_], wub[:, cols_], wdb[cols_])
shards = [bf16(t).contiguous() for t in (wgb[:, lo:hi], wub[:, lo:hi], wdb[lo:hi])]
dxb = bf16(xb)
failures = []
for collective, options in (("nccl", {}), ("peer", {}), ("nvls", {"overlap_blocks": 0}),
                            ("pull", {"overlap_blocks": 0}), ("pull", {}),
                            ("pull", {"overlap_blocks": 4}), ("nvls", {"overlap_blocks": 4}),
                            ("pull", {"overlap_blocks": 1}),
                            ("nvls", {"partial_dtype": torch.float32, "chunks": 2})):
    try:
        big = tp_mlp.TensorParallelMLP(*shards, collective=collective, **options)
        for _ in range(3):
            yb = big.forward(dxb, None)
    except RuntimeError as exc:
        if collective == "nvls" and "multicast" in str(exc):
            print(f"rank {rank}: nvls unavailable ({exc})")
            continue
        raise
    torch.cuda.synchronize()
    # a mismatch is reported after the process group is torn down: no rank leaves while its
    # memory is still bound to the symmetric / multicast buffers the others use
    try:
        ops.device_status(torch.cuda.current_stream().cuda_stream)
        oracle.compare(yb[sel].float().cpu().numpy().astype(np.float64), expected, 2e-2, 2e-2,
                       name=f"tp mlp at the benchmark shape ({collective})")
    except Exception as exc:
        failures.append(f"{collective} {options}: {exc}")
    dist.barrier()
    del big

rows, cols = 64, 4000                                # row shards of one masked softmax
xs = (rng.standard_normal((rows * world, cols)) * 2).astype(np.float16)
rlo, rhi = shard.block_range(rows * world, rank, world)
dx = torch.from_numpy(xs[rlo:rhi]).cuda()
dy = torch.empty_like(dx)
ops.softmax(dx, dy, causal_mod=True, row_offset=rlo, stream=torch.cuda.current_stream().cuda_stream)
full = oracle.masked_softmax_ref(xs, 0)
oracle.compare(dy.float().cpu().numpy().astype(np.float64), full[rlo:rhi], 1e-2, 1e-2, name="softmax shard")
dist.barrier()
torch.cuda.synchronize()
dist.destroy_process_group()
if failures:
    sys.stderr.write(f"[rank {rank}] " + " | ".join(failures)[-1500:] + "\n")
    sys.exit(1)
print(f"rank {rank} ok")
'''


def _gpu_count():
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:  # noqa: BLE001
        return 0


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_mlp_and_row_shards(world, tmp_path):
    if _gpu_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, B200_REPO=str(ROOT), NCCL_NVLS_ENABLE="0")
    result = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
         "--master-addr", "127.0.0.1", "--master-port", str(29500 + world), str(script)],
        capture_output=True, text=True, env=env, timeout=540)
    failures = "\n".join(line for line in result.stderr.splitlines() if line.startswith("[rank"))
    assert result.returncode == 0, failures[-4000:] + result.stdout[-1500:] + result.stderr[-1500:]
    assert result.stdout.count(" ok") == world
