"""Tensor-parallel SwiGLU MLP: y = (silu(x @ Wg) * (x @ Wu)) @ Wd across the GPUs of one box.

The reference has no multi-device path (its only parallelism is 1/2/4/8 workers of one
process striding over program instances and merging partial results behind a stage
barrier, a100c/plan/partition.py:26-34, a100c/plan/stages.py:668-715).  Here the workers
are GPUs, one process each:

  * Wg / Wu are column-sharded and Wd row-sharded (``shard.column_range``), x is replicated;
  * each rank runs ONE fused kernel for h = silu(x Wg_r) * (x Wu_r) (two accumulators in
    tensor memory, SwiGLU in the epilogue) and one GEMM for its partial y_r = h Wd_r;
  * the partials are summed with an NCCL all-reduce over NVLink -- the merge step of the
    reference's two-phase plan.  The rows of y are split into chunks so the all-reduce of
    chunk i runs on NCCL's stream while the GEMM of chunk i+1 runs on the compute stream.

torch supplies device memory, streams and the process group; the arithmetic is the
library's own kernels.
"""
from __future__ import annotations

from compiler_b200 import ops, shard
from compiler_b200.runtime import abi


class TensorParallelMLP:
    kernels_per_forward = None  # set in __init__: 1 fused up-projection + one GEMM per chunk

    def __init__(self, wg, wu, wd, *, group=None, chunks: int = 4):
        """wg, wu: this rank's [hidden, ffn/tp] column shards; wd: its [ffn/tp, hidden] row
        shard (CUDA bf16/fp16 torch tensors, contiguous)."""
        import torch
        self.torch = torch
        self.wg, self.wu, self.wd = wg, wu, wd
        self.group = group
        self.chunks = max(1, int(chunks))
        self.kernels_per_forward = 1 + self.chunks
        self._h = None

    @classmethod
    def synthetic(cls, hidden, ffn, rank, world, seed=0, dtype=None, chunks=4):
        """Random-normal(0, 0.02) weights; every rank draws only its own shard, from a
        generator seeded by (seed, rank)."""
        import torch
        dtype = dtype or torch.bfloat16
        lo, hi = shard.column_range(ffn, rank, world)
        gen = torch.Generator(device="cuda").manual_seed(seed * 1000 + rank)
        make = lambda *s: (torch.randn(s, generator=gen, device="cuda") * 0.02).to(dtype)  # noqa: E731
        return cls(make(hidden, hi - lo), make(hidden, hi - lo), make(hi - lo, hidden),
                   chunks=chunks)

    def forward(self, x, y):
        """x: [M, hidden] replicated; y: [M, hidden] receives the all-reduced result."""
        torch = self.torch
        import torch.distributed as dist
        m = x.shape[0]
        cols = self.wg.shape[1]
        if self._h is None or self._h.shape != (m, cols) or self._h.dtype != x.dtype:
            self._h = torch.empty((m, cols), device=x.device, dtype=x.dtype)
        stream = torch.cuda.current_stream().cuda_stream
        ops.gemm(x, self.wg, self._h, b2=self.wu, act=abi.ACT_SWIGLU, stream=stream)
        pending = []
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(
            self.group) > 1
        for lo, hi in shard.row_chunks(m, self.chunks):
            ops.gemm(self._h[lo:hi], self.wd, y[lo:hi], stream=stream)
            if distributed:
                pending.append(dist.all_reduce(y[lo:hi], group=self.group, async_op=True))
        for work in pending:
            work.wait()
        return y
