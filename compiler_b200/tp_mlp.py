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

Two ways to sum the partials:

  * ``collective="nccl"``: fp32 partials, NCCL all-reduce per row chunk overlapped with the
    next chunk's GEMM, one rounding at the end (the baseline);
  * ``collective="peer"``: the down-projection GEMM's epilogue stores every finished tile
    straight into the memory of the rank that owns those rows (``b200_gemm_scatter_rows``,
    plain peer stores through NVSwitch), so the reduce-scatter half of the all-reduce moves
    while the tensor cores are still busy; after a cross-rank barrier each rank sums its
    ``world`` staged slices and stores the result into every rank's output
    (``b200_reduce_slices_broadcast``), and a second barrier publishes it.  Buffers come from
    ``torch.distributed._symmetric_memory``; only its barrier is used, the data moves in this
    library's kernels.  The staged partials are 16-bit, their sum is taken in fp32 (every
    partial is rounded once, the running sum never).  Needs M to be a multiple of 128 * world;
  * ``collective="nvls"``: every rank writes its 16-bit partial into a symmetric buffer that
    is bound to an NVSwitch multicast object; after a barrier each rank loads the in-switch
    sum of its 1/world share (``b200_multimem_allreduce``: ``multimem.ld_reduce``, fp32
    accumulation, one rounding) and stores it to all ranks at once (``multimem.st``), in
    place; a second barrier publishes it.  No partial crosses a link twice and the GEMM's
    epilogue stores stay local.  The result is returned in the symmetric buffer itself (no
    copy) when ``forward`` gets no ``y``.  Needs NVLS (a multicast pointer from
    ``torch.distributed._symmetric_memory``) and M * hidden to be a multiple of 8 * world;
  * ``collective="pull"``: the same structure without the switch's arithmetic
    (``b200_peer_allreduce``): each rank loads its share of every rank's partial with plain
    peer loads, adds in fp32 and stores the result to every rank.

The nvls and pull paths cut the down-projection into row chunks; the all-reduce of a chunk
carries its own cross-rank barriers (flags in symmetric memory, bounded waits) and runs on a
second stream beside the next chunk's GEMM.

``forward(x, y, mark=...)`` calls ``mark(name)`` after it has enqueued each phase, so a caller
can record a CUDA event per phase on the current stream.
"""
from __future__ import annotations

from compiler_b200 import ops, shard
from compiler_b200.runtime import abi


class TensorParallelMLP:
    kernels_per_forward = None  # set in __init__: 1 fused up-projection + one GEMM per chunk

    def __init__(self, wg, wu, wd, *, group=None, chunks=None, collective: str = "nccl",
                 partial_dtype=None, comm_ctas: int = 0, row_splits: int = 1,
                 overlap_blocks=None):
        """wg, wu: this rank's [hidden, ffn/tp] column shards; wd: its [ffn/tp, hidden] row
        shard (CUDA bf16/fp16 torch tensors, contiguous).

        ``chunks``: row chunks of the down-projection whose all-reduce overlaps the next
        chunk's GEMM (default: 4 for the nccl path, whose all-reduce runs on NCCL's own
        stream and copy engines; 1 for the nvls and pull paths, where an all-reduce kernel
        beside the GEMM took more from it than the overlap gave back on 2 GPUs).  ``partial_dtype`` (peer and nvls paths): the type
        the partial products are staged in -- ``torch.float16`` by default: against bfloat16 it
        keeps three more mantissa bits at the same traffic, which is what keeps the sum of
        ``world`` partials within 2e-2 of the float64 result where bfloat16 partials of
        opposite sign cancel; its range is 65504, so operands whose partial products can
        exceed that need ``torch.float32`` (nvls path only: twice the traffic into the switch,
        the exact sum) -- or the weights' own type.  ``comm_ctas``: grid limit of the
        all-reduce kernel while it runs beside a GEMM (0 = default).  ``row_splits`` (nvls and
        pull paths): run the whole MLP in this many blocks of rows, the all-reduce of a
        block's result on a second stream beside both projections of the next block.
        ``overlap_blocks`` (pull and nvls paths, 1 or more): ONE down-projection launch that counts
        its finished tiles per block of rows, and the all-reduce kernel launched behind it as
        its programmatic dependent: it runs beside the GEMM and takes each block of rows as
        soon as every rank has counted it complete, so only the last block's all-reduce is
        left when the GEMM ends -- no second stream and no extra partial waves.  With 1 the
        all-reduce kernel still becomes resident while the GEMM runs and starts on the whole
        result the moment the GEMM has counted it complete (its launch latency and the wait
        for the peers' kernels to start are hidden), but nothing is reduced early.  0: off.
        None (default): 4 on the pull and nvls paths in a world of up to 4 ranks, where it
        measured faster (0.524 -> 0.510 ms at 2 ranks, 0.333 -> 0.317 ms at 4), otherwise off
        (at 8 ranks a flag barrier per block costs more than the 50 us GEMM can hide)."""
        import torch
        self.torch = torch
        self.wg, self.wu, self.wd = wg, wu, wd
        self.group = group
        if chunks is None:
            chunks = 4 if collective == "nccl" else 1
        self.chunks = max(1, int(chunks))
        if collective not in ("nccl", "peer", "nvls", "pull"):
            raise ValueError("collective must be 'nccl', 'peer', 'nvls' or 'pull'")
        self.collective = collective
        # this library's kernels per forward (NCCL's and the barrier kernels are not counted)
        self.kernels_per_forward = {"nccl": 1 + self.chunks, "peer": 3,
                                    "nvls": 1 + 2 * self.chunks,
                                    "pull": 1 + 2 * self.chunks}[collective]
        self.partial_dtype = torch.float16 if partial_dtype is None else partial_dtype
        if collective in ("peer", "pull") and self.partial_dtype not in (torch.float16,
                                                                         torch.bfloat16):
            raise ValueError(f"collective='{collective}' stages 16-bit partials")
        self.comm_ctas = int(comm_ctas)
        self.row_splits = max(1, int(row_splits))
        if overlap_blocks is None:
            import torch.distributed as dist
            world = (dist.get_world_size(group) if dist.is_available() and dist.is_initialized()
                     else 1)
            overlap_blocks = 4 if (collective in ("pull", "nvls") and 1 < world <= 4
                                   and self.row_splits == 1 and self.chunks == 1) else 0
        self.overlap_blocks = max(0, int(overlap_blocks))
        if self.overlap_blocks > 0 and collective not in ("pull", "nvls"):
            raise ValueError("overlap_blocks needs collective='pull' or 'nvls'")
        self._progress = None
        self._epoch = 0
        self._comm_stream = None
        self._h = None
        self._partial = None
        self._peer = None  # (rows, staging, staging handle, y, y handle)
        self._nvls = None  # (key, partial, handle)

    @classmethod
    def synthetic(cls, hidden, ffn, rank, world, seed=0, dtype=None, chunks=None,
                  collective="nccl", **options):
        """Random-normal(0, 0.02) weights; every rank draws only its own shard, from a
        generator seeded by (seed, rank)."""
        import torch
        dtype = dtype or torch.bfloat16
        lo, hi = shard.column_range(ffn, rank, world)
        gen = torch.Generator(device="cuda").manual_seed(seed * 1000 + rank)
        make = lambda *s: (torch.randn(s, generator=gen, device="cuda") * 0.02).to(dtype)  # noqa: E731
        return cls(make(hidden, hi - lo), make(hidden, hi - lo), make(hi - lo, hidden),
                   chunks=chunks, collective=collective, **options)

    def forward(self, x, y=None, mark=None):
        """x: [M, hidden] replicated; y: [M, hidden] receives the all-reduced result.  With
        ``y=None`` the peer and nvls paths return their own symmetric output buffer (valid
        until the next call) and save the copy; the NCCL path allocates one."""
        torch = self.torch
        import torch.distributed as dist
        mark = mark or (lambda name: None)
        m = x.shape[0]
        cols = self.wg.shape[1]
        if self._h is None or self._h.shape != (m, cols) or self._h.dtype != x.dtype:
            self._h = torch.empty((m, cols), device=x.device, dtype=x.dtype)
        stream = torch.cuda.current_stream().cuda_stream
        if self.collective in ("nvls", "pull") and self.row_splits > 1:
            return self._forward_nvls(y, stream, mark, x=x)
        ops.gemm(x, self.wg, self._h, b2=self.wu, act=abi.ACT_SWIGLU, stream=stream)
        mark("up_projection")
        if self.collective == "peer":
            return self._forward_peer(y, stream, mark)
        if self.collective in ("nvls", "pull"):
            return self._forward_nvls(y, stream, mark)
        if y is None:
            y = torch.empty((m, self.wd.shape[1]), device=x.device, dtype=x.dtype)
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(
            self.group) > 1
        if not distributed:
            ops.gemm(self._h, self.wd, y, stream=stream)
            mark("down_projection")
            return y
        # fp32 partials: a 16-bit ring all-reduce rounds the running sum at every hop, which
        # at 4 ranks already exceeds the 2e-2 tolerance against the unsharded result
        if self._partial is None or self._partial.shape != y.shape:
            self._partial = torch.empty(y.shape, device=y.device, dtype=torch.float32)
        pending = []
        for lo, hi in shard.row_chunks(m, self.chunks):
            ops.gemm(self._h[lo:hi], self.wd, self._partial[lo:hi], stream=stream)
            pending.append((lo, hi, dist.all_reduce(self._partial[lo:hi], group=self.group,
                                                    async_op=True)))
        mark("down_projection_chunks_issued")
        for lo, hi, work in pending:
            work.wait()
            y[lo:hi].copy_(self._partial[lo:hi])  # one rounding to the storage type
        mark("all_reduce_tail_and_rounding")
        return y

    # ------------------------------------------------------------------ peer path
    def _peer_buffers(self, m, hidden, dtype, device):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        world = dist.get_world_size(self.group)
        if m % (128 * world):
            raise ValueError(f"collective='peer' needs M ({m}) to be a multiple of {128 * world}")
        if self._peer is None or self._peer[0] != (m, hidden, dtype):
            group = self.group if self.group is not None else dist.group.WORLD
            rows = m // world
            staging = symm_mem.empty((world, rows, hidden), dtype=self.partial_dtype,
                                     device=device)
            staging_h = symm_mem.rendezvous(staging, group=group)
            out = symm_mem.empty((m, hidden), dtype=dtype, device=device)
            out_h = symm_mem.rendezvous(out, group=group)
            self._peer = ((m, hidden, dtype), rows, staging, staging_h, out, out_h)
        return self._peer[1:]

    def _forward_peer(self, y, stream, mark):
        """Down-projection with the reduce-scatter in its epilogue, then sum + broadcast."""
        import ctypes

        import torch.distributed as dist
        m, hidden = self._h.shape[0], self.wd.shape[1]
        rows, staging, staging_h, out, out_h = self._peer_buffers(m, hidden, self._h.dtype,
                                                                   self._h.device)
        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        lib = abi.lib()
        pointer_array = ctypes.c_void_p * world
        staging_ptrs = pointer_array(*[int(p) for p in staging_h.buffer_ptrs])
        out_ptrs = pointer_array(*[int(p) for p in out_h.buffer_ptrs])
        hd = abi.make_tensor(self._h.data_ptr(), self._h.shape, self._h.dtype,
                             tuple(self._h.stride()))
        wd = abi.make_tensor(self.wd.data_ptr(), self.wd.shape, self.wd.dtype,
                             tuple(self.wd.stride()))
        c_like = abi.make_tensor(out.data_ptr(), (m, hidden), staging.dtype)
        abi.check(lib.b200_gemm_scatter_rows(ctypes.byref(hd), ctypes.byref(wd),
                                             ctypes.byref(c_like), staging_ptrs, world, rank,
                                             rows, stream))
        mark("down_projection_scatter")
        staging_h.barrier(channel=0)  # every rank's tiles for my rows have landed
        mark("barrier_partials")
        abi.check(lib.b200_reduce_slices_broadcast(
            staging.data_ptr(), abi.DTYPE_CODES[abi.dtype_name(staging.dtype)],
            abi.DTYPE_CODES[abi.dtype_name(out.dtype)], world, rows, hidden, rank * rows,
            out_ptrs, stream))
        mark("reduce_broadcast")
        out_h.barrier(channel=1)      # every rank's slice is in my output
        mark("barrier_result")
        if y is not None and y.data_ptr() != out.data_ptr():
            y.copy_(out)
            mark("copy_out")
            return y
        return out

    # ------------------------------------------------------------------ in-switch path
    def _nvls_buffers(self, m, hidden, dtype, device):
        """(partial, partial handle, out, out handle, pad pointers): the partial in
        ``partial_dtype``, the result in the operands' type (the same buffer when both are
        16-bit: reduced in place), and the flag arrays of the kernel's own barriers."""
        import ctypes

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        torch = self.torch
        world = dist.get_world_size(self.group)
        if (m * hidden) % (8 * world):
            raise ValueError(f"collective='nvls' needs M * hidden ({m * hidden}) to be a "
                             f"multiple of {8 * world}")
        key = (m, hidden, dtype, self.partial_dtype)
        if self._nvls is None or self._nvls[0] != key:
            group = self.group if self.group is not None else dist.group.WORLD
            partial = symm_mem.empty((m, hidden), dtype=self.partial_dtype, device=device)
            partial_h = symm_mem.rendezvous(partial, group=group)
            if partial.element_size() == 2:
                out, out_h = partial.view(dtype), partial_h
            else:
                out = symm_mem.empty((m, hidden), dtype=dtype, device=device)
                out_h = symm_mem.rendezvous(out, group=group)
            for handle in (partial_h, out_h):
                if self.collective == "nvls" and not int(getattr(handle, "multicast_ptr", 0)
                                                         or 0):
                    raise RuntimeError("symmetric memory has no multicast pointer on this "
                                       "system (NVLS unavailable): use collective='peer'")
            words = abi.lib().b200_signal_pad_bytes() // 4
            pad = symm_mem.empty((words,), dtype=torch.int32, device=device)
            pad.zero_()
            pad_h = symm_mem.rendezvous(pad, group=group)
            torch.cuda.synchronize(device)
            pad_h.barrier(channel=0)  # every rank's flags are zero before anyone signals
            torch.cuda.synchronize(device)
            pads = (ctypes.c_void_p * world)(*[int(p) for p in pad_h.buffer_ptrs])
            self._epoch = 0
            self._nvls = (key, partial, partial_h, out, out_h, pads, pad, pad_h)
        return self._nvls[1:6]

    def _forward_nvls(self, y, stream, mark, x=None):
        """Down-projection into the symmetric partial in row chunks; each chunk's all-reduce
        (in the switch, or over plain peer memory for ``collective="pull"``; with its own
        cross-rank barriers) runs on a second stream beside the next chunk's GEMM."""
        import ctypes

        import torch.distributed as dist
        torch = self.torch
        m, hidden = self._h.shape[0], self.wd.shape[1]
        partial, partial_h, out, out_h, pads = self._nvls_buffers(m, hidden, self._h.dtype,
                                                                  self._h.device)
        world, rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream(device=self._h.device, priority=-1)
        comm = self._comm_stream
        main = torch.cuda.current_stream()
        lib = abi.lib()
        in_code = abi.DTYPE_CODES[abi.dtype_name(partial.dtype)]
        out_code = abi.DTYPE_CODES[abi.dtype_name(out.dtype)]
        pointer_array = ctypes.c_void_p * world
        partial_ptrs = pointer_array(*[int(p) for p in partial_h.buffer_ptrs])
        out_ptrs = pointer_array(*[int(p) for p in out_h.buffer_ptrs])
        # x given: the whole MLP runs block of rows by block of rows (row_splits blocks), so
        # that the all-reduce of a block's result runs beside BOTH projections of the next one
        pieces = self.row_splits if x is not None else self.chunks
        chunks = [c for c in shard.row_chunks(m, pieces)
                  if ((c[1] - c[0]) * hidden) % (8 * world) == 0]
        if sum(hi - lo for lo, hi in chunks) != m:
            chunks = [(0, m)]
        if self.overlap_blocks > 0 and x is None:
            rows = max(256, (m // self.overlap_blocks) // 256 * 256)
            if m % 256 == 0 and (rows * hidden) % (8 * world) == 0:
                if self._progress is None:
                    self._progress = torch.zeros((lib.b200_progress_words(),), device=out.device,
                                                 dtype=torch.int32)
                targets = ops.gemm_progress(self._h, self.wd, partial, rows, self._progress,
                                            stream=stream)
                epoch0 = self._epoch + 1
                self._epoch += len(targets)
                if self.collective == "nvls":
                    ops.multimem_allreduce_blocks(
                        partial_h.multicast_ptr, out_h.multicast_ptr, m * hidden, rows * hidden,
                        self._progress, targets, rank, world, in_dtype=partial.dtype,
                        out_dtype=out.dtype, signal_pads=pads, epoch0=epoch0,
                        ctas=self.comm_ctas, stream=stream)
                else:
                    ops.peer_allreduce_blocks(
                        partial_h.buffer_ptrs, out_h.buffer_ptrs, m * hidden, rows * hidden,
                        self._progress, targets, rank, world, in_dtype=partial.dtype,
                        out_dtype=out.dtype, signal_pads=pads, epoch0=epoch0,
                        ctas=self.comm_ctas, stream=stream)
                mark("down_projection_with_the_all_reduce_beside_it")
                if y is not None and y.data_ptr() != out.data_ptr():
                    y.copy_(out)
                    mark("copy_out")
                    return y
                return out
        overlapped = len(chunks) > 1
        reduce_stream = comm.cuda_stream if overlapped else stream
        for lo, hi in chunks:
            if x is not None:
                ops.gemm(x[lo:hi], self.wg, self._h[lo:hi], b2=self.wu, act=abi.ACT_SWIGLU,
                         stream=stream)
            ops.gemm(self._h[lo:hi], self.wd, partial[lo:hi], stream=stream)
            if overlapped:  # one chunk: nothing to run beside, the all-reduce follows in line
                ready = torch.cuda.Event()
                ready.record(main)
                comm.wait_event(ready)
            else:
                mark("down_projection")
            self._epoch += 1
            if self.collective == "nvls":
                abi.check(lib.b200_multimem_allreduce(
                    int(partial_h.multicast_ptr), in_code, int(out_h.multicast_ptr), out_code,
                    lo * hidden, (hi - lo) * hidden, rank, world, pads, self._epoch,
                    self.comm_ctas, reduce_stream))
            else:
                abi.check(lib.b200_peer_allreduce(
                    partial_ptrs, in_code, out_ptrs, out_code, lo * hidden, (hi - lo) * hidden,
                    rank, world, pads, self._epoch, self.comm_ctas, reduce_stream))
        if overlapped:
            mark("down_projection_chunks_issued")
            done = torch.cuda.Event()
            done.record(comm)
            main.wait_event(done)
            mark("all_reduce_tail")
        else:
            mark("all_reduce_with_its_barriers")
        if y is not None and y.data_ptr() != out.data_ptr():
            y.copy_(out)
            mark("copy_out")
            return y
        return out
