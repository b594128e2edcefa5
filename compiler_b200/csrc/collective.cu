// All-reduce of partial results through NVSwitch (NVLS): the merge step of the
// tensor-parallel MLP.  Every rank holds its partial in a buffer that is bound to one
// multicast address range; a load through that range (multimem.ld_reduce) returns the sum of
// all ranks' copies, added in the switch in fp32, and a store through it (multimem.st) writes
// all ranks' copies at once.  Rank r reduces the r-th share of the range and publishes it, so
// no partial crosses a link twice.  The reference's counterpart is the merge of per-worker
// partial slots behind a stage barrier (a100c/plan/stages.py:278-316, runtime barrier
// a100c/runtime/pool.c:187-190); it has no multi-device form.
//
// The kernel can carry its own stage barriers: CTA b of every rank signals CTA b of every
// other rank through a small symmetric flag array ("signal pad") when it starts -- the
// producer of this rank's partial ran before it on the same stream, so the signal says "my
// partial is complete" -- waits for the others' signals, reduces and publishes its part, and
// signals / waits once more, so that when the kernel has finished on a rank every rank's
// share has landed in that rank's copy.  Every wait is bounded (about two seconds by
// %globaltimer): a rank whose peers never arrive records B200_TIMEOUT in the device status
// word, skips the data phase and returns.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;  // small enough to be resident beside a persistent GEMM CTA
constexpr int kMaxCtas = 512;                 // CTAs a signal pad has flags for
constexpr uint64_t kFlagWaitNs = 2000000000ull;
constexpr uint32_t kSiteStart = 40, kSiteEnd = 41;

__device__ __forceinline__ uint64_t timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const unsigned int *p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys16(const void *p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// 16 bytes of 16-bit partials: the switch adds in fp32 and returns the rounded sum
template <int KIND>
__device__ __forceinline__ uint4 multimem_ld_reduce16(const void *mc) {
  uint4 v;
  if constexpr (KIND == B200_DTYPE_BFLOAT16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  } else {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  }
  return v;
}
__device__ __forceinline__ float4 multimem_ld_reduce_f32(const void *mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st16(void *mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               :: "l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <int OUT> __device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (OUT == B200_DTYPE_BFLOAT16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
  } else {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
  }
}
template <int IN> __device__ __forceinline__ float2 unpack2(uint32_t w) {
  if constexpr (IN == B200_DTYPE_BFLOAT16)
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
  else
    return __half22float2(*reinterpret_cast<const __half2 *>(&w));
}

// One output vector of 8 elements (16 bytes): the in-switch sum of the 8 input elements that
// start at element `e` of the partial, rounded once to the output type.
template <int IN, int OUT>
__device__ __forceinline__ uint4 reduced_vector(const uint8_t *in_mc, int64_t e) {
  if constexpr (IN == B200_DTYPE_FLOAT32) {
    const float4 a = multimem_ld_reduce_f32(in_mc + e * 4);
    const float4 b = multimem_ld_reduce_f32(in_mc + e * 4 + 16);
    return make_uint4(pack2<OUT>(a.x, a.y), pack2<OUT>(a.z, a.w), pack2<OUT>(b.x, b.y),
                      pack2<OUT>(b.z, b.w));
  } else {
    uint4 v = multimem_ld_reduce16<IN>(in_mc + e * 2);
    if constexpr (IN != OUT) {
      uint32_t *w = &v.x;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = unpack2<IN>(w[i]);
        w[i] = pack2<OUT>(f.x, f.y);
      }
    }
    return v;
  }
}

struct SignalPads {
  uint32_t *pad[8];  // pad[k]: rank k's flag array [2][kMaxCtas][8], mapped into this process
};

// Signals every rank and waits for every rank, for this CTA's index.  Returns false when a
// wait ran out.  phase 0 = start of the kernel, 1 = end.
__device__ __forceinline__ bool cross_rank_barrier(const SignalPads &pads, int rank, int world,
                                                   int phase, uint32_t epoch,
                                                   unsigned int *status, uint32_t site) {
  __shared__ int ok_flag[2];
  if (threadIdx.x == 0) ok_flag[phase] = 1;
  __syncthreads();  // also: this CTA's earlier stores are ordered before the signals below
  if ((int)threadIdx.x < world) {
    const int peer = (int)threadIdx.x;
    const size_t slot = ((size_t)phase * kMaxCtas + blockIdx.x) * 8;
    st_release_sys(pads.pad[peer] + slot + rank, epoch);
    const uint32_t *mine = pads.pad[rank] + slot + peer;
    const uint64_t t0 = timer_ns();
    for (uint32_t it = 0;; ++it) {
      // flags only grow; a peer can be at most one epoch ahead
      if ((int32_t)(ld_acquire_sys(mine) - epoch) >= 0) break;
      if ((it & 0x3f) == 0x3f && timer_ns() - t0 > kFlagWaitNs) {
        atomicOr(status, (unsigned)B200_TIMEOUT | (site << 8));
        ok_flag[phase] = 0;
        break;
      }
    }
  }
  __syncthreads();
  return ok_flag[phase] != 0;
}

// vecs output vectors (8 elements each) of this rank's share; the share starts at element
// `first` of both buffers.  Eight reduced loads in flight per thread, then the eight stores.
template <int IN, int OUT, bool SYNC>
__global__ void __launch_bounds__(kThreads)
multimem_allreduce_kernel(const uint8_t *in_mc, uint8_t *out_mc, int64_t first, int64_t vecs,
                          SignalPads pads, int rank, int world, uint32_t epoch,
                          unsigned int *status) {
  if constexpr (SYNC) {
    if (!cross_rank_barrier(pads, rank, world, 0, epoch, status, kSiteStart)) return;
  }
  constexpr int U = 8;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < vecs) v[u] = reduced_vector<IN, OUT>(in_mc, first + (i + u * stride) * 8);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < vecs) multimem_st16(out_mc + (first + (i + u * stride) * 8) * 2, v[u]);
  }
  if constexpr (SYNC) cross_rank_barrier(pads, rank, world, 1, epoch, status, kSiteEnd);
}

// The same all-reduce without the switch's arithmetic: this rank loads its share of every
// rank's partial with plain peer loads (16 bytes each, all ranks' loads of a vector in
// flight together), adds them in fp32 in rank order, rounds once and stores the result into
// every rank's output with plain peer stores.
struct RankPointers {
  void *ptr[8];
};

// This rank's share: vecs output vectors of 8 elements from element `first` on.  U vectors per
// thread and step, W >= world: U x W = 16 peer loads of 16 bytes in flight per thread (the
// links' latency, not the adder, sets the pace: 2 ranks moved 16 MiB each way in 53 us with
// four loads in flight per thread).  COHERENT: the partials were written while this kernel was
// already running (by the GEMM it was launched behind), so the loads must not take the
// read-only path.
template <typename TIn, typename TOut, int U, int W, bool COHERENT>
__device__ __forceinline__ void peer_reduce_share(const RankPointers &partial,
                                                  const RankPointers &out, int64_t first,
                                                  int64_t vecs, int world) {
  constexpr int N = 8;  // elements per 16-byte vector of a 16-bit type
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride * U) {
    vec16<TIn> v[U][W];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t e = first + (i + u * stride) * N;
      if (i + u * stride < vecs) {
#pragma unroll
        for (int w = 0; w < W; ++w)
          if (w < world) {
            const TIn *src = static_cast<const TIn *>(partial.ptr[w]) + e;
            v[u][w].raw = COHERENT ? ld_relaxed_sys16(src) : ld_stream16(src);
          }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (i + u * stride >= vecs) continue;
      const int64_t e = first + (i + u * stride) * N;
      float acc[N];
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = 0.f;
#pragma unroll
      for (int w = 0; w < W; ++w)
        if (w < world) {
#pragma unroll
          for (int j = 0; j < N; ++j) acc[j] += io<TIn>::load(v[u][w].e[j]);
        }
      vec16<TOut> r;
#pragma unroll
      for (int j = 0; j < N; ++j) r.e[j] = io<TOut>::store(acc[j]);
#pragma unroll
      for (int w = 0; w < W; ++w)
        if (w < world) *reinterpret_cast<uint4 *>(static_cast<TOut *>(out.ptr[w]) + e) = r.raw;
    }
  }
}

template <typename TIn, typename TOut, bool SYNC, int U, int W>
__global__ void __launch_bounds__(kThreads)
peer_allreduce_kernel(RankPointers partial, RankPointers out, int64_t first, int64_t vecs,
                      SignalPads pads, int rank, int world, uint32_t epoch,
                      unsigned int *status) {
  if constexpr (SYNC) {
    if (!cross_rank_barrier(pads, rank, world, 0, epoch, status, kSiteStart)) return;
  }
  peer_reduce_share<TIn, TOut, U, W, false>(partial, out, first, vecs, world);
  if constexpr (SYNC) cross_rank_barrier(pads, rank, world, 1, epoch, status, kSiteEnd);
}

// The same all-reduce, block of rows by block of rows, BESIDE the GEMM that produces the
// partial.  The kernel is launched as the programmatic dependent of that GEMM, so its CTAs (128
// threads: they fit beside a persistent GEMM CTA) become resident while the GEMM runs.  For
// every block of rows: thread 0 waits until this rank's GEMM has counted the block complete
// (progress[b] >= target[b]; the GEMM is resident and waits for nothing of this kernel), the
// CTA signals and awaits its peers' CTAs for this block (epoch0 + b), and reduces this rank's
// share of the block.  So only the last block's all-reduce is left when the GEMM ends.  At the
// end: the closing cross-rank barrier, the counters put back to zero by the last CTA to have
// read them, and griddepcontrol.wait, so that this kernel does not end before the GEMM has.
// Every wait is bounded; a wait that runs out records B200_TIMEOUT and the rest is skipped.
constexpr int kBlockThreads = 128;
constexpr int kMaxBlocks = 16;
constexpr uint32_t kSiteProgress = 42;
struct BlockPlan {
  unsigned int target[kMaxBlocks];
};

// What moves a share of a block: plain peer loads and stores, or the switch.
template <typename TIn, typename TOut, int U, int W> struct PeerMover {
  RankPointers partial, out;
  __device__ __forceinline__ void run(int64_t first, int64_t vecs, int world) const {
    peer_reduce_share<TIn, TOut, U, W, true>(partial, out, first, vecs, world);
  }
};
template <int IN, int OUT> struct SwitchMover {
  const uint8_t *in_mc;
  uint8_t *out_mc;
  __device__ __forceinline__ void run(int64_t first, int64_t vecs, int) const {
    constexpr int U = 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i + u * stride < vecs)
          v[u] = reduced_vector<IN, OUT>(in_mc, first + (i + u * stride) * 8);
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i + u * stride < vecs) multimem_st16(out_mc + (first + (i + u * stride) * 8) * 2, v[u]);
    }
  }
};

template <typename Mover, bool SYNC>
__global__ void __launch_bounds__(kBlockThreads, 4)  // at most 128 registers: see the launcher
allreduce_blocks_kernel(const __grid_constant__ Mover mover, int64_t total,
                        int64_t block_elems, int nblocks, unsigned int *progress,
                        const __grid_constant__ BlockPlan plan,
                        const __grid_constant__ SignalPads pads, int rank, int world,
                        uint32_t epoch0, unsigned int *status) {
  __shared__ int ready;
  bool alive = true;
  // trace (CTA 0, thread 0; 64-bit nanoseconds after the counters): [0] entry of the kernel,
  // [1 + 2b] block b counted complete by this rank's GEMM, [2 + 2b] block b reduced
  unsigned long long *trace =
      progress != nullptr && blockIdx.x == 0 && threadIdx.x == 0
          ? reinterpret_cast<unsigned long long *>(progress + kMaxBlocks + 2) : nullptr;
  if (trace != nullptr) trace[0] = timer_ns();
  for (int b = 0; b < nblocks && alive; ++b) {
    if (progress != nullptr) {
      if (threadIdx.x == 0) {
        int ok = 1;
        const uint64_t t0 = timer_ns();
        while (ld_acquire_gpu_u32(progress + b) < plan.target[b]) {
          __nanosleep(200);
          if (timer_ns() - t0 > kFlagWaitNs) {
            atomicOr(status, (unsigned)B200_TIMEOUT | (kSiteProgress << 8));
            ok = 0;
            break;
          }
        }
        ready = ok;
        if (trace != nullptr) trace[1 + 2 * b] = timer_ns();
      }
      __syncthreads();
      alive = ready != 0;
      __syncthreads();  // everyone has read `ready` before thread 0 writes it again
    }
    if constexpr (SYNC) {
      if (alive && !cross_rank_barrier(pads, rank, world, 0, epoch0 + (uint32_t)b, status,
                                       kSiteStart))
        alive = false;
    }
    if (alive) {
      const int64_t lo = (int64_t)b * block_elems;
      const int64_t n = total - lo < block_elems ? total - lo : block_elems;
      const int64_t share = n / world;
      mover.run(lo + (int64_t)rank * share, share / 8, world);
      if (trace != nullptr) trace[2 + 2 * b] = timer_ns();
    }
  }
  if constexpr (SYNC) {
    if (alive)
      cross_rank_barrier(pads, rank, world, 1, epoch0 + (uint32_t)(nblocks - 1), status, kSiteEnd);
  }
  if (progress != nullptr && threadIdx.x == 0) {
    unsigned int *done = progress + kMaxBlocks;
    if (atomicAdd(done, 1u) == gridDim.x - 1) {
      for (int b = 0; b < nblocks; ++b) progress[b] = 0u;
      *done = 0u;
      __threadfence();
    }
  }
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename TIn, typename TOut, int U, int W>
int launch_peer_u(const RankPointers &partial, const RankPointers &out, int64_t first,
                  int64_t vecs, const SignalPads &pads, bool sync, int rank, int world,
                  uint32_t epoch, int ctas, cudaStream_t s) {
  int64_t blocks = (vecs + kThreads * U - 1) / (kThreads * U);
  int64_t cap = ctas > 0 ? ctas : (int64_t)sm_count() * 2;
  if (cap > kMaxCtas) cap = kMaxCtas;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  unsigned int *status = device_status_word();
  if (status == nullptr) return fail(B200_RESOURCE, "no status word on this device");
  if (sync)
    peer_allreduce_kernel<TIn, TOut, true, U, W><<<(unsigned)blocks, kThreads, 0, s>>>(
        partial, out, first, vecs, pads, rank, world, epoch, status);
  else
    peer_allreduce_kernel<TIn, TOut, false, U, W><<<(unsigned)blocks, kThreads, 0, s>>>(
        partial, out, first, vecs, pads, rank, world, epoch, status);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

// sixteen 16-byte loads in flight per thread whatever the number of ranks
template <typename TIn, typename TOut>
int launch_peer(const RankPointers &partial, const RankPointers &out, int64_t first, int64_t vecs,
                const SignalPads &pads, bool sync, int rank, int world, uint32_t epoch, int ctas,
                cudaStream_t s) {
  if (world <= 2)
    return launch_peer_u<TIn, TOut, 8, 2>(partial, out, first, vecs, pads, sync, rank, world, epoch,
                                       ctas, s);
  if (world <= 4)
    return launch_peer_u<TIn, TOut, 4, 4>(partial, out, first, vecs, pads, sync, rank, world, epoch,
                                       ctas, s);
  return launch_peer_u<TIn, TOut, 2, 8>(partial, out, first, vecs, pads, sync, rank, world, epoch,
                                     ctas, s);
}

template <typename Mover>
int launch_blocks(const Mover &mover, int64_t total, int64_t block_elems, int nblocks,
                  unsigned int *progress, const BlockPlan &plan, const SignalPads &pads,
                  bool sync, int rank, int world, uint32_t epoch0, int ctas, cudaStream_t s) {
  // One CTA of 128 threads and at most 128 registers per SM: that fits beside the CTA-pair
  // GEMM (an SM sub-partition's 16 K registers then hold two GEMM warps of 184 registers and
  // one warp of this kernel).  Sixteen 16-byte loads in flight per thread: 148 CTAs hold
  // 4.6 MiB in flight, more than the links' latency x bandwidth.
  int64_t blocks = ctas > 0 ? ctas : sm_count();
  if (blocks > kMaxCtas) blocks = kMaxCtas;
  unsigned int *status = device_status_word();
  if (status == nullptr) return fail(B200_RESOURCE, "no status word on this device");
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)blocks);
  config.blockDim = dim3(kBlockThreads);
  config.dynamicSmemBytes = 0;
  config.stream = s;
  // programmatic dependent of the kernel before it on the stream: may start once that kernel's
  // CTAs have released their dependents (a kernel that never does releases them at its end)
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = progress != nullptr ? 1 : 0;
  config.attrs = &attr;
  config.numAttrs = 1;
  // the same shared-memory carve-out as the GEMM it runs beside (which takes the maximum)
  static bool configured[64] = {false};  // per device: function attributes belong to a context
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  if (dev >= 64) return fail(B200_RESOURCE, "device index %d out of range", dev);
  if (!configured[dev]) {
    B200_CUDA_OK(cudaFuncSetAttribute(allreduce_blocks_kernel<Mover, true>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    B200_CUDA_OK(cudaFuncSetAttribute(allreduce_blocks_kernel<Mover, false>,
                                      cudaFuncAttributePreferredSharedMemoryCarveout,
                                      cudaSharedmemCarveoutMaxShared));
    configured[dev] = true;
  }
  if (sync)
    B200_CUDA_OK(cudaLaunchKernelEx(&config, allreduce_blocks_kernel<Mover, true>, mover, total,
                                    block_elems, nblocks, progress, plan, pads, rank, world,
                                    epoch0, status));
  else
    B200_CUDA_OK(cudaLaunchKernelEx(&config, allreduce_blocks_kernel<Mover, false>, mover, total,
                                    block_elems, nblocks, progress, plan, pads, rank, world,
                                    epoch0, status));
  return B200_OK;
}

template <typename TIn, typename TOut>
int launch_peer_blocks(const RankPointers &partial, const RankPointers &out, int64_t total,
                       int64_t block_elems, int nblocks, unsigned int *progress,
                       const BlockPlan &plan, const SignalPads &pads, bool sync, int rank,
                       int world, uint32_t epoch0, int ctas, cudaStream_t s) {
  if (world <= 2)
    return launch_blocks(PeerMover<TIn, TOut, 8, 2>{partial, out}, total, block_elems, nblocks,
                         progress, plan, pads, sync, rank, world, epoch0, ctas, s);
  if (world <= 4)
    return launch_blocks(PeerMover<TIn, TOut, 4, 4>{partial, out}, total, block_elems, nblocks,
                         progress, plan, pads, sync, rank, world, epoch0, ctas, s);
  return launch_blocks(PeerMover<TIn, TOut, 2, 8>{partial, out}, total, block_elems, nblocks,
                       progress, plan, pads, sync, rank, world, epoch0, ctas, s);
}

template <int IN, int OUT>
int launch(const void *in_mc, void *out_mc, int64_t first, int64_t vecs, const SignalPads &pads,
           bool sync, int rank, int world, uint32_t epoch, int ctas, cudaStream_t s) {
  int64_t blocks = (vecs + kThreads * 8 - 1) / (kThreads * 8);
  int64_t cap = ctas > 0 ? ctas : (int64_t)sm_count() * 2;
  if (cap > kMaxCtas) cap = kMaxCtas;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  unsigned int *status = device_status_word();
  if (status == nullptr) return fail(B200_RESOURCE, "no status word on this device");
  if (sync)
    multimem_allreduce_kernel<IN, OUT, true><<<(unsigned)blocks, kThreads, 0, s>>>(
        (const uint8_t *)in_mc, (uint8_t *)out_mc, first, vecs, pads, rank, world, epoch, status);
  else
    multimem_allreduce_kernel<IN, OUT, false><<<(unsigned)blocks, kThreads, 0, s>>>(
        (const uint8_t *)in_mc, (uint8_t *)out_mc, first, vecs, pads, rank, world, epoch, status);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" size_t b200_signal_pad_bytes(void) {
  return (size_t)2 * b200::kMaxCtas * 8 * sizeof(uint32_t);
}

extern "C" int b200_multimem_allreduce(const void *in_multicast, uint32_t in_dtype,
                                       void *out_multicast, uint32_t out_dtype, int64_t offset,
                                       int64_t count, int rank, int world,
                                       void *const *signal_pads, uint32_t epoch, int ctas,
                                       void *stream) {
  using namespace b200;
  if (in_multicast == nullptr || out_multicast == nullptr)
    return fail(B200_USAGE, "null multicast pointer");
  B200_REQUIRE(in_dtype == B200_DTYPE_BFLOAT16 || in_dtype == B200_DTYPE_FLOAT16 ||
               in_dtype == B200_DTYPE_FLOAT32, "partials are f16, bf16 or f32");
  B200_REQUIRE(out_dtype == B200_DTYPE_BFLOAT16 || out_dtype == B200_DTYPE_FLOAT16,
               "the result is f16 or bf16");
  B200_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world,
               "rank %d / world %d out of range", rank, world);
  B200_REQUIRE(offset >= 0 && count >= 0 && offset % 8 == 0 && count % (8 * world) == 0,
               "offset and count / world must be multiples of 8 elements");
  B200_REQUIRE((uintptr_t)in_multicast % 16 == 0 && (uintptr_t)out_multicast % 16 == 0,
               "multicast pointers must be 16-byte aligned");
  B200_REQUIRE(in_dtype != B200_DTYPE_FLOAT32 || in_multicast != out_multicast,
               "f32 partials cannot be reduced in place into a 16-bit result");
  SignalPads pads;
  for (int k = 0; k < 8; ++k) pads.pad[k] = nullptr;
  const bool sync = signal_pads != nullptr;
  if (sync) {
    B200_REQUIRE(epoch != 0, "epoch 0 is the cleared state of the signal pads: start at 1");
    for (int k = 0; k < world; ++k) {
      B200_REQUIRE(signal_pads[k] != nullptr && (uintptr_t)signal_pads[k] % 4 == 0,
                   "signal pad of rank %d is null or unaligned", k);
      pads.pad[k] = static_cast<uint32_t *>(signal_pads[k]);
    }
  }
  if (count == 0 && !sync) return B200_OK;
  const int64_t share = count / world;
  const int64_t first = offset + (int64_t)rank * share;
  const int64_t vecs = share / 8;
  cudaStream_t s = (cudaStream_t)stream;
#define B200_AR(IN, OUT) \
  return launch<IN, OUT>(in_multicast, out_multicast, first, vecs, pads, sync, rank, world, \
                         epoch, ctas, s)
  if (out_dtype == B200_DTYPE_BFLOAT16) {
    if (in_dtype == B200_DTYPE_FLOAT32) B200_AR(B200_DTYPE_FLOAT32, B200_DTYPE_BFLOAT16);
    if (in_dtype == B200_DTYPE_FLOAT16) B200_AR(B200_DTYPE_FLOAT16, B200_DTYPE_BFLOAT16);
    B200_AR(B200_DTYPE_BFLOAT16, B200_DTYPE_BFLOAT16);
  }
  if (in_dtype == B200_DTYPE_FLOAT32) B200_AR(B200_DTYPE_FLOAT32, B200_DTYPE_FLOAT16);
  if (in_dtype == B200_DTYPE_BFLOAT16) B200_AR(B200_DTYPE_BFLOAT16, B200_DTYPE_FLOAT16);
  B200_AR(B200_DTYPE_FLOAT16, B200_DTYPE_FLOAT16);
#undef B200_AR
}

extern "C" int b200_peer_allreduce(void *const *partial_rank, uint32_t in_dtype,
                                   void *const *out_rank, uint32_t out_dtype, int64_t offset,
                                   int64_t count, int rank, int world, void *const *signal_pads,
                                   uint32_t epoch, int ctas, void *stream) {
  using namespace b200;
  if (partial_rank == nullptr || out_rank == nullptr) return fail(B200_USAGE, "null argument");
  B200_REQUIRE((in_dtype == B200_DTYPE_BFLOAT16 || in_dtype == B200_DTYPE_FLOAT16) &&
               (out_dtype == B200_DTYPE_BFLOAT16 || out_dtype == B200_DTYPE_FLOAT16),
               "partials and result are f16 or bf16");
  B200_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world,
               "rank %d / world %d out of range", rank, world);
  B200_REQUIRE(offset >= 0 && count >= 0 && offset % 8 == 0 && count % (8 * world) == 0,
               "offset and count / world must be multiples of 8 elements");
  RankPointers partial, out;
  SignalPads pads;
  for (int k = 0; k < 8; ++k) partial.ptr[k] = out.ptr[k] = nullptr, pads.pad[k] = nullptr;
  for (int k = 0; k < world; ++k) {
    B200_REQUIRE(partial_rank[k] != nullptr && (uintptr_t)partial_rank[k] % 16 == 0 &&
                 out_rank[k] != nullptr && (uintptr_t)out_rank[k] % 16 == 0,
                 "buffer of rank %d is null or unaligned", k);
    partial.ptr[k] = partial_rank[k];
    out.ptr[k] = out_rank[k];
  }
  const bool sync = signal_pads != nullptr;
  if (sync) {
    B200_REQUIRE(epoch != 0, "epoch 0 is the cleared state of the signal pads: start at 1");
    for (int k = 0; k < world; ++k) {
      B200_REQUIRE(signal_pads[k] != nullptr && (uintptr_t)signal_pads[k] % 4 == 0,
                   "signal pad of rank %d is null or unaligned", k);
      pads.pad[k] = static_cast<uint32_t *>(signal_pads[k]);
    }
  }
  if (count == 0 && !sync) return B200_OK;
  const int64_t share = count / world;
  const int64_t first = offset + (int64_t)rank * share;
  const int64_t vecs = share / 8;
  cudaStream_t s = (cudaStream_t)stream;
#define B200_PAR(TIn, TOut) \
  return launch_peer<TIn, TOut>(partial, out, first, vecs, pads, sync, rank, world, epoch, ctas, s)
  if (in_dtype == B200_DTYPE_BFLOAT16 && out_dtype == B200_DTYPE_BFLOAT16)
    B200_PAR(__nv_bfloat16, __nv_bfloat16);
  if (in_dtype == B200_DTYPE_FLOAT16 && out_dtype == B200_DTYPE_BFLOAT16)
    B200_PAR(__half, __nv_bfloat16);
  if (in_dtype == B200_DTYPE_BFLOAT16) B200_PAR(__nv_bfloat16, __half);
  B200_PAR(__half, __half);
#undef B200_PAR
}

extern "C" int b200_peer_allreduce_blocks(void *const *partial_rank, uint32_t in_dtype,
                                          void *const *out_rank, uint32_t out_dtype,
                                          int64_t total, int64_t block_elems,
                                          unsigned int *progress, const unsigned int *targets,
                                          int rank, int world, void *const *signal_pads,
                                          uint32_t epoch0, int ctas, void *stream) {
  using namespace b200;
  if (partial_rank == nullptr || out_rank == nullptr) return fail(B200_USAGE, "null argument");
  B200_REQUIRE((in_dtype == B200_DTYPE_BFLOAT16 || in_dtype == B200_DTYPE_FLOAT16) &&
               (out_dtype == B200_DTYPE_BFLOAT16 || out_dtype == B200_DTYPE_FLOAT16),
               "partials and result are f16 or bf16");
  B200_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world,
               "rank %d / world %d out of range", rank, world);
  B200_REQUIRE(total > 0 && block_elems > 0 && block_elems % (8 * world) == 0 &&
               total % (8 * world) == 0,
               "total and block size / world must be multiples of 8 elements");
  const int64_t nblocks = (total + block_elems - 1) / block_elems;
  B200_REQUIRE(nblocks <= kMaxBlocks, "%lld blocks, at most %d", (long long)nblocks, kMaxBlocks);
  B200_REQUIRE((progress == nullptr) == (targets == nullptr),
               "progress counters and their targets come together");
  B200_REQUIRE(progress == nullptr || (uintptr_t)progress % 4 == 0, "progress is unaligned");
  RankPointers partial, out;
  SignalPads pads;
  BlockPlan plan;
  for (int k = 0; k < 8; ++k) partial.ptr[k] = out.ptr[k] = nullptr, pads.pad[k] = nullptr;
  for (int b = 0; b < kMaxBlocks; ++b) plan.target[b] = targets && b < nblocks ? targets[b] : 0u;
  for (int k = 0; k < world; ++k) {
    B200_REQUIRE(partial_rank[k] != nullptr && (uintptr_t)partial_rank[k] % 16 == 0 &&
                 out_rank[k] != nullptr && (uintptr_t)out_rank[k] % 16 == 0,
                 "buffer of rank %d is null or unaligned", k);
    partial.ptr[k] = partial_rank[k];
    out.ptr[k] = out_rank[k];
  }
  const bool sync = signal_pads != nullptr;
  if (sync) {
    B200_REQUIRE(epoch0 != 0, "epoch 0 is the cleared state of the signal pads: start at 1");
    for (int k = 0; k < world; ++k) {
      B200_REQUIRE(signal_pads[k] != nullptr && (uintptr_t)signal_pads[k] % 4 == 0,
                   "signal pad of rank %d is null or unaligned", k);
      pads.pad[k] = static_cast<uint32_t *>(signal_pads[k]);
    }
  }
  cudaStream_t s = (cudaStream_t)stream;
#define B200_PARB(TIn, TOut)                                                                  \
  return launch_peer_blocks<TIn, TOut>(partial, out, total, block_elems, (int)nblocks, progress, \
                                       plan, pads, sync, rank, world, epoch0, ctas, s)
  if (in_dtype == B200_DTYPE_BFLOAT16 && out_dtype == B200_DTYPE_BFLOAT16)
    B200_PARB(__nv_bfloat16, __nv_bfloat16);
  if (in_dtype == B200_DTYPE_FLOAT16 && out_dtype == B200_DTYPE_BFLOAT16)
    B200_PARB(__half, __nv_bfloat16);
  if (in_dtype == B200_DTYPE_BFLOAT16) B200_PARB(__nv_bfloat16, __half);
  B200_PARB(__half, __half);
#undef B200_PARB
}

extern "C" int b200_multimem_allreduce_blocks(const void *in_multicast, uint32_t in_dtype,
                                              void *out_multicast, uint32_t out_dtype,
                                              int64_t total, int64_t block_elems,
                                              unsigned int *progress, const unsigned int *targets,
                                              int rank, int world, void *const *signal_pads,
                                              uint32_t epoch0, int ctas, void *stream) {
  using namespace b200;
  if (in_multicast == nullptr || out_multicast == nullptr)
    return fail(B200_USAGE, "null multicast pointer");
  B200_REQUIRE(in_dtype == B200_DTYPE_BFLOAT16 || in_dtype == B200_DTYPE_FLOAT16 ||
               in_dtype == B200_DTYPE_FLOAT32, "partials are f16, bf16 or f32");
  B200_REQUIRE(out_dtype == B200_DTYPE_BFLOAT16 || out_dtype == B200_DTYPE_FLOAT16,
               "the result is f16 or bf16");
  B200_REQUIRE(in_dtype == B200_DTYPE_FLOAT32 || in_dtype == B200_DTYPE_FLOAT16 ||
               out_dtype == B200_DTYPE_BFLOAT16, "bf16 partials give a bf16 result");
  B200_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world,
               "rank %d / world %d out of range", rank, world);
  B200_REQUIRE(total > 0 && block_elems > 0 && block_elems % (8 * world) == 0 &&
               total % (8 * world) == 0,
               "total and block size / world must be multiples of 8 elements");
  B200_REQUIRE((uintptr_t)in_multicast % 16 == 0 && (uintptr_t)out_multicast % 16 == 0,
               "multicast pointers must be 16-byte aligned");
  const int64_t nblocks = (total + block_elems - 1) / block_elems;
  B200_REQUIRE(nblocks <= kMaxBlocks, "%lld blocks, at most %d", (long long)nblocks, kMaxBlocks);
  B200_REQUIRE((progress == nullptr) == (targets == nullptr),
               "progress counters and their targets come together");
  SignalPads pads;
  BlockPlan plan;
  for (int k = 0; k < 8; ++k) pads.pad[k] = nullptr;
  for (int b = 0; b < kMaxBlocks; ++b) plan.target[b] = targets && b < nblocks ? targets[b] : 0u;
  const bool sync = signal_pads != nullptr;
  if (sync) {
    B200_REQUIRE(epoch0 != 0, "epoch 0 is the cleared state of the signal pads: start at 1");
    for (int k = 0; k < world; ++k) {
      B200_REQUIRE(signal_pads[k] != nullptr && (uintptr_t)signal_pads[k] % 4 == 0,
                   "signal pad of rank %d is null or unaligned", k);
      pads.pad[k] = static_cast<uint32_t *>(signal_pads[k]);
    }
  }
  cudaStream_t s = (cudaStream_t)stream;
#define B200_SWB(IN, OUT)                                                                      \
  if (in_dtype == IN && out_dtype == OUT)                                                      \
    return launch_blocks(SwitchMover<IN, OUT>{(const uint8_t *)in_multicast,                   \
                                              (uint8_t *)out_multicast},                       \
                         total, block_elems, (int)nblocks, progress, plan, pads, sync, rank,   \
                         world, epoch0, ctas, s)
  B200_SWB(B200_DTYPE_FLOAT32, B200_DTYPE_BFLOAT16);
  B200_SWB(B200_DTYPE_FLOAT32, B200_DTYPE_FLOAT16);
  B200_SWB(B200_DTYPE_FLOAT16, B200_DTYPE_BFLOAT16);
  B200_SWB(B200_DTYPE_FLOAT16, B200_DTYPE_FLOAT16);
  B200_SWB(B200_DTYPE_BFLOAT16, B200_DTYPE_BFLOAT16);
#undef B200_SWB
  return fail(B200_REJECTED, "unsupported type pair");
}

// counters [kMaxBlocks], the count of CTAs that are done with them, one word of padding, and
// the trace: 1 + 2 * kMaxBlocks 64-bit time stamps
extern "C" int b200_progress_words(void) {
  return b200::kMaxBlocks + 2 + 2 * (1 + 2 * b200::kMaxBlocks);
}
