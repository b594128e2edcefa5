// Row-wise reduction scaffolding shared by RMSNorm and softmax.
//
// A row is owned by a GROUP of G threads (G = 8..1024, a power of two); a CTA
// of kThreads threads holds kThreads/G rows.  Each thread keeps up to VPT
// 16-byte vectors of its row in registers, so the row is read from HBM exactly
// once; vector slots past the row end are predicated off (the masked tail).
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kRowThreads = 256;

struct SumOp {
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
  static __device__ __forceinline__ float identity() { return 0.f; }
};
struct MaxOp {
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
  static __device__ __forceinline__ float identity() { return -INFINITY; }
};

// Reduce `v` over the G consecutive threads that own one row.  `scratch` has
// 2 x (one float per warp of the CTA); `buf` (0 or 1) selects the half, and
// successive reductions in one kernel must alternate it: a thread can only
// reach reduction k+2 after every thread of its group has passed the barrier
// of reduction k+1, i.e. has finished reading the half reduction k wrote.
// The barrier is a named one per row group, so the rows of a CTA do not wait
// for each other.  Every thread of the group must call this.
template <int G, typename Op>
__device__ __forceinline__ float group_reduce(float v, float *scratch, int buf) {
  constexpr int kIntra = G < 32 ? G : 32;
#pragma unroll
  for (int o = kIntra / 2; o > 0; o >>= 1)
    v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  if constexpr (G > 32) {
    constexpr int kWarps = G / 32;
    const int group = threadIdx.x / G;
    float *slot = scratch + buf * (blockDim.x >> 5);
    if ((threadIdx.x & 31) == 0) slot[threadIdx.x >> 5] = v;
    // literal barrier ids: a register id would make ptxas reserve all 16 hardware
    // barriers per CTA and cap the CTAs per SM at 4
    if constexpr (G >= 2 * kRowThreads) {
      // 16 or 32 warps (the CTA is the group): the first warp folds the warps' values with
      // shuffles and publishes the result, instead of every thread reading 16 or 32 slots
      // itself -- with 1024 threads those broadcast reads kept the shared-memory queue full
      // (the wide-row softmax waited 5.7 cycles per issued instruction on it)
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = (int)threadIdx.x < kWarps ? slot[threadIdx.x] : Op::identity();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t = Op::apply(t, __shfl_xor_sync(0xffffffffu, t, o));
        if (threadIdx.x == 0) slot[0] = t;
      }
      __syncthreads();
      return slot[0];
    } else if constexpr (G >= kRowThreads) {
      __syncthreads();
    } else if constexpr (G == kRowThreads / 2) {
      if (group == 0) asm volatile("bar.sync 1, %0;" ::"n"(G) : "memory");
      else asm volatile("bar.sync 2, %0;" ::"n"(G) : "memory");
    } else {
      static_assert(G == kRowThreads / 4, "row groups are 64, 128 or >= 256 threads");
      if (group == 0) asm volatile("bar.sync 1, %0;" ::"n"(G) : "memory");
      else if (group == 1) asm volatile("bar.sync 2, %0;" ::"n"(G) : "memory");
      else if (group == 2) asm volatile("bar.sync 3, %0;" ::"n"(G) : "memory");
      else asm volatile("bar.sync 4, %0;" ::"n"(G) : "memory");
    }
    const int first = group * kWarps;
    v = slot[first];
#pragma unroll
    for (int i = 1; i < kWarps; ++i) v = Op::apply(v, slot[first + i]);
  }
  return v;
}

// Rows wider than one CTA holds (rowwise_cluster.cu): a cluster of 2, 4 or 8 CTAs per row,
// partial results merged through distributed shared memory.  *taken = false: nothing launched.
template <typename T>
int rmsnorm_cluster_rows(const b200_tensor *x, const b200_tensor *w, b200_tensor *y,
                         b200_tensor *rinv, float eps, float gamma_offset, cudaStream_t stream,
                         bool *taken);
template <typename T>
int softmax_cluster_rows(const b200_tensor *x, b200_tensor *y, int mask_kind, int64_t row_offset,
                         cudaStream_t stream, bool *taken);

// Picks the group size: the smallest power of two G in [8, 1024] with
// G * vpt >= nvec.  Returns 0 when the row does not fit (caller falls back to
// the looping kernel).
inline int pick_group(int64_t nvec, int vpt) {
  for (int g = 8; g <= 1024; g <<= 1)
    if ((int64_t)g * vpt >= nvec) return g;
  return 0;
}

}  // namespace b200
