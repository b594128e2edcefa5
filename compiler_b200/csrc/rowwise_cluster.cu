// Rows wider than one CTA can hold in registers: a thread-block CLUSTER per row.
//
// The register-resident row kernels (rmsnorm.cu, softmax.cu) give a row to at most 1024
// threads x 4 vectors = 32768 16-bit or 16384 32-bit elements.  Wider rows used to fall to
// the scalar looping kernels, which read the row three times.  Here a cluster of 2, 4 or 8
// CTAs (up to 8 x 4096 vectors) owns a row: every CTA keeps its slice of the row in
// registers, reduces it with shuffles and shared memory, publishes its partial result in its
// own shared memory, and after a cluster barrier every CTA reads all partials through
// distributed shared memory -- the row is still read from HBM once and written once.  This is
// the two-phase partial / merge plan of the reference (a100c/plan/stages.py:668-715: owned
// partial slots, a stage barrier, a merge in slot order) with the workers being the CTAs of
// a cluster and the slots their shared memory.
//
// Semantics as in the one-CTA kernels: rms_layernorm_forward_kernel
// (ops/suite/perf/fast_rms_layernorm.py:19-44) and softmax_kernel
// (ops/suite/perf/softmax.py:20-31) with the optional causal-mod mask
// (ops/suite/perf/attn_fwd_causal.py:46-47).
#include <cooperative_groups.h>

#include "rowwise.cuh"

namespace cg = cooperative_groups;

namespace b200 {
namespace {

constexpr int kClusterThreads = 1024;
constexpr int kClusterVpt = 4;
constexpr int kVecPerCta = kClusterThreads * kClusterVpt;  // 4096 16-byte vectors per CTA
constexpr int kMaxCluster = 8;

// Reduce v over the CTA, publish the CTA's value in `slot` (this CTA's shared memory), and
// fold the values of all CTAs of the cluster in rank order, so every CTA gets the same bits.
// `scratch` holds one float per warp.  Two cluster barriers: the first publishes the slots,
// the second keeps a CTA from overwriting its slot (next use) or leaving while a peer reads.
template <typename Op>
__device__ __forceinline__ float cluster_reduce(float v, float *scratch, float *slot,
                                                cg::cluster_group &cluster) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < kClusterThreads / 32 ? scratch[threadIdx.x] : Op::identity();
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = Op::apply(t, __shfl_xor_sync(0xffffffffu, t, o));
    if (threadIdx.x == 0) *slot = t;
  }
  cluster.sync();
  float total = Op::identity();
  const unsigned ranks = cluster.num_blocks();
  for (unsigned r = 0; r < ranks; ++r) total = Op::apply(total, *cluster.map_shared_rank(slot, r));
  cluster.sync();
  return total;
}

template <typename T>
__global__ void __launch_bounds__(kClusterThreads, 1)
rmsnorm_cluster_kernel(const T *__restrict__ x, int64_t x_stride, const T *__restrict__ w,
                       T *__restrict__ y, int64_t y_stride, T *__restrict__ rinv, int cols,
                       float eps, float gamma_offset) {
  constexpr int N = vec16<T>::N;
  __shared__ float scratch[kClusterThreads / 32];
  __shared__ float slot;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  const int64_t row = blockIdx.x / cluster.num_blocks();
  const int nvec = cols / N;
  const int first = (int)rank * kVecPerCta;

  vec16<T> xv[kClusterVpt];
  float acc = 0.f;
  const T *xrow = x + row * x_stride;
#pragma unroll
  for (int i = 0; i < kClusterVpt; ++i) {
    const int v = first + (int)threadIdx.x + i * kClusterThreads;
    if (v < nvec) {
      xv[i].raw = ld_stream16(xrow + (int64_t)v * N);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float f = io<T>::load(xv[i].e[j]);
        acc = fmaf(f, f, acc);
      }
    }
  }
  acc = cluster_reduce<SumOp>(acc, scratch, &slot, cluster);
  const float inv = 1.0f / sqrtf(acc / (float)cols + eps);
  if (rank == 0 && threadIdx.x == 0 && rinv != nullptr) rinv[row] = io<T>::store(inv);
  T *yrow = y + row * y_stride;
#pragma unroll
  for (int i = 0; i < kClusterVpt; ++i) {
    const int v = first + (int)threadIdx.x + i * kClusterThreads;
    if (v < nvec) {
      vec16<T> wv, out;
      wv.raw = *reinterpret_cast<const uint4 *>(w + (int64_t)v * N);
#pragma unroll
      for (int j = 0; j < N; ++j)
        out.e[j] = io<T>::store(io<T>::load(xv[i].e[j]) * inv * (io<T>::load(wv.e[j]) + gamma_offset));
      st_stream16(yrow + (int64_t)v * N, out.raw);
    }
  }
}

template <typename T> __device__ __forceinline__ float exp_for(float v) { return __expf(v); }
template <> __device__ __forceinline__ float exp_for<float>(float v) { return expf(v); }

template <typename T>
__global__ void __launch_bounds__(kClusterThreads, 1)
softmax_cluster_kernel(const T *__restrict__ x, T *__restrict__ y, int cols, int mask_kind,
                       int64_t row_offset) {
  constexpr int N = vec16<T>::N;
  __shared__ float scratch[kClusterThreads / 32];
  __shared__ float slot;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  const int64_t row = blockIdx.x / cluster.num_blocks();
  const int nvec = cols / N;
  const int first = (int)rank * kVecPerCta;
  // kept columns of this row: [0, keep)
  int keep = cols;
  if (mask_kind == B200_MASK_CAUSAL_MOD) keep = (int)((row_offset + row) % cols) + 1;
  const int kept_vec = (keep + N - 1) / N;

  vec16<T> xv[kClusterVpt];
  float m = -INFINITY;
  const T *xrow = x + row * (int64_t)cols;
  T *yrow = y + row * (int64_t)cols;
#pragma unroll
  for (int i = 0; i < kClusterVpt; ++i) {
    const int v = first + (int)threadIdx.x + i * kClusterThreads;
    if (v >= kept_vec && v < nvec) st_stream16(yrow + (int64_t)v * N, make_uint4(0u, 0u, 0u, 0u));
    if (v < kept_vec) {
      xv[i].raw = ld_stream16(xrow + (int64_t)v * N);
#pragma unroll
      for (int j = 0; j < N; ++j)
        if (v * N + j < keep) m = fmaxf(m, io<T>::load(xv[i].e[j]));
    }
  }
  m = cluster_reduce<MaxOp>(m, scratch, &slot, cluster);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < kClusterVpt; ++i) {
    const int v = first + (int)threadIdx.x + i * kClusterThreads;
    if (v < kept_vec) {
#pragma unroll
      for (int j = 0; j < N; ++j)
        if (v * N + j < keep) s += exp_for<T>(io<T>::load(xv[i].e[j]) - m);
    }
  }
  s = cluster_reduce<SumOp>(s, scratch, &slot, cluster);
  const float r = 1.0f / s;
#pragma unroll
  for (int i = 0; i < kClusterVpt; ++i) {
    const int v = first + (int)threadIdx.x + i * kClusterThreads;
    if (v < kept_vec) {
      vec16<T> out;
#pragma unroll
      for (int j = 0; j < N; ++j)
        out.e[j] = io<T>::store(v * N + j < keep ? exp_for<T>(io<T>::load(xv[i].e[j]) - m) * r : 0.f);
      st_stream16(yrow + (int64_t)v * N, out.raw);
    }
  }
}

// Cluster size for a row of nvec vectors: the smallest of 2, 4, 8 whose CTAs hold it; 0 = none.
int cluster_for(int64_t nvec) {
  for (int c = 2; c <= kMaxCluster; c <<= 1)
    if ((int64_t)c * kVecPerCta >= nvec) return c;
  return 0;
}

template <typename Kernel, typename... Args>
int launch_cluster(Kernel kernel, int cluster, int64_t rows, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((unsigned)(rows * cluster));
  config.blockDim = dim3(kClusterThreads);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = (unsigned)cluster;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  config.attrs = &attr;
  config.numAttrs = 1;
  B200_CUDA_OK(cudaLaunchKernelEx(&config, kernel, args...));
  return B200_OK;
}

}  // namespace

// Both return B200_OK with *taken = true when the cluster kernel was launched; *taken = false
// (nothing launched) when the row does not need or does not fit a cluster.
template <typename T>
int rmsnorm_cluster_rows(const b200_tensor *x, const b200_tensor *w, b200_tensor *y,
                         b200_tensor *rinv, float eps, float gamma_offset, cudaStream_t stream,
                         bool *taken) {
  constexpr int N = vec16<T>::N;
  const int64_t rows = x->shape[0], cols = x->shape[1];
  *taken = false;
  const int cluster = cols % N == 0 && cols / N > kVecPerCta ? cluster_for(cols / N) : 0;
  if (cluster == 0 || rows * cluster > 0x7fffffffLL) return B200_OK;
  *taken = true;
  return launch_cluster(rmsnorm_cluster_kernel<T>, cluster, rows, stream, (const T *)x->data,
                        (int64_t)x->stride[0], (const T *)w->data, (T *)y->data,
                        (int64_t)y->stride[0], rinv ? (T *)rinv->data : (T *)nullptr, (int)cols,
                        eps, gamma_offset);
}

template <typename T>
int softmax_cluster_rows(const b200_tensor *x, b200_tensor *y, int mask_kind, int64_t row_offset,
                         cudaStream_t stream, bool *taken) {
  constexpr int N = vec16<T>::N;
  const int64_t rows = x->shape[0], cols = x->shape[1];
  *taken = false;
  const int cluster = cols % N == 0 && cols / N > kVecPerCta ? cluster_for(cols / N) : 0;
  if (cluster == 0 || rows * cluster > 0x7fffffffLL) return B200_OK;
  *taken = true;
  return launch_cluster(softmax_cluster_kernel<T>, cluster, rows, stream, (const T *)x->data,
                        (T *)y->data, (int)cols, mask_kind, row_offset);
}

#define B200_INSTANTIATE(T)                                                                     \
  template int rmsnorm_cluster_rows<T>(const b200_tensor *, const b200_tensor *, b200_tensor *, \
                                       b200_tensor *, float, float, cudaStream_t, bool *);      \
  template int softmax_cluster_rows<T>(const b200_tensor *, b200_tensor *, int, int64_t,        \
                                       cudaStream_t, bool *);
B200_INSTANTIATE(float)
B200_INSTANTIATE(__half)
B200_INSTANTIATE(__nv_bfloat16)
#undef B200_INSTANTIATE

}  // namespace b200
