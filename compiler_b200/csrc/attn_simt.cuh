// CUDA-core attention forward: one CTA per (query row, batch*head).  Serves the
// shapes the tensor-core kernel does not take (head_dim other than 64/128,
// fp32 tensors, short or ragged sequences).  Same arithmetic as
// attn_fwd_causal_kernel (ops/suite/perf/attn_fwd_causal.py:29-57): fp32
// scores, max, exp, normalise, weighted sum of V.
#pragma once

#include "common.cuh"

namespace b200 {
namespace attn {

constexpr int kSimtThreads = 256;
constexpr int kSimtMaxKeys = 8192;  // scores of one row are staged in shared memory

template <typename T>
__global__ void __launch_bounds__(kSimtThreads)
attn_simt_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                 T *__restrict__ o, float *__restrict__ lse, int64_t lse_z, int64_t lse_h, int H,
                 int kv_group, int N, int NK, int D,
                 int64_t qz, int64_t qh, int64_t qm, int64_t kz, int64_t kh, int64_t kn,
                 int64_t vz, int64_t vh, int64_t vn, int64_t oz, int64_t oh, int64_t om,
                 float scale, int causal) {
  extern __shared__ float sm[];
  float *scores = sm;            // [NK]
  float *qrow = sm + NK;         // [D]
  __shared__ float red[kSimtThreads / 32];
  const int m = blockIdx.x;
  const int zh = blockIdx.y;
  const int z = zh / H, h = zh % H;
  const T *qp = q + z * qz + h * qh + (int64_t)m * qm;
  const T *kp = k + z * kz + (h / kv_group) * kh;
  const T *vp = v + z * vz + (h / kv_group) * vh;
  const int keys = causal ? min(NK, m + 1 + (NK - N)) : NK;
  for (int d = threadIdx.x; d < D; d += kSimtThreads) qrow[d] = io<T>::load(qp[d]);
  __syncthreads();
  float mx = -INFINITY;
  for (int j = threadIdx.x; j < keys; j += kSimtThreads) {
    const T *kr = kp + (int64_t)j * kn;
    float acc = 0.f;
    for (int d = 0; d < D; ++d) acc = fmaf(qrow[d], io<T>::load(kr[d]), acc);
    acc *= scale;
    scores[j] = acc;
    mx = fmaxf(mx, acc);
  }
  mx = warp_max(mx);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
  for (int i = 1; i < kSimtThreads / 32; ++i) mx = fmaxf(mx, red[i]);
  __syncthreads();
  float sum = 0.f;
  for (int j = threadIdx.x; j < keys; j += kSimtThreads) {
    const float e = expf(scores[j] - mx);
    scores[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sum;
  __syncthreads();
  sum = 0.f;
  for (int i = 0; i < kSimtThreads / 32; ++i) sum += red[i];
  const float inv = 1.0f / sum;
  T *op = o + z * oz + h * oh + (int64_t)m * om;
  for (int d = threadIdx.x; d < D; d += kSimtThreads) {
    float acc = 0.f;
    for (int j = 0; j < keys; ++j) acc = fmaf(scores[j], io<T>::load(vp[(int64_t)j * vn + d]), acc);
    op[d] = io<T>::store(acc * inv);
  }
  if (lse != nullptr && threadIdx.x == 0) lse[z * lse_z + h * lse_h + m] = mx + logf(sum);
}

}  // namespace attn
}  // namespace b200
