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

// The other modes of flash_varlen_fwd_kernel (ops/suite/dev/flash_varlen_fwd_kernel.py), on the
// raw score S = q.k before the softmax scale:
//   soft-cap  (:121-124)  S = tanh(S * softcap)
//   ALiBi     (:76-81, :125-133)  causal: S += slope / scale * (j - N_K + 1);
//             otherwise S -= slope / scale * |j - N_K + N - i|        (slope per batch and head)
//   local window (:56-61, :137-146)  keys max(0, i + N_K - N - left) .. min(N_K - 1, i + N_K - N + right)
// A row that sees no key gets zeros and lse = +inf (:309-310).
struct SimtModes {
  float softcap;        // 0: off
  const float *alibi;   // nullptr: off; slope of (z, h) at alibi[z * alibi_z + h]
  int64_t alibi_z;
  int local;            // 1: the window below applies
  int window_left, window_right;
  // paged K / V (:91-108): key j of batch z lives in physical page
  // page_table[z * page_table_z + j / block_size], at page * page_stride +
  // (j % block_size) * (row stride of k) past the head's base -- for K and V alike
  const int *page_table;  // nullptr: off
  int64_t page_table_z;
  int block_size;
  int64_t page_stride;
};

template <typename T>
__global__ void __launch_bounds__(kSimtThreads)
attn_simt_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                 T *__restrict__ o, float *__restrict__ lse, int64_t lse_z, int64_t lse_h, int H,
                 int kv_group, int N, int NK, int D,
                 int64_t qz, int64_t qh, int64_t qm, int64_t kz, int64_t kh, int64_t kn,
                 int64_t vz, int64_t vh, int64_t vn, int64_t oz, int64_t oh, int64_t om,
                 float scale, int causal, SimtModes modes) {
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
  // keys [first, keys) of this row
  int first = 0;
  int keys = causal ? min(NK, m + 1 + (NK - N)) : NK;
  if (modes.local) {
    first = max(0, m + (NK - N) - modes.window_left);
    keys = min(NK, m + 1 + (NK - N) + modes.window_right);
  }
  T *op = o + z * oz + h * oh + (int64_t)m * om;
  if (keys <= first) {  // no key in sight
    for (int d = threadIdx.x; d < D; d += kSimtThreads) op[d] = io<T>::store(0.f);
    if (lse != nullptr && threadIdx.x == 0) lse[z * lse_z + h * lse_h + m] = INFINITY;
    return;
  }
  const float slope = modes.alibi != nullptr ? modes.alibi[z * modes.alibi_z + h] : 0.f;
  const int *pages = modes.page_table != nullptr ? modes.page_table + z * modes.page_table_z
                                                 : nullptr;
  // offset of key j's row past the head's base (V shares K's page and row pitch when paged)
  auto key_row = [&](int j, int64_t pitch) -> int64_t {
    if (pages == nullptr) return (int64_t)j * pitch;
    return (int64_t)pages[j / modes.block_size] * modes.page_stride +
           (int64_t)(j % modes.block_size) * kn;
  };
  for (int d = threadIdx.x; d < D; d += kSimtThreads) qrow[d] = io<T>::load(qp[d]);
  __syncthreads();
  float mx = -INFINITY;
  for (int j = first + threadIdx.x; j < keys; j += kSimtThreads) {
    const T *kr = kp + key_row(j, kn);
    float acc = 0.f;
    for (int d = 0; d < D; ++d) acc = fmaf(qrow[d], io<T>::load(kr[d]), acc);
    if (modes.softcap != 0.f) acc = tanhf(acc * modes.softcap);
    acc *= scale;
    // the bias is slope / scale on the raw score, i.e. slope on the scaled one
    if (modes.alibi != nullptr)
      acc += causal ? slope * (float)(j - NK + 1) : -slope * fabsf((float)(j - NK + N - m));
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
  for (int j = first + threadIdx.x; j < keys; j += kSimtThreads) {
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
  for (int d = threadIdx.x; d < D; d += kSimtThreads) {
    float acc = 0.f;
    for (int j = first; j < keys; ++j)
      acc = fmaf(scores[j], io<T>::load(vp[key_row(j, vn) + d]), acc);
    op[d] = io<T>::store(acc * inv);
  }
  if (lse != nullptr && threadIdx.x == 0) lse[z * lse_z + h * lse_h + m] = mx + logf(sum);
}

}  // namespace attn
}  // namespace b200
