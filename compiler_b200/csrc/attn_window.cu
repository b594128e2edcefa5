// Causal sliding-window attention with a gate bias and an attention sink, token-major
// layout.  Native form of parallel_attn_fwd_kernel
// (ops/suite/dev/parallel_attn_fwd_kernel.py, reference arithmetic :142-166):
//   logit[t, j] = scale * log2(e) * q[t] . k[j] + g[t] - g[j]      for max(0, t-W+1) <= j <= t
//   m = max(max_j logit, sink);  den = sum_j 2^(logit - m) + 2^(sink - m)
//   o[t] = sum_j 2^(logit - m) v[j] / den;  lse[t] = m + log2(den)
// q [B,T,HQ,K], k [B,T,H,K], v [B,T,H,V], o [B,T,HQ,V], g [B,T,HQ], sink [HQ], lse [B,T,HQ];
// query head hq reads K / V head hq / (HQ / H).  Key and value widths are free (7 and 9 in
// the reference's cases), so this is a CUDA-core kernel: one CTA per (token, batch * head),
// the window's logits in shared memory, one thread per output column for the weighted sum.
#include "common.cuh"

namespace b200 {
namespace window {

constexpr int THREADS = 128;
constexpr int kMaxKeys = 8192;  // logits of one row in shared memory

struct Params {
  const void *q, *k, *v, *g, *sink;
  void *o, *lse;
  int64_t qb, qt, qh, kb, kt, kh, vb, vt, vh, ob, ot, oh, gb, gt, lb, lt;  // element strides
  int T, H, HQ, K, V, window;  // window <= 0: every earlier token
  float scale;
  int lse_is_f32;
};

template <typename T>
__global__ void __launch_bounds__(THREADS)
attn_window_kernel(const Params p) {
  extern __shared__ float logits[];  // window keys, then K floats of q
  __shared__ float red[THREADS / 32];
  const int t = blockIdx.x, bh = blockIdx.y;
  const int b = bh / p.HQ, hq = bh % p.HQ, h = hq / (p.HQ / p.H);
  const int first = p.window > 0 ? max(0, t - p.window + 1) : 0;
  const int keys = t - first + 1;
  float *qrow = logits + keys;
  const T *q = reinterpret_cast<const T *>(p.q) + b * p.qb + (int64_t)t * p.qt + hq * p.qh;
  const T *kbase = reinterpret_cast<const T *>(p.k) + b * p.kb + h * p.kh;
  const T *vbase = reinterpret_cast<const T *>(p.v) + b * p.vb + h * p.vh;
  const T *g = p.g ? reinterpret_cast<const T *>(p.g) + b * p.gb + hq : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int d = threadIdx.x; d < p.K; d += THREADS) qrow[d] = io<T>::load(q[d]);
  __syncthreads();
  const float gt = g ? io<T>::load(g[(int64_t)t * p.gt]) : 0.f;
  const float sink = p.sink ? io<T>::load(reinterpret_cast<const T *>(p.sink)[hq]) : -INFINITY;
  float mx = sink;
  for (int j = threadIdx.x; j < keys; j += THREADS) {
    const T *kr = kbase + (int64_t)(first + j) * p.kt;
    float dot = 0.f;
    for (int d = 0; d < p.K; ++d) dot = fmaf(qrow[d], io<T>::load(kr[d]), dot);
    float z = dot * p.scale * 1.4426950216f;
    if (g) z += gt - io<T>::load(g[(int64_t)(first + j) * p.gt]);
    logits[j] = z;
    mx = fmaxf(mx, z);
  }
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  mx = red[0];
  for (int w = 1; w < THREADS / 32; ++w) mx = fmaxf(mx, red[w]);
  __syncthreads();
  float sum = 0.f;
  for (int j = threadIdx.x; j < keys; j += THREADS) {
    const float e = exp2f(logits[j] - mx);
    logits[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  float den = p.sink ? exp2f(sink - mx) : 0.f;
  for (int w = 0; w < THREADS / 32; ++w) den += red[w];
  T *o = reinterpret_cast<T *>(p.o) + b * p.ob + (int64_t)t * p.ot + hq * p.oh;
  for (int d = threadIdx.x; d < p.V; d += THREADS) {
    float acc = 0.f;
    for (int j = 0; j < keys; ++j)
      acc = fmaf(logits[j], io<T>::load(vbase[(int64_t)(first + j) * p.vt + d]), acc);
    o[d] = io<T>::store(acc / den);
  }
  if (p.lse != nullptr && threadIdx.x == 0) {
    const float value = mx + log2f(den);
    const int64_t at = b * p.lb + (int64_t)t * p.lt + hq;
    if (p.lse_is_f32) reinterpret_cast<float *>(p.lse)[at] = value;
    else reinterpret_cast<T *>(p.lse)[at] = io<T>::store(value);
  }
}

}  // namespace window
}  // namespace b200

extern "C" int b200_attn_window_fwd(const b200_tensor *q, const b200_tensor *k, const b200_tensor *v,
                                    b200_tensor *o, const b200_tensor *g_cumsum,
                                    const b200_tensor *sink_bias, b200_tensor *lse, float scale,
                                    int window, void *stream) {
  using namespace b200;
  int st;
  if ((st = check_tensor(q, "q", 4)) || (st = check_tensor(k, "k", 4)) ||
      (st = check_tensor(v, "v", 4)) || (st = check_tensor(o, "o", 4)))
    return st;
  if (g_cumsum != nullptr && (st = check_tensor(g_cumsum, "g_cumsum", 3))) return st;
  if (sink_bias != nullptr && (st = check_tensor(sink_bias, "sink_bias", 1))) return st;
  if (lse != nullptr && (st = check_tensor(lse, "lse", 3))) return st;
  B200_REQUIRE(is_float_io(q->dtype), "q: dtype %u is not f16/bf16/f32", q->dtype);
  B200_REQUIRE(k->dtype == q->dtype && v->dtype == q->dtype && o->dtype == q->dtype,
               "q/k/v/o dtypes differ");
  const int64_t B = q->shape[0], T = q->shape[1], HQ = q->shape[2], K = q->shape[3];
  const int64_t H = k->shape[2], V = v->shape[3];
  B200_REQUIRE(k->shape[0] == B && k->shape[1] == T && k->shape[3] == K, "k must be [B,T,H,K]");
  B200_REQUIRE(v->shape[0] == B && v->shape[1] == T && v->shape[2] == H, "v must be [B,T,H,V]");
  B200_REQUIRE(o->shape[0] == B && o->shape[1] == T && o->shape[2] == HQ && o->shape[3] == V,
               "o must be [B,T,HQ,V]");
  B200_REQUIRE(H > 0 ? HQ % H == 0 : HQ == 0, "query heads %lld are not a multiple of K/V heads %lld",
               (long long)HQ, (long long)H);
  B200_REQUIRE(q->stride[3] == 1 && k->stride[3] == 1 && v->stride[3] == 1 && o->stride[3] == 1,
               "last-dim stride must be 1");
  if (g_cumsum != nullptr)
    B200_REQUIRE(g_cumsum->dtype == q->dtype && g_cumsum->shape[0] == B && g_cumsum->shape[1] == T &&
                 g_cumsum->shape[2] == HQ && g_cumsum->stride[2] == 1, "g_cumsum must be [B,T,HQ]");
  if (sink_bias != nullptr)
    B200_REQUIRE(sink_bias->dtype == q->dtype && sink_bias->shape[0] == HQ && sink_bias->stride[0] == 1,
                 "sink_bias must be contiguous [HQ]");
  if (lse != nullptr)
    B200_REQUIRE((lse->dtype == q->dtype || lse->dtype == B200_DTYPE_FLOAT32) && lse->shape[0] == B &&
                 lse->shape[1] == T && lse->shape[2] == HQ && lse->stride[2] == 1,
                 "lse must be [B,T,HQ] in q's type or f32");
  B200_REQUIRE(scale == scale && scale > 0.f, "scale must be positive");
  B200_REQUIRE(B * HQ < 65536 && K <= 4096 && V <= 4096, "extent out of range");
  if (B * HQ == 0 || T == 0) return B200_OK;
  const int64_t keys = window > 0 && window < T ? window : T;
  B200_REQUIRE(keys <= window::kMaxKeys, "the window (%lld keys) exceeds this kernel's limit %d",
               (long long)keys, window::kMaxKeys);

  window::Params p;
  p.q = q->data; p.k = k->data; p.v = v->data; p.o = o->data;
  p.g = g_cumsum ? g_cumsum->data : nullptr;
  p.sink = sink_bias ? sink_bias->data : nullptr;
  p.lse = lse ? lse->data : nullptr;
  p.qb = q->stride[0]; p.qt = q->stride[1]; p.qh = q->stride[2];
  p.kb = k->stride[0]; p.kt = k->stride[1]; p.kh = k->stride[2];
  p.vb = v->stride[0]; p.vt = v->stride[1]; p.vh = v->stride[2];
  p.ob = o->stride[0]; p.ot = o->stride[1]; p.oh = o->stride[2];
  p.gb = g_cumsum ? g_cumsum->stride[0] : 0; p.gt = g_cumsum ? g_cumsum->stride[1] : 0;
  p.lb = lse ? lse->stride[0] : 0; p.lt = lse ? lse->stride[1] : 0;
  p.T = (int)T; p.H = (int)H; p.HQ = (int)HQ; p.K = (int)K; p.V = (int)V; p.window = window;
  p.scale = scale;
  p.lse_is_f32 = lse != nullptr && lse->dtype == B200_DTYPE_FLOAT32;
  const size_t smem = (size_t)(keys + K) * sizeof(float);
  dim3 grid((unsigned)T, (unsigned)(B * HQ));
  cudaStream_t s = (cudaStream_t)stream;
#define B200_AW(T_)                                                                             \
  do {                                                                                          \
    if (smem > 48 * 1024)                                                                       \
      B200_CUDA_OK(cudaFuncSetAttribute(window::attn_window_kernel<T_>,                         \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    window::attn_window_kernel<T_><<<grid, window::THREADS, smem, s>>>(p);                      \
  } while (0)
  if (q->dtype == B200_DTYPE_FLOAT32) B200_AW(float);
  else if (q->dtype == B200_DTYPE_FLOAT16) B200_AW(__half);
  else B200_AW(__nv_bfloat16);
#undef B200_AW
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}
