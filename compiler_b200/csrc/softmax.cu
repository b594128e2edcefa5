// Row softmax with an index-computed mask, for sm_100a.
//
// Semantics follow softmax_kernel (ops/suite/perf/softmax.py:20-31): fp32
// row max, e = exp(x - max), y = e / sum(e), one rounding at the store.  With
// B200_MASK_CAUSAL_MOD the columns col > (row_offset + row) % n_cols are
// treated as -inf exactly like `tl.where(offs_n <= pid_m, qk, -inf)`
// (ops/suite/perf/attn_fwd_causal.py:46-47): they add 0 to the sum and are
// written as 0.  Column 0 is always kept, so no row is fully masked.
//
// HBM-bound: the row stays in registers between max, sum and the store; the
// masked part of a row is never loaded (its output is a constant 0), so the
// DRAM read traffic is below the algorithmic 2 B/element of an fp16 read.
#include "rowwise.cuh"

namespace b200 {

template <typename T> __device__ __forceinline__ float fast_exp(float v) {
  return __expf(v);  // 16-bit outputs: ex2.approx error is far below 1 ulp of T
}
template <> __device__ __forceinline__ float fast_exp<float>(float v) { return expf(v); }

__device__ __forceinline__ float ex2_approx(float v) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(v));
  return y;
}

// Per-type handling of one 16-byte vector of a row.
template <typename T> struct RowVec;

template <> struct RowVec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void mask_tail(uint4 &raw, int count) {
    float *e = reinterpret_cast<float *>(&raw);
#pragma unroll
    for (int j = 0; j < N; ++j)
      if (j >= count) e[j] = -INFINITY;
  }
  static __device__ __forceinline__ float vmax(const uint4 &raw) {
    const float *e = reinterpret_cast<const float *>(&raw);
    return fmaxf(fmaxf(e[0], e[1]), fmaxf(e[2], e[3]));
  }
  // sum of exp(x[j] - m)
  static __device__ __forceinline__ float expsum(const uint4 &raw, float m, float) {
    const float *e = reinterpret_cast<const float *>(&raw);
    return (expf(e[0] - m) + expf(e[1] - m)) + (expf(e[2] - m) + expf(e[3] - m));
  }
  // exp(x[j] - m) * r in the storage type
  static __device__ __forceinline__ uint4 scaled(const uint4 &raw, float m, float, float r) {
    const float *e = reinterpret_cast<const float *>(&raw);
    uint4 out;
    float *o = reinterpret_cast<float *>(&out);
#pragma unroll
    for (int j = 0; j < N; ++j) o[j] = expf(e[j] - m) * r;
    return out;
  }
};

// 16-bit rows: the max is taken on packed pairs in the storage type (exact),
// exp is one FFMA + one ex2 per element: 2^(x*log2e - m*log2e).
template <typename T2, typename T1> struct RowVec16 {
  static constexpr int N = 8;
  static __device__ __forceinline__ void mask_tail(uint4 &raw, int count) {
    T1 *e = reinterpret_cast<T1 *>(&raw);
    const T1 ninf = io<T1>::store(-INFINITY);
#pragma unroll
    for (int j = 0; j < N; ++j)
      if (j >= count) e[j] = ninf;
  }
  static __device__ __forceinline__ float vmax(const uint4 &raw) {
    const T2 *p = reinterpret_cast<const T2 *>(&raw);
    const T2 a = __hmax2(__hmax2(p[0], p[1]), __hmax2(p[2], p[3]));
    return fmaxf(io<T1>::load(a.x), io<T1>::load(a.y));
  }
  static __device__ __forceinline__ float e2(T1 x, float neg_m_log2e) {
    return ex2_approx(fmaf(io<T1>::load(x), 1.4426950408889634f, neg_m_log2e));
  }
  static __device__ __forceinline__ float expsum(const uint4 &raw, float, float neg_m_log2e) {
    const T1 *e = reinterpret_cast<const T1 *>(&raw);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < N; j += 2) {
      s0 += e2(e[j], neg_m_log2e);
      s1 += e2(e[j + 1], neg_m_log2e);
    }
    return s0 + s1;
  }
};
// The exponentials are recomputed for the store instead of being kept: 16 registers
// of packed inputs per thread instead of 32 of fp32 results, which is what lets 8 CTAs
// share an SM; the extra ex2 work rides on an otherwise idle pipe.
template <> struct RowVec<__half> : RowVec16<__half2, __half> {
  static __device__ __forceinline__ uint4 scaled(const uint4 &raw, float, float neg_m_log2e,
                                                 float r) {
    const __half *e = reinterpret_cast<const __half *>(&raw);
    uint4 out;
    __half2 *o = reinterpret_cast<__half2 *>(&out);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = __floats2half2_rn(e2(e[2 * j], neg_m_log2e) * r, e2(e[2 * j + 1], neg_m_log2e) * r);
    return out;
  }
};
template <> struct RowVec<__nv_bfloat16> : RowVec16<__nv_bfloat162, __nv_bfloat16> {
  static __device__ __forceinline__ uint4 scaled(const uint4 &raw, float, float neg_m_log2e,
                                                 float r) {
    const __nv_bfloat16 *e = reinterpret_cast<const __nv_bfloat16 *>(&raw);
    uint4 out;
    __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(&out);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = __floats2bfloat162_rn(e2(e[2 * j], neg_m_log2e) * r,
                                   e2(e[2 * j + 1], neg_m_log2e) * r);
    return out;
  }
};

template <typename T, int G, int VPT>
__global__ void __launch_bounds__((G > kRowThreads ? G : kRowThreads),
                                  (G > kRowThreads ? 1 : 8))
softmax_rows_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows,
                    int cols, int mask_kind, int64_t row_offset) {
  constexpr int kThreads = G > kRowThreads ? G : kRowThreads;
  constexpr int kRowsPerCta = kThreads / G;
  using V = RowVec<T>;
  constexpr int N = V::N;
  __shared__ float scratch[2 * (kThreads / 32)];

  const int lane = threadIdx.x % G;
  const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + threadIdx.x / G;
  const bool row_ok = row < rows;
  const int nvec = cols / N;
  // kept columns of this row: [0, keep); vectors [0, full_vec) are kept whole,
  // vector full_vec (if keep % N != 0) partly, everything after is masked
  int keep = cols;
  if (mask_kind == B200_MASK_CAUSAL_MOD && row_ok)
    keep = (int)((row_offset + row) % cols) + 1;
  const int full_vec = keep / N;
  const int kept_vec = row_ok ? (keep + N - 1) / N : 0;

  // the kept part of the row is loaded once and stays in registers; the masked
  // part is never loaded and costs no arithmetic
  uint4 raw[VPT];
  float m = -INFINITY;
  const T *xrow = x + row * (int64_t)cols;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    if (v < kept_vec) {
      raw[i] = ld_stream16(xrow + (int64_t)v * N);
      if (v >= full_vec) V::mask_tail(raw[i], keep - v * N);
      m = fmaxf(m, V::vmax(raw[i]));
    }
  }
  m = group_reduce<G, MaxOp>(m, scratch, 0);
  const float neg_m_log2e = -m * 1.4426950408889634f;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    if (v < kept_vec) s += V::expsum(raw[i], m, neg_m_log2e);
  }
  s = group_reduce<G, SumOp>(s, scratch, 1);
  const float r = 1.0f / s;

  T *yrow = y + row * (int64_t)cols;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    if (row_ok && v < nvec) {
      const uint4 out =
          v < kept_vec ? V::scaled(raw[i], m, neg_m_log2e, r) : make_uint4(0u, 0u, 0u, 0u);
      st_stream16(yrow + (int64_t)v * N, out);
    }
  }
}

// Any width / alignment: one CTA per row, three scalar passes (the row is
// re-read from L2).  Used for ragged widths such as 97.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
softmax_loop_kernel(const T *__restrict__ x, T *__restrict__ y, int cols,
                    int mask_kind, int64_t row_offset) {
  __shared__ float scratch[2 * (kRowThreads / 32)];
  const int64_t row = blockIdx.x;
  int keep = cols;
  if (mask_kind == B200_MASK_CAUSAL_MOD) keep = (int)((row_offset + row) % cols) + 1;
  const T *xrow = x + row * (int64_t)cols;
  T *yrow = y + row * (int64_t)cols;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < keep; c += kRowThreads) m = fmaxf(m, io<T>::load(xrow[c]));
  m = group_reduce<kRowThreads, MaxOp>(m, scratch, 0);
  float s = 0.f;
  for (int c = threadIdx.x; c < keep; c += kRowThreads)
    s += fast_exp<T>(io<T>::load(xrow[c]) - m);
  s = group_reduce<kRowThreads, SumOp>(s, scratch, 1);
  const float r = 1.0f / s;
  for (int c = threadIdx.x; c < cols; c += kRowThreads)
    yrow[c] = io<T>::store(c < keep ? fast_exp<T>(io<T>::load(xrow[c]) - m) * r : 0.f);
}

template <typename T, int G, int VPT>
static void launch_rows(const b200_tensor *x, b200_tensor *y, int mask_kind,
                        int64_t row_offset, cudaStream_t stream) {
  constexpr int kThreads = G > kRowThreads ? G : kRowThreads;
  constexpr int kRowsPerCta = kThreads / G;
  const int64_t rows = x->shape[0];
  const unsigned grid = (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta);
  softmax_rows_kernel<T, G, VPT><<<grid, kThreads, 0, stream>>>(
      (const T *)x->data, (T *)y->data, rows, (int)x->shape[1], mask_kind, row_offset);
}

template <typename T>
static int dispatch(const b200_tensor *x, b200_tensor *y, int mask_kind,
                    int64_t row_offset, cudaStream_t stream) {
  constexpr int N = vec16<T>::N;
  constexpr int VPT = 4;
  const int64_t rows = x->shape[0], cols = x->shape[1];
  const bool aligned = cols % N == 0 && ((uintptr_t)x->data % 16) == 0 &&
                       ((uintptr_t)y->data % 16) == 0;
  const int g = aligned ? pick_group(cols / N, VPT) : 0;
  switch (g) {
    case 8: launch_rows<T, 8, VPT>(x, y, mask_kind, row_offset, stream); break;
    case 16: launch_rows<T, 16, VPT>(x, y, mask_kind, row_offset, stream); break;
    case 32: launch_rows<T, 32, VPT>(x, y, mask_kind, row_offset, stream); break;
    case 64: launch_rows<T, 64, VPT>(x, y, mask_kind, row_offset, stream); break;
    case 128: launch_rows<T, 128, VPT>(x, y, mask_kind, row_offset, stream); break;
    case 256: launch_rows<T, 256, VPT>(x, y, mask_kind, row_offset, stream); break;
    case 512: launch_rows<T, 512, VPT>(x, y, mask_kind, row_offset, stream); break;
    case 1024: launch_rows<T, 1024, VPT>(x, y, mask_kind, row_offset, stream); break;
    default:
      softmax_loop_kernel<T><<<(unsigned)rows, kRowThreads, 0, stream>>>(
          (const T *)x->data, (T *)y->data, (int)cols, mask_kind, row_offset);
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

extern "C" int b200_softmax_fwd(const b200_tensor *x, b200_tensor *y, int mask_kind,
                                int64_t row_offset, void *stream) {
  using namespace b200;
  int st;
  if ((st = check_tensor(x, "x", 2)) || (st = check_tensor(y, "y", 2))) return st;
  if (mask_kind != B200_MASK_NONE && mask_kind != B200_MASK_CAUSAL_MOD)
    return fail(B200_USAGE, "mask_kind %d is not a b200_mask value", mask_kind);
  B200_REQUIRE(is_float_io(x->dtype), "x: dtype %u is not f16/bf16/f32", x->dtype);
  B200_REQUIRE(y->dtype == x->dtype, "x/y dtypes differ (%u/%u)", x->dtype, y->dtype);
  const int64_t rows = x->shape[0], cols = x->shape[1];
  B200_REQUIRE(y->shape[0] == rows && y->shape[1] == cols, "y shape differs from x");
  B200_REQUIRE(x->stride[1] == 1 && y->stride[1] == 1 &&
               (rows <= 1 || (x->stride[0] == cols && y->stride[0] == cols)),
               "x/y must be contiguous [rows, cols] (row*n_cols addressing)");
  B200_REQUIRE(cols > 0 && cols < (1 << 30), "row width %lld out of range", (long long)cols);
  B200_REQUIRE(rows < (1LL << 31), "too many rows");
  B200_REQUIRE(row_offset >= 0, "row_offset must be non-negative");
  if (rows == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (x->dtype) {
    case B200_DTYPE_FLOAT32: return dispatch<float>(x, y, mask_kind, row_offset, s);
    case B200_DTYPE_FLOAT16: return dispatch<__half>(x, y, mask_kind, row_offset, s);
    default: return dispatch<__nv_bfloat16>(x, y, mask_kind, row_offset, s);
  }
}
