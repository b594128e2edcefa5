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

template <typename T, int G, int VPT>
__global__ void __launch_bounds__((G > kRowThreads ? G : kRowThreads))
softmax_rows_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows,
                    int cols, int mask_kind, int64_t row_offset) {
  constexpr int kThreads = G > kRowThreads ? G : kRowThreads;
  constexpr int kRowsPerCta = kThreads / G;
  constexpr int N = vec16<T>::N;
  __shared__ float scratch[kThreads / 32];

  const int lane = threadIdx.x % G;
  const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + threadIdx.x / G;
  const bool row_ok = row < rows;
  const int nvec = cols / N;
  // number of kept columns in this row: [0, keep)
  int keep = cols;
  if (mask_kind == B200_MASK_CAUSAL_MOD && row_ok)
    keep = (int)((row_offset + row) % cols) + 1;
  const int kept_vec = (keep + N - 1) / N;

  float f[VPT][N];
  float m = -INFINITY;
  const T *xrow = x + row * (int64_t)cols;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    if (row_ok && v < kept_vec) {
      vec16<T> xv;
      xv.raw = ld_stream16(xrow + (int64_t)v * N);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        f[i][j] = (v * N + j < keep) ? io<T>::load(xv.e[j]) : -INFINITY;
        m = fmaxf(m, f[i][j]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) f[i][j] = -INFINITY;
    }
  }
  m = group_reduce<G, MaxOp>(m, scratch);
  // a row whose kept values are all -inf would give inf-inf: keep it NaN like
  // the numpy formula does; with finite inputs m is finite here.
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i)
#pragma unroll
    for (int j = 0; j < N; ++j) {
      f[i][j] = fast_exp<T>(f[i][j] - m);
      s += f[i][j];
    }
  s = group_reduce<G, SumOp>(s, scratch);
  const float r = 1.0f / s;

  T *yrow = y + row * (int64_t)cols;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    if (row_ok && v < nvec) {
      vec16<T> out;
#pragma unroll
      for (int j = 0; j < N; ++j) out.e[j] = io<T>::store(f[i][j] * r);
      st_stream16(yrow + (int64_t)v * N, out.raw);
    }
  }
}

// Any width / alignment: one CTA per row, three scalar passes (the row is
// re-read from L2).  Used for ragged widths such as 97.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
softmax_loop_kernel(const T *__restrict__ x, T *__restrict__ y, int cols,
                    int mask_kind, int64_t row_offset) {
  __shared__ float scratch[kRowThreads / 32];
  const int64_t row = blockIdx.x;
  int keep = cols;
  if (mask_kind == B200_MASK_CAUSAL_MOD) keep = (int)((row_offset + row) % cols) + 1;
  const T *xrow = x + row * (int64_t)cols;
  T *yrow = y + row * (int64_t)cols;
  float m = -INFINITY;
  for (int c = threadIdx.x; c < keep; c += kRowThreads) m = fmaxf(m, io<T>::load(xrow[c]));
  m = group_reduce<kRowThreads, MaxOp>(m, scratch);
  float s = 0.f;
  for (int c = threadIdx.x; c < keep; c += kRowThreads)
    s += fast_exp<T>(io<T>::load(xrow[c]) - m);
  s = group_reduce<kRowThreads, SumOp>(s, scratch);
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
