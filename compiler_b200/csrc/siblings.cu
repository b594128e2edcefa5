// Sibling operators of the five families: the elementwise GELU / GEGLU / epilogue kernels and
// the softmax variants of the reference's corpus.  All are HBM-bound one-pass kernels; they
// exist so that the harness lanes of these families run through the same launch surface.
#include "rowwise.cuh"

namespace b200 {

__device__ __forceinline__ float gelu_erf_f(float z) {
  return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f));
}
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// out[i] = f(a[i], b[i]) over a flat range; OP is a b200_ewise code.
//   GELU_ERF              0.5 x (1 + erf(x / sqrt 2))                     (ops/suite/perf/gelu.py:21-27)
//   ADD_GELU_ERF          gelu_erf(x + p0 * o)                            (ops/suite/perf/add_gelu.py:21-30)
//   GEGLU_TANH            gelu_tanh(a) * b                                (ops/suite/perf/geglu_tanh_triton.py:19-37)
//   BIAS_SCALE_CLAMP_GELU gelu_erf(clamp((x + bias[i % n_cols]) * p0, p1, p2))
//                                                                         (ops/suite/dev/epilogue_kernel.py:24-32)
template <typename T, int OP>
__global__ void __launch_bounds__(256)
elementwise_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ out,
                   int64_t n, int64_t n_cols, float p0, float p1, float p2) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float x = io<T>::load(a[i]);
    float y;
    if constexpr (OP == B200_EW_GELU_ERF) {
      y = gelu_erf_f(x);
    } else if constexpr (OP == B200_EW_ADD_GELU_ERF) {
      y = gelu_erf_f(x + p0 * io<T>::load(b[i]));
    } else if constexpr (OP == B200_EW_GEGLU_TANH) {
      y = gelu_tanh_f(x) * io<T>::load(b[i]);
    } else {
      float z = (x + io<T>::load(b[i % n_cols])) * p0;
      z = fminf(fmaxf(z, p1), p2);
      y = gelu_erf_f(z);
    }
    out[i] = io<T>::store(y);
  }
}

template <typename T>
static int launch_elementwise(int op, const void *a, const void *b, void *out, int64_t n,
                              int64_t n_cols, float p0, float p1, float p2, cudaStream_t s) {
  int64_t blocks = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
#define B200_EW(OP)                                                                          \
  elementwise_kernel<T, OP><<<(unsigned)blocks, 256, 0, s>>>((const T *)a, (const T *)b,     \
                                                             (T *)out, n, n_cols, p0, p1, p2)
  switch (op) {
    case B200_EW_GELU_ERF: B200_EW(B200_EW_GELU_ERF); break;
    case B200_EW_ADD_GELU_ERF: B200_EW(B200_EW_ADD_GELU_ERF); break;
    case B200_EW_GEGLU_TANH: B200_EW(B200_EW_GEGLU_TANH); break;
    default: B200_EW(B200_EW_BIAS_SCALE_CLAMP_GELU); break;
  }
#undef B200_EW
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

// Row softmax variants, one CTA per row, scalar passes (rows re-read from L2):
//   mul != nullptr : y = softmax(x) * mul                    (ops/suite/perf/softmax_mul.py:21-32)
//   log_input      : y = softmax(log x); a NaN in log x makes the whole row NaN, like
//                    max() over the row does in the reference's oracle
//                                                            (ops/suite/perf/softmax_log.py:20-40)
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
softmax_variant_kernel(const T *__restrict__ x, const T *__restrict__ mul, T *__restrict__ y,
                       int cols, int log_input) {
  __shared__ float scratch[2 * (kRowThreads / 32)];
  const int64_t row = blockIdx.x;
  const T *xrow = x + row * (int64_t)cols;
  const T *mrow = mul ? mul + row * (int64_t)cols : nullptr;
  T *yrow = y + row * (int64_t)cols;
  float m = -INFINITY, nan_seen = 0.f;
  for (int c = threadIdx.x; c < cols; c += kRowThreads) {
    float z = io<T>::load(xrow[c]);
    if (log_input) z = logf(z);
    if (z != z) nan_seen = 1.f;
    m = fmaxf(m, z);
  }
  m = group_reduce<kRowThreads, MaxOp>(m, scratch, 0);
  nan_seen = group_reduce<kRowThreads, MaxOp>(nan_seen, scratch, 1);
  if (nan_seen != 0.f) m = __int_as_float(0x7fc00000);
  float s = 0.f;
  for (int c = threadIdx.x; c < cols; c += kRowThreads) {
    float z = io<T>::load(xrow[c]);
    if (log_input) z = logf(z);
    s += expf(z - m);
  }
  s = group_reduce<kRowThreads, SumOp>(s, scratch, 0);
  for (int c = threadIdx.x; c < cols; c += kRowThreads) {
    float z = io<T>::load(xrow[c]);
    if (log_input) z = logf(z);
    float v = expf(z - m) / s;
    if (mrow) v *= io<T>::load(mrow[c]);
    yrow[c] = io<T>::store(v);
  }
}

// y[row, p] = x[row, p / R] - logsumexp_p(x[row, p / R]), p in [0, L)
// (ops/suite/perf/fused_repeat_interleave_log_softmax.py:19-31)
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
repeat_log_softmax_kernel(const T *__restrict__ x, T *__restrict__ y, int cols, int repeat,
                          int length) {
  __shared__ float scratch[2 * (kRowThreads / 32)];
  const int64_t row = blockIdx.x;
  const T *xrow = x + row * (int64_t)cols;
  T *yrow = y + row * (int64_t)length;
  float m = -INFINITY;
  for (int p = threadIdx.x; p < length; p += kRowThreads) m = fmaxf(m, io<T>::load(xrow[p / repeat]));
  m = group_reduce<kRowThreads, MaxOp>(m, scratch, 0);
  float s = 0.f;
  for (int p = threadIdx.x; p < length; p += kRowThreads) s += expf(io<T>::load(xrow[p / repeat]) - m);
  s = group_reduce<kRowThreads, SumOp>(s, scratch, 1);
  const float lse = m + logf(s);
  for (int p = threadIdx.x; p < length; p += kRowThreads)
    yrow[p] = io<T>::store(io<T>::load(xrow[p / repeat]) - lse);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_elementwise(int op, const b200_tensor *a, const b200_tensor *b,
                                b200_tensor *out, float p0, float p1, float p2, void *stream) {
  int st;
  if ((st = check_tensor(a, "a", 1)) || (st = check_tensor(out, "out", 1))) return st;
  if (op < B200_EW_GELU_ERF || op > B200_EW_BIAS_SCALE_CLAMP_GELU)
    return fail(B200_USAGE, "op %d is not a b200_ewise value", op);
  B200_REQUIRE(is_float_io(a->dtype) && out->dtype == a->dtype, "a/out must share f16/bf16/f32");
  B200_REQUIRE(a->stride[0] == 1 && out->stride[0] == 1 && out->shape[0] == a->shape[0],
               "a/out must be contiguous and of equal length");
  const int64_t n = a->shape[0];
  int64_t n_cols = 1;
  if (op != B200_EW_GELU_ERF) {
    if (b == nullptr) return fail(B200_USAGE, "op %d needs the second operand", op);
    if ((st = check_tensor(b, "b", 1))) return st;
    B200_REQUIRE(b->dtype == a->dtype && b->stride[0] == 1, "b must match a's dtype, contiguous");
    if (op == B200_EW_BIAS_SCALE_CLAMP_GELU) {
      n_cols = b->shape[0];
      B200_REQUIRE(n_cols > 0 && n % n_cols == 0, "bias length %lld does not divide %lld elements",
                   (long long)n_cols, (long long)n);
    } else {
      B200_REQUIRE(b->shape[0] == n, "b length differs from a");
    }
  }
  if (n == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const void *bp = b ? b->data : nullptr;
  switch (a->dtype) {
    case B200_DTYPE_FLOAT32:
      return launch_elementwise<float>(op, a->data, bp, out->data, n, n_cols, p0, p1, p2, s);
    case B200_DTYPE_FLOAT16:
      return launch_elementwise<__half>(op, a->data, bp, out->data, n, n_cols, p0, p1, p2, s);
    default:
      return launch_elementwise<__nv_bfloat16>(op, a->data, bp, out->data, n, n_cols, p0, p1, p2, s);
  }
}

extern "C" int b200_softmax_variant(const b200_tensor *x, const b200_tensor *mul, b200_tensor *y,
                                    int log_input, void *stream) {
  int st;
  if ((st = check_tensor(x, "x", 2)) || (st = check_tensor(y, "y", 2))) return st;
  if (mul != nullptr && (st = check_tensor(mul, "mul", 2))) return st;
  B200_REQUIRE(is_float_io(x->dtype) && y->dtype == x->dtype, "x/y must share f16/bf16/f32");
  const int64_t rows = x->shape[0], cols = x->shape[1];
  B200_REQUIRE(y->shape[0] == rows && y->shape[1] == cols, "y shape differs from x");
  B200_REQUIRE(x->stride[1] == 1 && y->stride[1] == 1 &&
               (rows <= 1 || (x->stride[0] == cols && y->stride[0] == cols)),
               "x/y must be contiguous [rows, cols]");
  if (mul != nullptr)
    B200_REQUIRE(mul->dtype == x->dtype && mul->shape[0] == rows && mul->shape[1] == cols &&
                 mul->stride[1] == 1 && (rows <= 1 || mul->stride[0] == cols),
                 "mul must match x in dtype, shape and layout");
  B200_REQUIRE(cols > 0 && cols < (1 << 30) && rows < (1LL << 31), "extent out of range");
  if (rows == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
#define B200_SV(T)                                                                         \
  softmax_variant_kernel<T><<<(unsigned)rows, kRowThreads, 0, s>>>(                        \
      (const T *)x->data, mul ? (const T *)mul->data : nullptr, (T *)y->data, (int)cols,   \
      log_input ? 1 : 0)
  if (x->dtype == B200_DTYPE_FLOAT32) B200_SV(float);
  else if (x->dtype == B200_DTYPE_FLOAT16) B200_SV(__half);
  else B200_SV(__nv_bfloat16);
#undef B200_SV
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

extern "C" int b200_repeat_log_softmax(const b200_tensor *x, b200_tensor *y, int repeat,
                                       void *stream) {
  int st;
  if ((st = check_tensor(x, "x", 2)) || (st = check_tensor(y, "y", 2))) return st;
  B200_REQUIRE(is_float_io(x->dtype) && y->dtype == x->dtype, "x/y must share f16/bf16/f32");
  const int64_t rows = x->shape[0], cols = x->shape[1], length = y->shape[1];
  B200_REQUIRE(y->shape[0] == rows, "row counts differ");
  B200_REQUIRE(repeat >= 1 && length >= 1 && length <= cols * (int64_t)repeat,
               "output length %lld exceeds cols * repeat", (long long)length);
  B200_REQUIRE(x->stride[1] == 1 && y->stride[1] == 1 &&
               (rows <= 1 || (x->stride[0] == cols && y->stride[0] == length)),
               "x/y must be contiguous");
  B200_REQUIRE(cols < (1 << 30) && length < (1 << 30) && rows < (1LL << 31), "extent out of range");
  if (rows == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
#define B200_RL(T)                                                                  \
  repeat_log_softmax_kernel<T><<<(unsigned)rows, kRowThreads, 0, s>>>(              \
      (const T *)x->data, (T *)y->data, (int)cols, repeat, (int)length)
  if (x->dtype == B200_DTYPE_FLOAT32) B200_RL(float);
  else if (x->dtype == B200_DTYPE_FLOAT16) B200_RL(__half);
  else B200_RL(__nv_bfloat16);
#undef B200_RL
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

// ---- int8 weights -> floats: out[k, n] = b[k, n] * scale[n] --------------------------------
// dequantize_kernel (ops/suite/perf/dequantize_matmul.py:27-40).  One thread converts 16
// consecutive columns (one 16-byte load of int8, 16-byte stores) when the rows allow it.
namespace b200 {
namespace {

template <typename T>
__global__ void __launch_bounds__(256)
dequantize_kernel(const int8_t *__restrict__ b, int64_t ldb, const T *__restrict__ scale,
                  T *__restrict__ out, int64_t ldo, int K, int N, int vector_ok) {
  const int groups = (N + 15) / 16;
  const int64_t total = (int64_t)K * groups;
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < total; i += (int64_t)gridDim.x * 256) {
    const int k = (int)(i / groups), n0 = (int)(i % groups) * 16;
    const int8_t *src = b + (int64_t)k * ldb + n0;
    T *dst = out + (int64_t)k * ldo + n0;
    if (vector_ok && n0 + 16 <= N) {
      const uint4 raw = ld_stream16(src);
      const int8_t *q = reinterpret_cast<const int8_t *>(&raw);
      constexpr int PER = 16 / (int)sizeof(T);
#pragma unroll
      for (int v = 0; v < 16 / PER; ++v) {
        vec16<T> o;
#pragma unroll
        for (int j = 0; j < PER; ++j)
          o.e[j] = io<T>::store((float)q[v * PER + j] * io<T>::load(scale[n0 + v * PER + j]));
        *reinterpret_cast<uint4 *>(dst + v * PER) = o.raw;
      }
    } else {
      for (int j = 0; j < 16 && n0 + j < N; ++j)
        dst[j] = io<T>::store((float)src[j] * io<T>::load(scale[n0 + j]));
    }
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_dequantize_cols(const b200_tensor *b, const b200_tensor *scale, b200_tensor *out,
                                    void *stream) {
  using namespace b200;
  int st;
  if ((st = check_tensor(b, "b", 2)) || (st = check_tensor(scale, "scale", 1)) ||
      (st = check_tensor(out, "out", 2)))
    return st;
  B200_REQUIRE(b->dtype == B200_DTYPE_INT8, "b must be int8");
  B200_REQUIRE(is_float_io(out->dtype) && scale->dtype == out->dtype,
               "scale and out must share f16/bf16/f32");
  const int64_t K = b->shape[0], N = b->shape[1];
  B200_REQUIRE(out->shape[0] == K && out->shape[1] == N && scale->shape[0] == N &&
               scale->stride[0] == 1, "out must be [K,N] and scale contiguous [N]");
  B200_REQUIRE(b->stride[1] == 1 && out->stride[1] == 1 && b->stride[0] >= N && out->stride[0] >= N,
               "b and out need unit column stride");
  B200_REQUIRE(K < (1LL << 31) && N < (1LL << 31), "extent out of range");
  if (K == 0 || N == 0) return B200_OK;
  const size_t es = dtype_size(out->dtype);
  const int vector_ok = (uintptr_t)b->data % 16 == 0 && b->stride[0] % 16 == 0 &&
                        (uintptr_t)out->data % 16 == 0 && (out->stride[0] * es) % 16 == 0;
  const int64_t work = K * ((N + 15) / 16);
  int64_t blocks = (work + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = (cudaStream_t)stream;
#define B200_DQ(T)                                                                              \
  dequantize_kernel<T><<<(unsigned)blocks, 256, 0, s>>>((const int8_t *)b->data, b->stride[0],  \
                                                        (const T *)scale->data, (T *)out->data, \
                                                        out->stride[0], (int)K, (int)N, vector_ok)
  if (out->dtype == B200_DTYPE_FLOAT32) B200_DQ(float);
  else if (out->dtype == B200_DTYPE_FLOAT16) B200_DQ(__half);
  else B200_DQ(__nv_bfloat16);
#undef B200_DQ
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}
