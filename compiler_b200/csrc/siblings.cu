// Sibling operators of the five families: the elementwise GELU / GEGLU / epilogue kernels and
// the softmax variants of the reference's corpus.  All are HBM-bound one-pass kernels; they
// exist so that the harness lanes of these families run through the same launch surface.
#include "rowwise.cuh"

namespace b200 {

// softmax.cu: the register-resident row kernel in its mul / log forms
bool softmax_variant_rows(const b200_tensor *x, const b200_tensor *mul, b200_tensor *y,
                          int log_input, cudaStream_t stream);

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
                   int64_t n, int64_t n_cols, float p0, float p1, float p2, int64_t first) {
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
      float z = (x + io<T>::load(b[(first + i) % n_cols])) * p0;
      z = fminf(fmaxf(z, p1), p2);
      y = gelu_erf_f(z);
    }
    out[i] = io<T>::store(y);
  }
}

// erf for 16-bit results: Abramowitz-Stegun 7.1.26, |error| <= 1.5e-7 (a 16-bit result
// carries 8 or 11 bits), one reciprocal and one ex2 instead of erff's polynomial pair.
__device__ __forceinline__ float erf_short(float x) {
  const float ax = fabsf(x);
  float t, e;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(fmaf(0.3275911f, ax, 1.0f)));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * ax * ax));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  return copysignf(fmaf(-poly * t, e, 1.0f), x);
}
template <typename T> __device__ __forceinline__ float gelu_erf_t(float z) {
  if constexpr (sizeof(T) == 4) return gelu_erf_f(z);
  return z * fmaf(0.5f, erf_short(z * 0.7071067811865476f), 0.5f);
}
template <typename T> __device__ __forceinline__ float gelu_tanh_t(float z) {
  if constexpr (sizeof(T) == 4) return gelu_tanh_f(z);
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  return 0.5f * z * (1.0f + t);
}

constexpr int kEwSwiglu = 100;  // internal: x * sigmoid(x) * b (b200_swiglu_fwd on contiguous rows)

// The erf-based GELUs on 16-bit data are bound by instruction issue and by the special-function
// unit, not by memory -- a 16-bit element is half the bytes for the same arithmetic.  Two
// things cut the work: the packed fp32x2 forms (common.cuh: fma2 / mul2) halve the
// multiply-add count at full fp32 precision, and the complementary error function is taken as
// ONE exponential of a polynomial, erfc(a sqrt 2) = 2^P(a), P of degree 5 without a constant
// term (fitted on a in [0, 3.2] against erfc weighted by erfc itself: |error| of erf
// <= 7e-7, a 16-bit result carries 8 or 11 bits; the leading coefficient is negative, so P keeps
// falling beyond the fitted range and 2^P goes to 0) -- one ex2 per element and no reciprocal,
// against Abramowitz-Stegun's reciprocal + ex2 + degree-4 polynomial above.
// With h = z / 2 and E = erf(|z| / sqrt 2) = 1 - 2^P(|h|):  gelu(z) = h + |h| E.
__device__ __forceinline__ float2 gelu_erf_short2(float2 z) {
  const float2 h = mul2(z, splat(0.5f));
  const float2 ah = make_float2(fabsf(h.x), fabsf(h.y));
  float2 p = fma2(ah, splat(-0.016686532646417618f), splat(0.1184384673833847f));
  p = fma2(p, ah, splat(-0.4205521047115326f));
  p = fma2(p, ah, splat(-1.837000846862793f));
  p = fma2(p, ah, splat(-2.3021841049194336f));
  p = mul2(p, ah);
  float2 e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(p.x));
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(p.y));
  const float2 big_e = fma2(e, splat(-1.0f), splat(1.0f));
  return fma2(ah, big_e, h);
}

// The operators that have a packed form (16-bit data only): pairs of elements.
template <typename T, int OP> constexpr bool ew_packed() {
  return sizeof(T) == 2 && (OP == B200_EW_GELU_ERF || OP == B200_EW_ADD_GELU_ERF ||
                            OP == B200_EW_BIAS_SCALE_CLAMP_GELU);
}
template <int OP>
__device__ __forceinline__ float2 ew_apply2(float2 x, float2 o, float p0, float p1, float p2) {
  if constexpr (OP == B200_EW_GELU_ERF) return gelu_erf_short2(x);
  if constexpr (OP == B200_EW_ADD_GELU_ERF) return gelu_erf_short2(fma2(o, splat(p0), x));
  float2 z = mul2(make_float2(x.x + o.x, x.y + o.y), splat(p0));
  z.x = fminf(fmaxf(z.x, p1), p2);
  z.y = fminf(fmaxf(z.y, p1), p2);
  return gelu_erf_short2(z);
}
template <typename T> __device__ __forceinline__ float2 unpack_pair(uint32_t w);
template <> __device__ __forceinline__ float2 unpack_pair<__nv_bfloat16>(uint32_t w) {
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <> __device__ __forceinline__ float2 unpack_pair<__half>(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2 *>(&w));
}
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float2 v);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float2 v) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
  return *reinterpret_cast<const uint32_t *>(&h);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float2 v) {
  const __half2 h = __floats2half2_rn(v.x, v.y);
  return *reinterpret_cast<const uint32_t *>(&h);
}

template <typename T, int OP> __device__ __forceinline__ float ew_apply(float x, float o, float p0,
                                                                        float p1, float p2) {
  if constexpr (OP == B200_EW_GELU_ERF) return gelu_erf_t<T>(x);
  if constexpr (OP == B200_EW_ADD_GELU_ERF) return gelu_erf_t<T>(x + p0 * o);
  if constexpr (OP == B200_EW_GEGLU_TANH) return gelu_tanh_t<T>(x) * o;
  if constexpr (OP == kEwSwiglu) {
    if constexpr (sizeof(T) == 4) return x / (1.0f + __expf(-x)) * o;
    return __fdividef(x, 1.0f + __expf(-x)) * o;
  }
  const float z = fminf(fmaxf((x + o) * p0, p1), p2);
  return gelu_erf_t<T>(z);
}

// The same operators on 16-byte vectors: every thread has U vectors of each operand in
// flight before it starts on the arithmetic.  a, b, out 16-byte aligned; the bias of
// BIAS_SCALE_CLAMP_GELU is n_cols long with n_cols a multiple of the vector length, so a
// vector never wraps.  Elements past the last whole vector are left to the caller.
template <typename T, int OP, int U>
__global__ void __launch_bounds__(256)
elementwise_vec_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ out,
                       int64_t nvec, int64_t n_cols, float p0, float p1, float p2) {
  constexpr int N = vec16<T>::N;
  constexpr bool kHasB = OP != B200_EW_GELU_ERF;
  constexpr bool kBias = OP == B200_EW_BIAS_SCALE_CLAMP_GELU;
  const int64_t tile = 256 * U;
  // BIAS_SCALE_CLAMP_GELU: the bias column of a vector is (v * N) % n_cols.  One remainder per
  // thread, before the loop; after that the column advances by constants (the 256 vectors
  // between a thread's slots, the grid's stride between its tiles) with a conditional
  // subtraction -- a 64-bit remainder per vector costs more than the GELU.
  int64_t col0 = 0, slot_step = 0, tile_step = 0;
  if constexpr (kBias) {
    col0 = (((int64_t)blockIdx.x * tile + threadIdx.x) * N) % n_cols;
    slot_step = ((int64_t)256 * N) % n_cols;
    tile_step = (((int64_t)gridDim.x * tile) % n_cols * N) % n_cols;
  }
  for (int64_t base = (int64_t)blockIdx.x * tile; base < nvec; base += (int64_t)gridDim.x * tile) {
    vec16<T> va[U], vb[U];
    int64_t col = col0;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = base + u * 256 + threadIdx.x;
      if (v < nvec) {
        va[u].raw = ld_stream16(a + v * N);
        if constexpr (kBias) {
          vb[u].raw = __ldg(reinterpret_cast<const uint4 *>(b + col));
        } else if constexpr (kHasB) {
          vb[u].raw = ld_stream16(b + v * N);
        }
      }
      if constexpr (kBias) {
        col += slot_step;
        if (col >= n_cols) col -= n_cols;
      }
    }
    if constexpr (kBias) {
      col0 += tile_step;
      if (col0 >= n_cols) col0 -= n_cols;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t v = base + u * 256 + threadIdx.x;
      if (v < nvec) {
        vec16<T> o;
        if constexpr (ew_packed<T, OP>()) {
          const uint32_t *wa = reinterpret_cast<const uint32_t *>(&va[u].raw);
          const uint32_t *wb = reinterpret_cast<const uint32_t *>(&vb[u].raw);
          uint32_t *wo = reinterpret_cast<uint32_t *>(&o.raw);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            wo[j] = pack_pair<T>(ew_apply2<OP>(
                unpack_pair<T>(wa[j]), kHasB ? unpack_pair<T>(wb[j]) : make_float2(0.f, 0.f), p0,
                p1, p2));
        } else {
#pragma unroll
          for (int j = 0; j < N; ++j)
            o.e[j] = io<T>::store(ew_apply<T, OP>(io<T>::load(va[u].e[j]),
                                                  kHasB ? io<T>::load(vb[u].e[j]) : 0.f, p0, p1, p2));
        }
        st_stream16(out + v * N, o.raw);
      }
    }
  }
}

template <typename T, int OP>
static void launch_elementwise_op(const T *a, const T *b, T *out, int64_t n, int64_t n_cols,
                                  float p0, float p1, float p2, cudaStream_t s) {
  constexpr int N = vec16<T>::N;
  constexpr int U = 4;
  const bool vec_ok = (uintptr_t)a % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                      (b == nullptr || (uintptr_t)b % 16 == 0) &&
                      (OP != B200_EW_BIAS_SCALE_CLAMP_GELU || n_cols % N == 0);
  const int64_t nvec = vec_ok ? n / N : 0;
  if (nvec > 0) {
    int64_t blocks = (nvec + 256 * U - 1) / (256 * U);
    const int64_t cap = (int64_t)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    elementwise_vec_kernel<T, OP, U><<<(unsigned)blocks, 256, 0, s>>>(a, b, out, nvec, n_cols, p0,
                                                                    p1, p2);
  }
  const int64_t done = nvec * N;
  if (done < n) {
    // the ragged end (or everything, for unaligned operands): scalar kernel
    if constexpr (OP != kEwSwiglu) {
      const int64_t rest = n - done;
      int64_t blocks = (rest + 255) / 256;
      const int64_t cap = (int64_t)sm_count() * 16;
      if (blocks > cap) blocks = cap;
      const T *bb = b;
      if (OP != B200_EW_BIAS_SCALE_CLAMP_GELU && b != nullptr) bb = b + done;
      // done is a multiple of n_cols' vector length, not of n_cols: the bias index of the
      // scalar kernel is (done + i) % n_cols, which its `first` argument carries
      elementwise_kernel<T, OP><<<(unsigned)blocks, 256, 0, s>>>(a + done, bb, out + done, rest,
                                                                 n_cols, p0, p1, p2, done);
    }
  }
}

template <typename T>
static int launch_elementwise(int op, const void *a, const void *b, void *out, int64_t n,
                              int64_t n_cols, float p0, float p1, float p2, cudaStream_t s) {
#define B200_EW(OP) \
  launch_elementwise_op<T, OP>((const T *)a, (const T *)b, (T *)out, n, n_cols, p0, p1, p2, s)
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

// x * sigmoid(x) * y over a flat contiguous range (elementwise.cu: b200_swiglu_fwd);
// n must be a multiple of the 16-byte vector length and the pointers 16-byte aligned
void swiglu_flat(uint32_t dtype, const void *x, const void *y, void *out, int64_t n,
                 cudaStream_t s) {
  if (dtype == B200_DTYPE_FLOAT32)
    launch_elementwise_op<float, kEwSwiglu>((const float *)x, (const float *)y, (float *)out, n, 1,
                                            0.f, 0.f, 0.f, s);
  else if (dtype == B200_DTYPE_FLOAT16)
    launch_elementwise_op<__half, kEwSwiglu>((const __half *)x, (const __half *)y, (__half *)out,
                                             n, 1, 0.f, 0.f, 0.f, s);
  else
    launch_elementwise_op<__nv_bfloat16, kEwSwiglu>((const __nv_bfloat16 *)x,
                                                    (const __nv_bfloat16 *)y,
                                                    (__nv_bfloat16 *)out, n, 1, 0.f, 0.f, 0.f, s);
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

// The same with 16-byte loads and stores: the input row is read twice (the second time from
// L1 / L2) and every output vector is assembled from the one or two inputs it repeats.  A row
// belongs to a group of G threads (256 / G rows per CTA), sized so that a thread has about four
// output vectors.  x rows and y rows 16-byte aligned, cols and length multiples of the vector
// length.
template <typename T, int G>
__global__ void __launch_bounds__(kRowThreads)
repeat_log_softmax_vec_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows, int cols,
                              int repeat, int length) {
  constexpr int N = vec16<T>::N;
  __shared__ float scratch[2 * (kRowThreads / 32)];
  const int lane = threadIdx.x % G;
  const int64_t row = (int64_t)blockIdx.x * (kRowThreads / G) + threadIdx.x / G;
  if (row >= rows) return;  // the whole group leaves: its barrier has no other member
  const T *xrow = x + row * (int64_t)cols;
  T *yrow = y + row * (int64_t)length;
  const int used = (length + repeat - 1) / repeat;  // inputs that reach the output
  const int in_vec = (used + N - 1) / N;
  float m = -INFINITY;
  for (int v = lane; v < in_vec; v += G) {
    vec16<T> a;
    a.raw = __ldg(reinterpret_cast<const uint4 *>(xrow) + v);
#pragma unroll
    for (int j = 0; j < N; ++j)
      if (v * N + j < used) m = fmaxf(m, io<T>::load(a.e[j]));
  }
  m = group_reduce<G, MaxOp>(m, scratch, 0);
  float s = 0.f;
  for (int v = lane; v < in_vec; v += G) {
    vec16<T> a;
    a.raw = __ldg(reinterpret_cast<const uint4 *>(xrow) + v);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const int c = v * N + j;
      // input c is repeated `repeat` times, the last used one possibly fewer
      const int count = min(repeat, length - c * repeat);
      if (c < used) s += (float)count * expf(io<T>::load(a.e[j]) - m);
    }
  }
  s = group_reduce<G, SumOp>(s, scratch, 1);
  const float lse = m + logf(s);
  const int out_vec = length / N;
  for (int v = lane; v < out_vec; v += G) {
    int c = (v * N) / repeat;
    int rem = (v * N) - c * repeat;
    float cur = io<T>::load(xrow[c]) - lse;
    vec16<T> o;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      o.e[j] = io<T>::store(cur);
      if (++rem == repeat) {
        rem = 0;
        ++c;
        if (j + 1 < N && c < cols) cur = io<T>::load(xrow[c]) - lse;
      }
    }
    st_stream16(yrow + (int64_t)v * N, o.raw);
  }
}

// Short input rows (at most one 16-byte vector per thread of the group): the vector stays in
// registers between the maximum and the sum, and the row goes to shared memory as floats once,
// so the output pass reads its repeated inputs from there instead of from global memory.
template <typename T, int G, int REP>
__global__ void __launch_bounds__(kRowThreads)
repeat_log_softmax_cached_kernel(const T *__restrict__ x, T *__restrict__ y, int64_t rows,
                                 int cols, int repeat, int length) {
  constexpr int N = vec16<T>::N;
  constexpr int kRows = kRowThreads / G;
  __shared__ float scratch[2 * (kRowThreads / 32)];
  __shared__ float cache[kRows][G * N];  // the used part of each row
  const int lane = threadIdx.x % G;
  const int group = threadIdx.x / G;
  const int64_t row = (int64_t)blockIdx.x * kRows + group;
  if (row >= rows) return;  // the whole group leaves: its barrier has no other member
  const T *xrow = x + row * (int64_t)cols;
  T *yrow = y + row * (int64_t)length;
  const int used = (length + repeat - 1) / repeat;  // inputs that reach the output, <= G * N
  float f[N];
  float m = -INFINITY;
  if (lane * N < used) {
    vec16<T> a;
    a.raw = ld_stream16(xrow + lane * N);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      f[j] = io<T>::load(a.e[j]);
      cache[group][lane * N + j] = f[j];
      if (lane * N + j < used) m = fmaxf(m, f[j]);
    }
  }
  m = group_reduce<G, MaxOp>(m, scratch, 0);
  float s = 0.f;
  if (lane * N < used) {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const int c = lane * N + j;
      const int count = min(repeat, length - c * repeat);  // the last used input may repeat less
      if (c < used) s += (float)count * (sizeof(T) == 4 ? expf(f[j] - m) : __expf(f[j] - m));
    }
  }
  // the reduction's barrier also publishes the cached row to the whole group
  s = group_reduce<G, SumOp>(s, scratch, 1);
  if constexpr (G <= 32) __syncwarp();
  const float lse = m + logf(s);
  const int out_vec = length / N;
  if constexpr (REP > 0) {
    // REP divides the vector length and the output length: an output vector is N / REP
    // cached inputs, each written REP times -- no division, no running remainder
    constexpr int kIn = N / REP;
    for (int v = lane; v < out_vec; v += G) {
      vec16<T> o;
#pragma unroll
      for (int i = 0; i < kIn; ++i) {
        const T value = io<T>::store(cache[group][v * kIn + i] - lse);
#pragma unroll
        for (int j = 0; j < REP; ++j) o.e[i * REP + j] = value;
      }
      st_stream16(yrow + (int64_t)v * N, o.raw);
    }
    return;
  }
  for (int v = lane; v < out_vec; v += G) {
    int c = (v * N) / repeat;
    int rem = (v * N) - c * repeat;
    float cur = cache[group][c] - lse;
    vec16<T> o;
#pragma unroll
    for (int j = 0; j < N; ++j) {
      o.e[j] = io<T>::store(cur);
      if (++rem == repeat) {
        rem = 0;
        ++c;
        if (j + 1 < N && c < used) cur = cache[group][c] - lse;
      }
    }
    st_stream16(yrow + (int64_t)v * N, o.raw);
  }
}

template <typename T>
static void launch_repeat_vec(const b200_tensor *x, b200_tensor *y, int repeat, cudaStream_t s) {
  constexpr int N = vec16<T>::N;
  const int64_t rows = x->shape[0];
  const int cols = (int)x->shape[1], length = (int)y->shape[1];
  const int out_vec = length / N;
#define B200_RLV(G)                                                                         \
  repeat_log_softmax_vec_kernel<T, G><<<(unsigned)((rows + kRowThreads / G - 1) / (kRowThreads / G)), \
                                        kRowThreads, 0, s>>>((const T *)x->data, (T *)y->data, rows, \
                                                             cols, repeat, length)
  const int used = (length + repeat - 1) / repeat;
  // the repeat count as a compile-time constant when it divides the vector and the row
  const int rep = (length % repeat == 0 && N % repeat == 0 && repeat > 1) ? repeat : 0;
#define B200_RLC_R(G, R)                                                                    \
  repeat_log_softmax_cached_kernel<T, G, R><<<(unsigned)((rows + kRowThreads / G - 1) / (kRowThreads / G)), \
                                              kRowThreads, 0, s>>>((const T *)x->data, (T *)y->data, rows, \
                                                                   cols, repeat, length)
#define B200_RLC(G)                                                                         \
  do {                                                                                      \
    if (rep == 2) B200_RLC_R(G, 2);                                                         \
    else if (rep == 4) B200_RLC_R(G, 4);                                                    \
    else if (rep == 8 && N == 8) B200_RLC_R(G, (N == 8 ? 8 : 0));                           \
    else B200_RLC_R(G, 0);                                                                  \
  } while (0)
  // the cached form when a group's threads hold the used inputs in one vector each
  if (out_vec <= 32 * 4) { if (used <= 32 * N) B200_RLC(32); else B200_RLV(32); }
  else if (out_vec <= 64 * 4) { if (used <= 64 * N) B200_RLC(64); else B200_RLV(64); }
  else if (out_vec <= 128 * 4) { if (used <= 128 * N) B200_RLC(128); else B200_RLV(128); }
  else if (used <= 256 * N) B200_RLC(256);
  else B200_RLV(256);
#undef B200_RLC
#undef B200_RLC_R
#undef B200_RLV
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
  if (softmax_variant_rows(x, mul, y, log_input, s)) {
    B200_CUDA_OK(cudaGetLastError());
    return B200_OK;
  }
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
  const size_t es = dtype_size(x->dtype);
  const int64_t per_vec = 16 / (int64_t)es;
  const bool vec_ok = (uintptr_t)x->data % 16 == 0 && (uintptr_t)y->data % 16 == 0 &&
                      cols % per_vec == 0 && length % per_vec == 0;
#define B200_RL(T)                                                                      \
  do {                                                                                  \
    if (vec_ok)                                                                         \
      launch_repeat_vec<T>(x, y, repeat, s);                                            \
    else                                                                                \
      repeat_log_softmax_kernel<T><<<(unsigned)rows, kRowThreads, 0, s>>>(              \
          (const T *)x->data, (T *)y->data, (int)cols, repeat, (int)length);            \
  } while (0)
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

// Byte `lane` of `biased` (an int8 with its sign bit flipped, i.e. value + 128) as a float:
// the byte is placed into the low mantissa bits of 2^23 (one byte permute) and 2^23 + 128 is
// subtracted -- exact, and on the full-rate pipes instead of the integer-to-float converter.
__device__ __forceinline__ float int8_lane_to_float(uint32_t biased, int lane) {
  return __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7440u + (uint32_t)lane)) - 8388736.0f;
}

// The aligned case: a thread owns the columns of one 16-byte output vector (8 for 16-bit
// results, 4 for fp32), keeps their scales in registers and walks down the rows (blockIdx.y
// strides over them, eight rows in flight), so there is no index division, the scales are read
// once per thread, and a warp reads and writes whole contiguous segments of a row.
template <typename T>
__global__ void __launch_bounds__(256)
dequantize_cols_kernel(const int8_t *__restrict__ b, int64_t ldb, const T *__restrict__ scale,
                       T *__restrict__ out, int64_t ldo, int K, int groups) {
  constexpr int PER = 16 / (int)sizeof(T);
  constexpr int R = 8;
  const int g = blockIdx.x * 256 + threadIdx.x;
  if (g >= groups) return;
  const int n0 = g * PER;
  float sc[PER];
#pragma unroll
  for (int j = 0; j < PER; ++j) sc[j] = io<T>::load(scale[n0 + j]);
  for (int k0 = blockIdx.y * R; k0 < K; k0 += gridDim.y * R) {
    uint32_t raw[R][PER / 4];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (k0 + r < K) {
        const int8_t *src = b + (int64_t)(k0 + r) * ldb + n0;
        if constexpr (PER == 8) {
          const uint2 t = __ldg(reinterpret_cast<const uint2 *>(src));
          raw[r][0] = t.x;
          raw[r][1] = t.y;
        } else {
          raw[r][0] = __ldg(reinterpret_cast<const uint32_t *>(src));
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (k0 + r >= K) break;
      vec16<T> o;
#pragma unroll
      for (int j = 0; j < PER; ++j)
        // sign bit flipped: the byte becomes value + 128 as unsigned
        o.e[j] = io<T>::store(int8_lane_to_float(raw[r][j >> 2] ^ 0x80808080u, j & 3) * sc[j]);
      st_stream16(out + (int64_t)(k0 + r) * ldo + n0, o.raw);
    }
  }
}

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
  const bool by_columns = vector_ok && N % 16 == 0;  // N > 0 here, so at least one group
  const int groups = (int)(N / (16 / (int64_t)es));  // one 16-byte output vector per thread
  const unsigned gx = by_columns ? (unsigned)((groups + 255) / 256) : 1u;
  int64_t gy = ((int64_t)sm_count() * 8 + gx - 1) / gx;
  if (gy > (K + 7) / 8) gy = (K + 7) / 8;
  if (gy > 65535) gy = 65535;
#define B200_DQ(T)                                                                              \
  do {                                                                                          \
    if (by_columns)                                                                             \
      dequantize_cols_kernel<T><<<dim3(gx, (unsigned)gy), 256, 0, s>>>(                         \
          (const int8_t *)b->data, b->stride[0], (const T *)scale->data, (T *)out->data,        \
          out->stride[0], (int)K, groups);                                                      \
    else                                                                                        \
      dequantize_kernel<T><<<(unsigned)blocks, 256, 0, s>>>(                                    \
          (const int8_t *)b->data, b->stride[0], (const T *)scale->data, (T *)out->data,        \
          out->stride[0], (int)K, (int)N, vector_ok);                                           \
  } while (0)
  if (out->dtype == B200_DTYPE_FLOAT32) B200_DQ(float);
  else if (out->dtype == B200_DTYPE_FLOAT16) B200_DQ(__half);
  else B200_DQ(__nv_bfloat16);
#undef B200_DQ
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}
