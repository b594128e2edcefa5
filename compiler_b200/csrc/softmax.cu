// Row softmax with an index-computed mask, for sm_100a.
//
// Semantics follow softmax_kernel (ops/suite/perf/softmax.py:20-31): fp32
// row max, e = exp(x - max), y = e / sum(e), one rounding at the store.  With
// B200_MASK_CAUSAL_MOD the columns col > (row_offset + row) % n_cols are
// treated as -inf exactly like `tl.where(offs_n <= pid_m, qk, -inf)`
// (ops/suite/perf/attn_fwd_causal.py:46-47): they add 0 to the sum and are
// written as 0.  Column 0 is always kept, so no row is fully masked.
//
// HBM-bound: the row stays in registers between max, sum and the store (the
// exponentials are computed once, in fp32); the masked part of a row is never
// loaded (its output is a constant 0), so the DRAM read traffic is below the
// algorithmic 2 B/element of an fp16 read.  The same kernel serves the variants
// softmax(x) * mul and softmax(log x) of the reference's corpus.
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
  // e[j] = exp(x[j] - m) (log_input: x[j] holds log x already); returns their sum
  static __device__ __forceinline__ float exps(const uint4 &raw, float m, float, float (&e)[N]) {
    const float *x = reinterpret_cast<const float *>(&raw);
#pragma unroll
    for (int j = 0; j < N; ++j) e[j] = expf(x[j] - m);
    return (e[0] + e[1]) + (e[2] + e[3]);
  }
  static __device__ __forceinline__ void unpack(const uint4 &raw, float (&f)[N]) {
    const float *x = reinterpret_cast<const float *>(&raw);
#pragma unroll
    for (int j = 0; j < N; ++j) f[j] = x[j];
  }
  // e[j] * r (* mul[j]) in the storage type
  static __device__ __forceinline__ uint4 scaled(const float (&e)[N], float r, const uint4 *mul) {
    uint4 out;
    float *o = reinterpret_cast<float *>(&out);
    const float *w = reinterpret_cast<const float *>(mul);
#pragma unroll
    for (int j = 0; j < N; ++j) o[j] = mul ? e[j] * r * w[j] : e[j] * r;
    return out;
  }
};

__device__ __forceinline__ float2 pair_to_float2(__half2 v) { return __half22float2(v); }
__device__ __forceinline__ float2 pair_to_float2(__nv_bfloat162 v) {
  const uint32_t w = *reinterpret_cast<const uint32_t *>(&v);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

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
  // e[j] = 2^(x[j] * log2e - m * log2e); returns their sum.  The multiply-add and the running
  // sum take two elements per instruction (fp32x2), the ex2 one each.
  static __device__ __forceinline__ float exps(const uint4 &raw, float, float neg_m_log2e,
                                               float (&e)[N]) {
    const T2 *x = reinterpret_cast<const T2 *>(&raw);
    float2 s = make_float2(0.f, 0.f);
#pragma unroll
    for (int j = 0; j < N / 2; ++j) {
      const float2 t = fma2(pair_to_float2(x[j]), splat(1.4426950408889634f), splat(neg_m_log2e));
      const float2 v = make_float2(ex2_approx(t.x), ex2_approx(t.y));
      e[2 * j] = v.x;
      e[2 * j + 1] = v.y;
      s = add2(s, v);
    }
    return s.x + s.y;
  }
  static __device__ __forceinline__ void unpack(const uint4 &raw, float (&f)[N]) {
    const T1 *x = reinterpret_cast<const T1 *>(&raw);
#pragma unroll
    for (int j = 0; j < N; ++j) f[j] = io<T1>::load(x[j]);
  }
};
// The exponentials are computed once, in fp32, and kept for the store: the packed inputs
// are dead after that pass, so a thread holds 32 fp32 results instead of 16 packed words.
template <> struct RowVec<__half> : RowVec16<__half2, __half> {
  static __device__ __forceinline__ uint4 scaled(const float (&e)[8], float r, const uint4 *mul) {
    uint4 out;
    __half2 *o = reinterpret_cast<__half2 *>(&out);
    const __half2 *w = reinterpret_cast<const __half2 *>(mul);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 v = mul2(make_float2(e[2 * j], e[2 * j + 1]), splat(r));
      if (mul) v = mul2(v, pair_to_float2(w[j]));
      o[j] = __floats2half2_rn(v.x, v.y);
    }
    return out;
  }
};
template <> struct RowVec<__nv_bfloat16> : RowVec16<__nv_bfloat162, __nv_bfloat16> {
  static __device__ __forceinline__ uint4 scaled(const float (&e)[8], float r, const uint4 *mul) {
    uint4 out;
    __nv_bfloat162 *o = reinterpret_cast<__nv_bfloat162 *>(&out);
    const __nv_bfloat162 *w = reinterpret_cast<const __nv_bfloat162 *>(mul);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 v = mul2(make_float2(e[2 * j], e[2 * j + 1]), splat(r));
      if (mul) v = mul2(v, pair_to_float2(w[j]));
      o[j] = __floats2bfloat162_rn(v.x, v.y);
    }
    return out;
  }
};

// (row_offset + row) % cols.  The kept width of a masked row stands before its loads, and a
// 64-bit remainder is a long dependent sequence: take the 32-bit one whenever the row index fits.
__device__ __forceinline__ int row_mod(int64_t index, int cols) {
  if (index < ((int64_t)1 << 32)) return (int)((uint32_t)index % (uint32_t)cols);
  return (int)(index % cols);
}

// MODE: the plain (optionally masked) softmax, softmax(x) * mul, or softmax(log x).
constexpr int kSoftmaxPlain = 0, kSoftmaxMul = 1, kSoftmaxLog = 2;

// softmax(log x) needs no logarithm: log is monotone, so max(log x) = log(max x) and
// exp(log x - log max) = x / max.  What the logarithm adds is its domain: a negative or NaN
// input makes log x NaN and, through the row maximum, the whole row NaN
// (ops/suite/perf/softmax_log.py:27-31); all-zero and infinite rows come out NaN by the
// arithmetic itself (0 / 0, inf / inf), as they do in the reference.
//
// KEEP: the exponentials are computed once, in fp32, and kept for the store (32 registers of
// results per thread for 16-bit rows, four CTAs of 256 threads per SM).  Without it they are
// recomputed for the store from the 16 registers of packed inputs, which lets eight CTAs share
// an SM: the choice for masked rows, where half of the row on average is never loaded or
// exponentiated and the kernel lives on the loads in flight.
template <typename T, int G, int VPT, int MODE, bool KEEP>
__global__ void __launch_bounds__((G > kRowThreads ? G : kRowThreads),
                                  (G > kRowThreads ? (KEEP ? 1 : 2048 / G) : (KEEP ? 4 : 8)))
softmax_rows_kernel(const T *__restrict__ x, const T *__restrict__ mul, T *__restrict__ y,
                    int64_t rows, int cols, int mask_kind, int64_t row_offset) {
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
  if (MODE == kSoftmaxPlain && mask_kind == B200_MASK_CAUSAL_MOD && row_ok)
    keep = row_mod(row_offset + row, cols) + 1;
  const int full_vec = keep / N;
  const int kept_vec = row_ok ? (keep + N - 1) / N : 0;

  // the kept part of the row is loaded once; the masked part is never loaded and costs
  // no arithmetic
  static_assert(KEEP || MODE == kSoftmaxPlain, "the variants keep their exponentials");
  uint4 raw[VPT];
  float e[KEEP ? VPT : 1][N];
  float m = -INFINITY;
  bool bad = false;
  const T *xrow = x + row * (int64_t)cols;
  T *yrow = y + row * (int64_t)cols;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    // the zeros of the masked columns depend on nothing: they leave while the loads are in
    // flight, instead of queueing behind both reductions with the rest of the row
    if (MODE == kSoftmaxPlain && row_ok && v >= kept_vec && v < nvec)
      st_stream16(yrow + (int64_t)v * N, make_uint4(0u, 0u, 0u, 0u));
    if (v < kept_vec) {
      raw[i] = ld_stream16(xrow + (int64_t)v * N);
      if constexpr (MODE == kSoftmaxLog) {
        V::unpack(raw[i], e[i]);
#pragma unroll
        for (int j = 0; j < N; ++j) {
          bad = bad || !(e[i][j] >= 0.f);
          m = fmaxf(m, e[i][j]);
        }
      } else {
        if (v >= full_vec) V::mask_tail(raw[i], keep - v * N);
        m = fmaxf(m, V::vmax(raw[i]));
      }
    }
  }
  if constexpr (MODE == kSoftmaxLog) {
    if (bad) m = INFINITY;  // poisons the row below: x * (1 / inf) sums to 0, 0 * inf = NaN
  }
  m = group_reduce<G, MaxOp>(m, scratch, 0);
  const float neg_m_log2e = -m * 1.4426950408889634f;
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    if (v < kept_vec) {
      if constexpr (MODE == kSoftmaxLog) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
          e[i][j] = sizeof(T) == 4 ? e[i][j] / m : e[i][j] * (1.0f / m);
          s += e[i][j];
        }
      } else {
        s += V::exps(raw[i], m, neg_m_log2e, e[KEEP ? i : 0]);
      }
    }
  }
  s = group_reduce<G, SumOp>(s, scratch, 1);
  float r = 1.0f / s;
  if constexpr (MODE == kSoftmaxLog) {
    if (m == INFINITY) r = __int_as_float(0x7fc00000);  // a NaN, negative or infinite input
  }

  if constexpr (MODE == kSoftmaxMul) {
    const T *mrow = mul + row * (int64_t)cols;
    uint4 w[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      if (v < kept_vec) w[i] = ld_stream16(mrow + (int64_t)v * N);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      if (v < kept_vec) st_stream16(yrow + (int64_t)v * N, V::scaled(e[i], r, &w[i]));
    }
  } else {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      if (v < kept_vec) {
        if constexpr (!KEEP) V::exps(raw[i], m, neg_m_log2e, e[0]);
        st_stream16(yrow + (int64_t)v * N, V::scaled(e[KEEP ? i : 0], r, nullptr));
      }
    }
  }
}

// The unmasked forms for many rows: a persistent CTA walks down the rows and has the
// next row's vectors in flight while it reduces, exponentiates and stores the current one, so
// the load latency is hidden by the arithmetic of the row before instead of by other CTAs.
// Three CTAs of 256 threads per SM (the two rows in flight per thread take about 80 registers),
// two for the form with the multiplier, which also holds that row's vectors.
constexpr int stream_ctas_per_sm(int mode) { return mode == kSoftmaxMul ? 2 : 3; }

// Rows of more than 256 x VPT vectors (G = 512 or 1024 threads): the CTA is the group, one row
// at a time with the next one in flight, in the LEAN form only (its 63 registers are what 1024
// threads leave each other); two CTAs per SM at 512 threads, one at 1024.  Before, such rows
// had one row in flight per SM and nothing to hide its load -> max -> sum -> store chain behind:
// fp16 [4096,16384] ran at 3.4 TB/s, [2048,32768] at 2.8 TB/s.
constexpr int stream_threads(int g) { return g > kRowThreads ? g : kRowThreads; }
constexpr int stream_lean_ctas_per_sm(int g) { return g > 512 ? 1 : (g > kRowThreads ? 2 : 4); }

template <typename T, int G, int VPT, int MODE, bool LEAN = false>
__global__ void __launch_bounds__(stream_threads(G),
                                  LEAN ? stream_lean_ctas_per_sm(G) : stream_ctas_per_sm(MODE))
softmax_stream_kernel(const T *__restrict__ x, const T *__restrict__ mul, T *__restrict__ y,
                      int64_t rows, int cols, int mask_kind, int64_t row_offset) {
  static_assert(G <= kRowThreads || LEAN, "wide rows take the lean form");
  constexpr int kThreads = G > kRowThreads ? G : kRowThreads;
  constexpr int kRowsPerCta = kThreads / G;
  using V = RowVec<T>;
  constexpr int N = V::N;
  __shared__ float scratch[2 * (kThreads / 32)];

  const int lane = threadIdx.x % G;
  const int nvec = cols / N;
  const int64_t stride = (int64_t)gridDim.x * kRowsPerCta;
  int64_t row = (int64_t)blockIdx.x * kRowsPerCta + threadIdx.x / G;
  // masked rows: row r keeps its first (row_offset + r) % cols + 1 columns; the remainder is
  // taken once and then advanced by the stride between this group's rows
  const bool masked = MODE == kSoftmaxPlain && mask_kind == B200_MASK_CAUSAL_MOD;
  const int step_mod = masked ? row_mod(stride, cols) : 0;
  int keep_next = masked ? row_mod(row_offset + row, cols) + 1 : cols;

  uint4 next[VPT];
  if (row < rows) {
    const int kv = (keep_next + N - 1) / N;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      if (v < kv) next[i] = ld_stream16(x + row * (int64_t)cols + (int64_t)v * N);
    }
  }
  for (; row < rows; row += stride) {
    const int keep = keep_next;
    const int full_vec = keep / N;
    const int kept_vec = (keep + N - 1) / N;
    if (masked) {
      keep_next += step_mod;  // keep - 1 is the remainder: stay in [1, cols]
      if (keep_next > cols) keep_next -= cols;
    }
    uint4 raw[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) raw[i] = next[i];
    if (row + stride < rows) {
      const T *ahead = x + (row + stride) * (int64_t)cols;
      const int kv = (keep_next + N - 1) / N;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = lane + i * G;
        if (v < kv) next[i] = ld_stream16(ahead + (int64_t)v * N);
      }
    }
    uint4 w[MODE == kSoftmaxMul ? VPT : 1];
    if constexpr (MODE == kSoftmaxMul) {
      const T *mrow = mul + row * (int64_t)cols;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = lane + i * G;
        if (v < nvec) w[i] = ld_stream16(mrow + (int64_t)v * N);
      }
    }

    // LEAN: the exponentials are taken again for the store instead of being kept (16 packed
    // registers per row in flight instead of 48): four CTAs per SM
    float e[LEAN ? 1 : VPT][N];
    float m = -INFINITY;
    bool bad = false;
    T *yrow = y + row * (int64_t)cols;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      // the zeros of the masked columns depend on nothing
      if (masked && v >= kept_vec && v < nvec)
        st_stream16(yrow + (int64_t)v * N, make_uint4(0u, 0u, 0u, 0u));
      if (v < kept_vec) {
        if constexpr (MODE == kSoftmaxLog) {
          V::unpack(raw[i], e[i]);
#pragma unroll
          for (int j = 0; j < N; ++j) {
            bad = bad || !(e[i][j] >= 0.f);
            m = fmaxf(m, e[i][j]);
          }
        } else {
          if (masked && v >= full_vec) V::mask_tail(raw[i], keep - v * N);
          m = fmaxf(m, V::vmax(raw[i]));
        }
      }
    }
    if constexpr (MODE == kSoftmaxLog) {
      if (bad) m = INFINITY;
    }
    m = group_reduce<G, MaxOp>(m, scratch, 0);
    const float neg_m_log2e = -m * 1.4426950408889634f;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      if (v < kept_vec) {
        if constexpr (MODE == kSoftmaxLog) {
#pragma unroll
          for (int j = 0; j < N; ++j) {
            e[i][j] = sizeof(T) == 4 ? e[i][j] / m : e[i][j] * (1.0f / m);
            s += e[i][j];
          }
        } else {
          s += V::exps(raw[i], m, neg_m_log2e, e[LEAN ? 0 : i]);
        }
      }
    }
    s = group_reduce<G, SumOp>(s, scratch, 1);
    float r = 1.0f / s;
    if constexpr (MODE == kSoftmaxLog) {
      if (m == INFINITY) r = __int_as_float(0x7fc00000);
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      if (v < kept_vec) {
        if constexpr (LEAN) V::exps(raw[i], m, neg_m_log2e, e[0]);
        st_stream16(yrow + (int64_t)v * N,
                    V::scaled(e[LEAN ? 0 : i], r,
                              MODE == kSoftmaxMul ? &w[MODE == kSoftmaxMul ? i : 0] : nullptr));
      }
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

template <typename T, int G, int VPT, int MODE, bool KEEP>
static void launch_rows(const b200_tensor *x, const b200_tensor *mul, b200_tensor *y,
                        int mask_kind, int64_t row_offset, cudaStream_t stream) {
  constexpr int kThreads = G > kRowThreads ? G : kRowThreads;
  constexpr int kRowsPerCta = kThreads / G;
  const int64_t rows = x->shape[0];
  const unsigned grid = (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta);
  if constexpr (G <= kRowThreads) {
    // more than one wave of resident CTAs: the pipelined persistent forms
    // (B200OPS_SOFTMAX_STREAM=0 keeps the one-row-per-group kernel for everything, 2 sends
    // masked rows through the pipelined form of the unmasked ones, 3 sends unmasked rows
    // through the lean form of the masked ones)
    static const int choice =
        getenv("B200OPS_SOFTMAX_STREAM") ? atoi(getenv("B200OPS_SOFTMAX_STREAM")) : 1;
    // masked rows, more than one wave: the pipelined form that takes the exponentials again
    // for the store (63 registers, four CTAs per SM): 34.6 us at 16384 x 4000 fp16 against
    // 38.6 us for the one-row-per-group kernel and 42.8 us for the pipelined form that keeps
    // them (B200OPS_SOFTMAX_STREAM=0 / 2 select those)
    if constexpr (MODE == kSoftmaxPlain) {
      if ((choice == 3 || (choice == 1 && mask_kind == B200_MASK_CAUSAL_MOD)) &&
          grid > (unsigned)(sm_count() * 4)) {
        softmax_stream_kernel<T, G, VPT, MODE, true><<<sm_count() * 4, kRowThreads, 0, stream>>>(
            (const T *)x->data, nullptr, (T *)y->data, rows, (int)x->shape[1], mask_kind,
            row_offset);
        return;
      }
    }
    const unsigned resident = (unsigned)(sm_count() * stream_ctas_per_sm(MODE));
    const bool take = choice == 2 || (choice == 1 && mask_kind == B200_MASK_NONE);
    if (take && grid > resident) {
      softmax_stream_kernel<T, G, VPT, MODE><<<resident, kRowThreads, 0, stream>>>(
          (const T *)x->data, mul ? (const T *)mul->data : nullptr, (T *)y->data, rows,
          (int)x->shape[1], mask_kind, row_offset);
      return;
    }
  } else if constexpr (MODE == kSoftmaxPlain) {
    // Rows of 512 / 1024 threads' width, by measurement.  Unmasked, more rows than resident
    // CTAs: the pipelined lean form with the CTA as the group (fp16 [2048,32768] 4.9 TB/s,
    // fp32 [2048,16384] 5.4 against 4.4 / 4.1 for the form below).  Masked, or few rows: the
    // one-row-per-CTA form that takes its exponentials again for the store -- it fits 32
    // registers, so two CTAs of 1024 threads (four of 512) share an SM and overlap each
    // other's load -> max -> sum -> store chains, and masked rows, which differ in length, gain
    // more from that than from a prefetched next row (fp16 [2048,32768] masked 4.7 TB/s in
    // bytes that move against 4.3; [4096,16384] 5.6 against 5.1).  The form that keeps its
    // exponentials leaves a CTA alone on its SM (3.0 TB/s) and is not used for these widths.
    // B200OPS_SOFTMAX_STREAM=0: never the pipelined form; 4: also for masked rows.
    static const int choice =
        getenv("B200OPS_SOFTMAX_STREAM") ? atoi(getenv("B200OPS_SOFTMAX_STREAM")) : 1;
    const unsigned resident = (unsigned)(sm_count() * stream_lean_ctas_per_sm(G));
    const bool pipelined = choice == 4 || (choice != 0 && mask_kind == B200_MASK_NONE);
    if (pipelined && grid > resident) {
      softmax_stream_kernel<T, G, VPT, MODE, true><<<resident, kThreads, 0, stream>>>(
          (const T *)x->data, nullptr, (T *)y->data, rows, (int)x->shape[1], mask_kind,
          row_offset);
      return;
    }
    softmax_rows_kernel<T, G, VPT, MODE, false><<<grid, kThreads, 0, stream>>>(
        (const T *)x->data, nullptr, (T *)y->data, rows, (int)x->shape[1], mask_kind,
        row_offset);
    return;
  }
  softmax_rows_kernel<T, G, VPT, MODE, KEEP><<<grid, kThreads, 0, stream>>>(
      (const T *)x->data, mul ? (const T *)mul->data : nullptr, (T *)y->data, rows,
      (int)x->shape[1], mask_kind, row_offset);
}

// true when the register-resident kernel took the row shape; false: the caller runs its
// looping kernel
template <typename T, int MODE, bool KEEP>
static bool dispatch_rows(const b200_tensor *x, const b200_tensor *mul, b200_tensor *y,
                          int mask_kind, int64_t row_offset, cudaStream_t stream) {
  constexpr int N = vec16<T>::N;
  constexpr int VPT = 4;
  const int64_t cols = x->shape[1];
  const bool aligned = cols % N == 0 && ((uintptr_t)x->data % 16) == 0 &&
                       ((uintptr_t)y->data % 16) == 0 &&
                       (mul == nullptr || ((uintptr_t)mul->data % 16) == 0);
  const int g = aligned ? pick_group(cols / N, VPT) : 0;
  switch (g) {
    case 8: launch_rows<T, 8, VPT, MODE, KEEP>(x, mul, y, mask_kind, row_offset, stream); break;
    case 16: launch_rows<T, 16, VPT, MODE, KEEP>(x, mul, y, mask_kind, row_offset, stream); break;
    case 32: launch_rows<T, 32, VPT, MODE, KEEP>(x, mul, y, mask_kind, row_offset, stream); break;
    case 64: launch_rows<T, 64, VPT, MODE, KEEP>(x, mul, y, mask_kind, row_offset, stream); break;
    case 128: launch_rows<T, 128, VPT, MODE, KEEP>(x, mul, y, mask_kind, row_offset, stream); break;
    case 256: launch_rows<T, 256, VPT, MODE, KEEP>(x, mul, y, mask_kind, row_offset, stream); break;
    case 512: launch_rows<T, 512, VPT, MODE, KEEP>(x, mul, y, mask_kind, row_offset, stream); break;
    case 1024: launch_rows<T, 1024, VPT, MODE, KEEP>(x, mul, y, mask_kind, row_offset, stream); break;
    default: return false;
  }
  return true;
}

template <typename T>
static int dispatch(const b200_tensor *x, b200_tensor *y, int mask_kind,
                    int64_t row_offset, cudaStream_t stream) {
  const bool taken =
      mask_kind == B200_MASK_NONE
          ? dispatch_rows<T, kSoftmaxPlain, true>(x, nullptr, y, mask_kind, row_offset, stream)
          : dispatch_rows<T, kSoftmaxPlain, false>(x, nullptr, y, mask_kind, row_offset, stream);
  bool clustered = false;
  if (!taken && ((uintptr_t)x->data % 16) == 0 && ((uintptr_t)y->data % 16) == 0) {
    // wider than one CTA holds in registers: a cluster per row
    const int st = softmax_cluster_rows<T>(x, y, mask_kind, row_offset, stream, &clustered);
    if (st != B200_OK) return st;
  }
  if (!taken && !clustered)
    softmax_loop_kernel<T><<<(unsigned)x->shape[0], kRowThreads, 0, stream>>>(
        (const T *)x->data, (T *)y->data, (int)x->shape[1], mask_kind, row_offset);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

// softmax(x) * mul and softmax(log x) for rows that fit the register-resident kernel;
// returns false (nothing launched) for the others
bool softmax_variant_rows(const b200_tensor *x, const b200_tensor *mul, b200_tensor *y,
                          int log_input, cudaStream_t stream) {
#define B200_SVR(T)                                                                      \
  (log_input ? dispatch_rows<T, kSoftmaxLog, true>(x, nullptr, y, B200_MASK_NONE, 0, stream)  \
             : dispatch_rows<T, kSoftmaxMul, true>(x, mul, y, B200_MASK_NONE, 0, stream))
  if (mul == nullptr && !log_input) return false;
  if (mul != nullptr && log_input) return false;
  if (x->dtype == B200_DTYPE_FLOAT32) return B200_SVR(float);
  if (x->dtype == B200_DTYPE_FLOAT16) return B200_SVR(__half);
  return B200_SVR(__nv_bfloat16);
#undef B200_SVR
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
