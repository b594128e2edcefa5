// RMSNorm forward for sm_100a.
//
// Semantics follow rms_layernorm_forward_kernel
// (ops/suite/perf/fast_rms_layernorm.py:19-44): fp32 accumulation of x*x over
// the row, inv = rsqrt(sum/n_cols + eps), y = (x*inv)*w, r[row] = inv, one
// rounding to the storage type at the store.
//
// HBM-bound: the row lives in registers between the reduction and the scale,
// so X is read once and Y written once (8 B/element for fp32).  Loads are
// 128-bit, streaming (no L1 allocation); stores are 128-bit, evict-first.
#include "rowwise.cuh"

namespace b200 {

// Rows of 512 / 1024 threads' width: at most 32 registers, so that CTAs fill the SM's 2048
// threads (the bfloat16 form took 48 and left a 1024-thread CTA alone on its SM).
template <typename T, int G, int VPT>
__global__ void __launch_bounds__((G > kRowThreads ? G : kRowThreads),
                                  (G > kRowThreads ? 2048 / G : 1))
rmsnorm_rows_kernel(const T *__restrict__ x, int64_t x_stride,
                    const T *__restrict__ w, T *__restrict__ y, int64_t y_stride,
                    T *__restrict__ rinv, int64_t rows, int cols, float eps, float gamma_offset) {
  constexpr int kThreads = G > kRowThreads ? G : kRowThreads;
  constexpr int kRowsPerCta = kThreads / G;
  constexpr int N = vec16<T>::N;
  __shared__ float scratch[2 * (kThreads / 32)];

  const int lane = threadIdx.x % G;
  const int64_t row = (int64_t)blockIdx.x * kRowsPerCta + threadIdx.x / G;
  const bool row_ok = row < rows;
  const int nvec = cols / N;

  vec16<T> xv[VPT];
  float acc = 0.f;
  const T *xrow = x + row * x_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    if (row_ok && v < nvec) {
      xv[i].raw = ld_stream16(xrow + (int64_t)v * N);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float f = io<T>::load(xv[i].e[j]);
        acc = fmaf(f, f, acc);
      }
    }
  }
  acc = group_reduce<G, SumOp>(acc, scratch, 0);
  const float inv = 1.0f / sqrtf(acc / (float)cols + eps);
  if (row_ok && lane == 0 && rinv != nullptr) rinv[row] = io<T>::store(inv);

  T *yrow = y + row * y_stride;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = lane + i * G;
    if (row_ok && v < nvec) {
      vec16<T> wv, out;
      wv.raw = *reinterpret_cast<const uint4 *>(w + (int64_t)v * N);
#pragma unroll
      for (int j = 0; j < N; ++j)
        out.e[j] = io<T>::store(io<T>::load(xv[i].e[j]) * inv * (io<T>::load(wv.e[j]) + gamma_offset));
      st_stream16(yrow + (int64_t)v * N, out.raw);
    }
  }
}

// Rows of 1024 threads' width, more rows than resident CTAs: a persistent CTA walks down the
// rows with the next row's vectors in flight while it reduces, scales and stores the current
// one.  Used for 32-bit rows only (see launch_rows).
template <typename T, int G, int VPT>
__global__ void __launch_bounds__(G, G > 512 ? 1 : 2)
rmsnorm_stream_kernel(const T *__restrict__ x, int64_t x_stride, const T *__restrict__ w,
                      T *__restrict__ y, int64_t y_stride, T *__restrict__ rinv, int64_t rows,
                      int cols, float eps, float gamma_offset) {
  static_assert(G > kRowThreads, "the CTA is the row group");
  constexpr int N = vec16<T>::N;
  __shared__ float scratch[2 * (G / 32)];
  const int lane = threadIdx.x;
  const int nvec = cols / N;
  const int64_t stride = gridDim.x;
  int64_t row = blockIdx.x;

  vec16<T> next[VPT];
  if (row < rows) {
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      if (v < nvec) next[i].raw = ld_stream16(x + row * x_stride + (int64_t)v * N);
    }
  }
  int buf = 0;  // consecutive rows reduce through alternating scratch halves
  for (; row < rows; row += stride) {
    vec16<T> xv[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) xv[i] = next[i];
    if (row + stride < rows) {
      const T *ahead = x + (row + stride) * x_stride;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int v = lane + i * G;
        if (v < nvec) next[i].raw = ld_stream16(ahead + (int64_t)v * N);
      }
    }
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (lane + i * G < nvec) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float f = io<T>::load(xv[i].e[j]);
          acc = fmaf(f, f, acc);
        }
      }
    }
    acc = group_reduce<G, SumOp>(acc, scratch, buf);
    buf ^= 1;
    const float inv = 1.0f / sqrtf(acc / (float)cols + eps);
    if (lane == 0 && rinv != nullptr) rinv[row] = io<T>::store(inv);
    T *yrow = y + row * y_stride;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int v = lane + i * G;
      if (v < nvec) {
        vec16<T> wv, out;
        wv.raw = *reinterpret_cast<const uint4 *>(w + (int64_t)v * N);
#pragma unroll
        for (int j = 0; j < N; ++j)
          out.e[j] =
              io<T>::store(io<T>::load(xv[i].e[j]) * inv * (io<T>::load(wv.e[j]) + gamma_offset));
        st_stream16(yrow + (int64_t)v * N, out.raw);
      }
    }
  }
}

// Any width / alignment: one CTA per row, scalar loads, the row is re-read
// from L2 for the scale pass.  Used for ragged widths such as 67.
template <typename T>
__global__ void __launch_bounds__(kRowThreads)
rmsnorm_loop_kernel(const T *__restrict__ x, int64_t x_stride,
                    const T *__restrict__ w, int64_t w_stride,
                    T *__restrict__ y, int64_t y_stride, T *__restrict__ rinv,
                    int64_t rinv_stride, int cols, float eps, float gamma_offset) {
  __shared__ float scratch[2 * (kRowThreads / 32)];
  const int64_t row = blockIdx.x;
  const T *xrow = x + row * x_stride;
  float acc = 0.f;
  for (int c = threadIdx.x; c < cols; c += kRowThreads) {
    const float f = io<T>::load(xrow[c]);
    acc = fmaf(f, f, acc);
  }
  acc = group_reduce<kRowThreads, SumOp>(acc, scratch, 0);
  const float inv = 1.0f / sqrtf(acc / (float)cols + eps);
  if (threadIdx.x == 0 && rinv != nullptr) rinv[row * rinv_stride] = io<T>::store(inv);
  T *yrow = y + row * y_stride;
  for (int c = threadIdx.x; c < cols; c += kRowThreads)
    yrow[c] = io<T>::store(io<T>::load(xrow[c]) * inv * (io<T>::load(w[c * w_stride]) + gamma_offset));
}

template <typename T, int G, int VPT>
static void launch_rows(const b200_tensor *x, const b200_tensor *w, b200_tensor *y,
                        b200_tensor *rinv, float eps, float gamma_offset, cudaStream_t stream) {
  constexpr int kThreads = G > kRowThreads ? G : kRowThreads;
  constexpr int kRowsPerCta = kThreads / G;
  const int64_t rows = x->shape[0];
  const unsigned grid = (unsigned)((rows + kRowsPerCta - 1) / kRowsPerCta);
  // Only where it measured faster: 32-bit rows of 1024 threads' width (fp32 [2048,16384]
  // 4.9 -> 6.1 TB/s).  16-bit rows of the same widths and 512-thread rows are faster with one
  // row per CTA -- several CTAs of that kernel share an SM and overlap each other's phases
  // (bf16 [4096,16384] 5.5 against 4.4 TB/s, [2048,32768] 4.7 against 3.7, fp32 [4096,8192]
  // 6.5 against 5.8).
  if constexpr (G > 512 && sizeof(T) == 4) {
    // (B200OPS_RMSNORM_STREAM=0 keeps one row per CTA)
    static const int choice =
        getenv("B200OPS_RMSNORM_STREAM") ? atoi(getenv("B200OPS_RMSNORM_STREAM")) : 1;
    const unsigned resident = (unsigned)(sm_count() * (G > 512 ? 1 : 2));
    if (choice != 0 && grid > resident) {
      rmsnorm_stream_kernel<T, G, VPT><<<resident, G, 0, stream>>>(
          (const T *)x->data, x->stride[0], (const T *)w->data, (T *)y->data, y->stride[0],
          rinv ? (T *)rinv->data : nullptr, rows, (int)x->shape[1], eps, gamma_offset);
      return;
    }
  }
  rmsnorm_rows_kernel<T, G, VPT><<<grid, kThreads, 0, stream>>>(
      (const T *)x->data, x->stride[0], (const T *)w->data, (T *)y->data,
      y->stride[0], rinv ? (T *)rinv->data : nullptr, rows, (int)x->shape[1], eps, gamma_offset);
}

template <typename T>
static int dispatch(const b200_tensor *x, const b200_tensor *w, b200_tensor *y,
                    b200_tensor *rinv, float eps, float gamma_offset, cudaStream_t stream) {
  constexpr int N = vec16<T>::N;
  constexpr int VPT = 4;
  const int64_t rows = x->shape[0], cols = x->shape[1];
  const bool aligned =
      cols % N == 0 && (x->stride[0] * sizeof(T)) % 16 == 0 &&
      (y->stride[0] * sizeof(T)) % 16 == 0 && ((uintptr_t)x->data % 16) == 0 &&
      ((uintptr_t)y->data % 16) == 0 && ((uintptr_t)w->data % 16) == 0 &&
      w->stride[0] == 1 && (rinv == nullptr || rinv->stride[0] == 1);
  const int g = aligned ? pick_group(cols / N, VPT) : 0;
  switch (g) {
    case 8: launch_rows<T, 8, VPT>(x, w, y, rinv, eps, gamma_offset, stream); break;
    case 16: launch_rows<T, 16, VPT>(x, w, y, rinv, eps, gamma_offset, stream); break;
    case 32: launch_rows<T, 32, VPT>(x, w, y, rinv, eps, gamma_offset, stream); break;
    case 64: launch_rows<T, 64, VPT>(x, w, y, rinv, eps, gamma_offset, stream); break;
    case 128: launch_rows<T, 128, VPT>(x, w, y, rinv, eps, gamma_offset, stream); break;
    case 256: launch_rows<T, 256, VPT>(x, w, y, rinv, eps, gamma_offset, stream); break;
    case 512: launch_rows<T, 512, VPT>(x, w, y, rinv, eps, gamma_offset, stream); break;
    case 1024: launch_rows<T, 1024, VPT>(x, w, y, rinv, eps, gamma_offset, stream); break;
    default: {
      // wider than one CTA holds in registers: a cluster per row when the layout allows it
      bool taken = false;
      if (aligned) {
        const int st = rmsnorm_cluster_rows<T>(x, w, y, rinv, eps, gamma_offset, stream, &taken);
        if (st != B200_OK) return st;
      }
      if (taken) break;
      rmsnorm_loop_kernel<T><<<(unsigned)rows, kRowThreads, 0, stream>>>(
          (const T *)x->data, x->stride[0], (const T *)w->data, w->stride[0],
          (T *)y->data, y->stride[0], rinv ? (T *)rinv->data : nullptr,
          rinv ? rinv->stride[0] : 0, (int)cols, eps, gamma_offset);
    }
  }
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

}  // namespace b200

extern "C" int b200_rmsnorm_fwd_ex(const b200_tensor *x, const b200_tensor *w,
                                   b200_tensor *y, b200_tensor *rinv, float eps,
                                   float gamma_offset, void *stream) {
  using namespace b200;
  int st;
  if ((st = check_tensor(x, "x", 2)) || (st = check_tensor(w, "w", 1)) ||
      (st = check_tensor(y, "y", 2)))
    return st;
  if (rinv != nullptr && (st = check_tensor(rinv, "rinv", 1))) return st;
  B200_REQUIRE(is_float_io(x->dtype), "x: dtype %u is not f16/bf16/f32", x->dtype);
  B200_REQUIRE(w->dtype == x->dtype && y->dtype == x->dtype,
               "x/w/y dtypes differ (%u/%u/%u)", x->dtype, w->dtype, y->dtype);
  B200_REQUIRE(rinv == nullptr || rinv->dtype == x->dtype, "rinv dtype differs from x");
  const int64_t rows = x->shape[0], cols = x->shape[1];
  B200_REQUIRE(y->shape[0] == rows && y->shape[1] == cols, "y shape differs from x");
  B200_REQUIRE(w->shape[0] == cols, "w has %lld elements, row width is %lld",
               (long long)w->shape[0], (long long)cols);
  B200_REQUIRE(rinv == nullptr || rinv->shape[0] == rows, "rinv length differs from rows");
  B200_REQUIRE(x->stride[1] == 1 && y->stride[1] == 1, "x/y need unit column stride");
  B200_REQUIRE(x->stride[0] >= cols && y->stride[0] >= cols, "row stride below row width");
  B200_REQUIRE(cols > 0 && cols < (1 << 30), "row width %lld out of range", (long long)cols);
  B200_REQUIRE(rows < (1LL << 31), "too many rows");
  B200_REQUIRE(!(eps < 0.f) && eps == eps, "eps must be a non-negative number");
  B200_REQUIRE(gamma_offset == gamma_offset, "gamma_offset must be a number");
  if (rows == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (x->dtype) {
    case B200_DTYPE_FLOAT32: return dispatch<float>(x, w, y, rinv, eps, gamma_offset, s);
    case B200_DTYPE_FLOAT16: return dispatch<__half>(x, w, y, rinv, eps, gamma_offset, s);
    default: return dispatch<__nv_bfloat16>(x, w, y, rinv, eps, gamma_offset, s);
  }
}

extern "C" int b200_rmsnorm_fwd(const b200_tensor *x, const b200_tensor *w,
                                b200_tensor *y, b200_tensor *rinv, float eps,
                                void *stream) {
  return b200_rmsnorm_fwd_ex(x, w, y, rinv, eps, 0.0f, stream);
}
