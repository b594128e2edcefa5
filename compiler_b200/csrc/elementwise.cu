// Elementwise operators and comparison helpers for sm_100a.
#include "common.cuh"

namespace b200 {

// siblings.cu: the flat 16-byte-vector form, four vectors of each operand in flight per thread
void swiglu_flat(uint32_t dtype, const void *x, const void *y, void *out, int64_t n,
                 cudaStream_t s);

// out = x * sigmoid(x) * y in fp32, one rounding at the store
// (swiglu_fwd_kernel, ops/suite/perf/swiglu_fwd.py:27-36).
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_vec_kernel(const T *__restrict__ x, int64_t xs, const T *__restrict__ y,
                  int64_t ys, T *__restrict__ out, int64_t os, int64_t rows,
                  int vec_per_row) {
  constexpr int N = vec16<T>::N;
  const int64_t total = rows * vec_per_row;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int64_t c = (i - r * vec_per_row) * N;
    vec16<T> a, b, o;
    a.raw = ld_stream16(x + r * xs + c);
    b.raw = ld_stream16(y + r * ys + c);
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const float xf = io<T>::load(a.e[j]);
      o.e[j] = io<T>::store(xf / (1.0f + __expf(-xf)) * io<T>::load(b.e[j]));
    }
    st_stream16(out + r * os + c, o.raw);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_scalar_kernel(const T *__restrict__ x, int64_t xs, const T *__restrict__ y,
                     int64_t ys, T *__restrict__ out, int64_t os, int64_t rows,
                     int64_t cols) {
  const int64_t total = rows * cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / cols, c = i - r * cols;
    const float xf = io<T>::load(x[r * xs + c]);
    out[r * os + c] = io<T>::store(xf / (1.0f + expf(-xf)) * io<T>::load(y[r * ys + c]));
  }
}

template <typename T>
static int swiglu_dispatch(const b200_tensor *x, const b200_tensor *y, b200_tensor *out,
                           cudaStream_t stream) {
  constexpr int N = vec16<T>::N;
  const int64_t rows = x->shape[0], cols = x->shape[1];
  const bool aligned = cols % N == 0 && (x->stride[0] * sizeof(T)) % 16 == 0 &&
                       (y->stride[0] * sizeof(T)) % 16 == 0 &&
                       (out->stride[0] * sizeof(T)) % 16 == 0 &&
                       (uintptr_t)x->data % 16 == 0 && (uintptr_t)y->data % 16 == 0 &&
                       (uintptr_t)out->data % 16 == 0;
  if (aligned && (rows == 1 || (x->stride[0] == cols && y->stride[0] == cols &&
                                out->stride[0] == cols))) {
    swiglu_flat(x->dtype, x->data, y->data, out->data, rows * cols, stream);
    B200_CUDA_OK(cudaGetLastError());
    return B200_OK;
  }
  const int64_t items = aligned ? rows * (cols / N) : rows * cols;
  int64_t blocks = (items + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (aligned)
    swiglu_vec_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(
        (const T *)x->data, x->stride[0], (const T *)y->data, y->stride[0],
        (T *)out->data, out->stride[0], rows, (int)(cols / N));
  else
    swiglu_scalar_kernel<T><<<(unsigned)blocks, 256, 0, stream>>>(
        (const T *)x->data, x->stride[0], (const T *)y->data, y->stride[0],
        (T *)out->data, out->stride[0], rows, cols);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}

// np.isclose(a, b, rtol, atol, equal_nan) in fp32 plus max |a-b| in fp64 over
// the elements that are not exactly equal
// (ops/harness/opslib/devices/_cuda_compare.py:24-46).
__global__ void __launch_bounds__(256)
allclose_f32_kernel(const float *__restrict__ a, const float *__restrict__ b,
                    int64_t n, float rtol, float atol, int equal_nan,
                    unsigned long long *bad, unsigned long long *maxerr_bits) {
  unsigned long long local_bad = 0;
  double local_err = 0.0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float av = a[i], bv = b[i];
    const float b_abs = fabsf(bv);
    const bool finite = b_abs < INFINITY;
    bool close = ((fabsf(av - bv) <= (atol + rtol * b_abs)) && finite) || (av == bv);
    bool equal = av == bv;
    if (equal_nan) {
      const bool both_nan = (av != av) && (bv != bv);
      close = close || both_nan;
      equal = equal || both_nan;
    }
    if (!close) ++local_bad;
    if (!equal) {
      const double d = fabs((double)av - (double)bv);
      // NaN deltas order above every finite value as bit patterns, like the
      // int64 atomic_max of the reference does
      if (d != d || d > local_err) local_err = d;
    }
  }
  if (local_bad) atomicAdd(bad, local_bad);
  if (local_err != 0.0 || local_err != local_err)
    atomicMax(maxerr_bits, (unsigned long long)__double_as_longlong(local_err));
}

// Second half of the tensor-parallel all-reduce: this rank owns `rows` rows of the result.
// staging holds the `world` partial slices of those rows ([world, rows, cols], written
// there by every rank's GEMM epilogue); each thread sums one 16-byte column group over
// the slices in fp32, rounds once and stores the result into the owned rows of EVERY
// rank's output (plain peer stores over NVLink for the other ranks).
template <typename T, typename OutT>
__global__ void __launch_bounds__(256)
reduce_slices_broadcast_kernel(const T *__restrict__ staging, int world, int64_t rows, int cols,
                               int64_t dst_row0, OutT *y0, OutT *y1, OutT *y2, OutT *y3, OutT *y4,
                               OutT *y5, OutT *y6, OutT *y7) {
  static_assert(sizeof(T) == sizeof(OutT), "staged and result elements have one size");
  constexpr int N = vec16<T>::N;
  OutT *const y_rank[8] = {y0, y1, y2, y3, y4, y5, y6, y7};
  const int vec_per_row = cols / N;
  const int64_t total = rows * vec_per_row;
  const int64_t slice = rows * (int64_t)cols;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int64_t c = (i - r * vec_per_row) * N;
    float acc[N];
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = 0.f;
    for (int w = 0; w < world; ++w) {
      vec16<T> v;
      v.raw = ld_stream16(staging + w * slice + r * cols + c);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] += io<T>::load(v.e[j]);
    }
    vec16<OutT> out;
#pragma unroll
    for (int j = 0; j < N; ++j) out.e[j] = io<OutT>::store(acc[j]);
    const int64_t off = (dst_row0 + r) * cols + c;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if (w < world) *reinterpret_cast<uint4 *>(y_rank[w] + off) = out.raw;
  }
}

// ---- allclose without any allocation ----------------------------------------------
// Scratch for b200_allclose_f32_static: one (bad count, max-error bits) pair per block.
// It lives in the library image, so every GPU that loads the library carries these
// 128 KiB until the process exits.
constexpr int kStaticBlockElems = 256 * 64;   // elements one block compares
constexpr int kStaticMaxBlocks = 8192;        // => at most 2^27 elements per call
static __device__ __align__(256) unsigned long long g_allclose_static[2 * kStaticMaxBlocks];

// Stage 1: block b compares its own slice and writes its pair to scratch[2b], [2b+1]
// (every launched block writes, so nothing needs to start at zero here).
__global__ void __launch_bounds__(256)
allclose_partial_kernel(const float *__restrict__ a, const float *__restrict__ b, int64_t n,
                        float rtol, float atol, int equal_nan, unsigned long long *scratch) {
  __shared__ unsigned long long s_bad[8];
  __shared__ unsigned long long s_err[8];
  unsigned long long local_bad = 0, local_err = 0;  // error kept as double bits: they order like the values
  const int64_t base = (int64_t)blockIdx.x * kStaticBlockElems;
  for (int k = 0; k < kStaticBlockElems / 256; ++k) {
    const int64_t i = base + (int64_t)k * 256 + threadIdx.x;
    if (i >= n) break;
    const float av = a[i], bv = b[i];
    const float b_abs = fabsf(bv);
    bool close = ((fabsf(av - bv) <= (atol + rtol * b_abs)) && b_abs < INFINITY) || (av == bv);
    bool equal = av == bv;
    if (equal_nan) {
      const bool both_nan = (av != av) && (bv != bv);
      close = close || both_nan;
      equal = equal || both_nan;
    }
    if (!close) ++local_bad;
    if (!equal) {
      const unsigned long long bits =
          (unsigned long long)__double_as_longlong(fabs((double)av - (double)bv));
      if (bits > local_err) local_err = bits;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    local_bad += __shfl_xor_sync(0xffffffffu, local_bad, o);
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, local_err, o);
    if (other > local_err) local_err = other;
  }
  if ((threadIdx.x & 31) == 0) {
    s_bad[threadIdx.x >> 5] = local_bad;
    s_err[threadIdx.x >> 5] = local_err;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) {
      local_bad += s_bad[w];
      if (s_err[w] > local_err) local_err = s_err[w];
    }
    scratch[2 * blockIdx.x] = local_bad;
    scratch[2 * blockIdx.x + 1] = local_err;
  }
}

// Stage 2: one block folds the per-block pairs into the pair at the END of the scratch
// array (slots 2*blocks, 2*blocks+1 are never a block's own pair; the last pair of the
// array is reserved for the result).
__global__ void __launch_bounds__(256)
allclose_final_kernel(unsigned long long *scratch, int blocks, unsigned long long *result) {
  __shared__ unsigned long long s_bad[8];
  __shared__ unsigned long long s_err[8];
  unsigned long long bad = 0, err = 0;
  for (int b = threadIdx.x; b < blocks; b += 256) {
    bad += scratch[2 * b];
    if (scratch[2 * b + 1] > err) err = scratch[2 * b + 1];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    bad += __shfl_xor_sync(0xffffffffu, bad, o);
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, err, o);
    if (other > err) err = other;
  }
  if ((threadIdx.x & 31) == 0) {
    s_bad[threadIdx.x >> 5] = bad;
    s_err[threadIdx.x >> 5] = err;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) {
      bad += s_bad[w];
      if (s_err[w] > err) err = s_err[w];
    }
    result[0] = bad;
    result[1] = err;
  }
}

// Device address of the scratch array on the current device.  In host code the array's
// name is only a stand-in for the symbol, not a device pointer: the address has to be
// asked for, once per device, with that device current.
static int allclose_static_scratch(unsigned long long **out) {
  static unsigned long long *cached[64] = {nullptr};
  int dev = 0;
  B200_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200_RESOURCE, "device index %d out of range", dev);
  if (cached[dev] == nullptr) {
    unsigned long long *ptr = nullptr;
    B200_CUDA_OK(cudaGetSymbolAddress((void **)&ptr, g_allclose_static));
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return B200_OK;
}

__global__ void __launch_bounds__(256)
bitwise_diff_kernel(const unsigned char *__restrict__ a, const unsigned char *__restrict__ b,
                    size_t n, unsigned int *diff) {
  unsigned int local = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (size_t)gridDim.x * blockDim.x)
    local |= (a[i] != b[i]);
  if (local) atomicOr(diff, 1u);
}

}  // namespace b200

extern "C" int b200_swiglu_fwd(const b200_tensor *x, const b200_tensor *y,
                               b200_tensor *out, void *stream) {
  using namespace b200;
  int st;
  if ((st = check_tensor(x, "x", 2)) || (st = check_tensor(y, "y", 2)) ||
      (st = check_tensor(out, "out", 2)))
    return st;
  B200_REQUIRE(is_float_io(x->dtype), "x: dtype %u is not f16/bf16/f32", x->dtype);
  B200_REQUIRE(y->dtype == x->dtype && out->dtype == x->dtype, "x/y/out dtypes differ");
  const int64_t rows = x->shape[0], cols = x->shape[1];
  B200_REQUIRE(y->shape[0] == rows && y->shape[1] == cols && out->shape[0] == rows &&
               out->shape[1] == cols, "x/y/out shapes differ");
  B200_REQUIRE(x->stride[1] == 1 && y->stride[1] == 1 && out->stride[1] == 1,
               "unit column stride required");
  if (rows == 0 || cols == 0) return B200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  switch (x->dtype) {
    case B200_DTYPE_FLOAT32: return swiglu_dispatch<float>(x, y, out, s);
    case B200_DTYPE_FLOAT16: return swiglu_dispatch<__half>(x, y, out, s);
    default: return swiglu_dispatch<__nv_bfloat16>(x, y, out, s);
  }
}

extern "C" int b200_allclose_f32(const void *actual, const void *expected, int64_t count,
                                 double rtol, double atol, int equal_nan,
                                 int64_t *bad_count, double *max_abs_err, void *stream) {
  using namespace b200;
  if (bad_count == nullptr || max_abs_err == nullptr)
    return fail(B200_USAGE, "null result pointer");
  *bad_count = 0;
  *max_abs_err = 0.0;
  if (count == 0) return B200_OK;
  B200_REQUIRE(count > 0 && actual != nullptr && expected != nullptr, "bad buffers");
  cudaStream_t s = (cudaStream_t)stream;
  unsigned long long *scratch = nullptr;
  B200_CUDA_OK(cudaMalloc(&scratch, 16));
  cudaMemsetAsync(scratch, 0, 16, s);
  int64_t blocks = (count + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  allclose_f32_kernel<<<(unsigned)blocks, 256, 0, s>>>(
      (const float *)actual, (const float *)expected, count, (float)rtol, (float)atol,
      equal_nan, scratch, scratch + 1);
  unsigned long long host[2] = {0, 0};
  cudaError_t err = cudaMemcpyAsync(host, scratch, 16, cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  cudaFree(scratch);
  if (err != cudaSuccess) return fail(B200_SYNC, "allclose: %s", cudaGetErrorString(err));
  *bad_count = (int64_t)host[0];
  double e;
  memcpy(&e, &host[1], sizeof e);
  *max_abs_err = e;
  return B200_OK;
}

extern "C" int b200_bitwise_equal(const void *first, const void *other, size_t bytes,
                                  int *equal, void *stream) {
  using namespace b200;
  if (equal == nullptr) return fail(B200_USAGE, "null result pointer");
  *equal = 1;
  if (bytes == 0) return B200_OK;
  B200_REQUIRE(first != nullptr && other != nullptr, "null buffer");
  cudaStream_t s = (cudaStream_t)stream;
  unsigned int *flag = nullptr;
  B200_CUDA_OK(cudaMalloc(&flag, 4));
  cudaMemsetAsync(flag, 0, 4, s);
  size_t blocks = (bytes + 255) / 256;
  const size_t cap = (size_t)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  bitwise_diff_kernel<<<(unsigned)blocks, 256, 0, s>>>(
      (const unsigned char *)first, (const unsigned char *)other, bytes, flag);
  unsigned int host = 0;
  cudaError_t err = cudaMemcpyAsync(&host, flag, 4, cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  cudaFree(flag);
  if (err != cudaSuccess) return fail(B200_SYNC, "bitwise_equal: %s", cudaGetErrorString(err));
  *equal = host ? 0 : 1;
  return host ? B200_REPEAT_MISMATCH : B200_OK;
}

extern "C" int b200_allclose_f32_static(const void *actual, const void *expected, int64_t count,
                                        double rtol, double atol, int equal_nan,
                                        int64_t *bad_count, double *max_abs_err, void *stream) {
  using namespace b200;
  if (bad_count == nullptr || max_abs_err == nullptr)
    return fail(B200_USAGE, "null result pointer");
  *bad_count = 0;
  *max_abs_err = 0.0;
  if (count == 0) return B200_OK;
  B200_REQUIRE(count > 0 && actual != nullptr && expected != nullptr, "bad buffers");
  // the last pair of the array holds the result, the rest one pair per block
  constexpr int64_t kMaxCount = (int64_t)(kStaticMaxBlocks - 1) * kStaticBlockElems;
  B200_REQUIRE(count <= kMaxCount,
               "count %lld exceeds the %lld elements the built-in scratch array covers; use "
               "b200_allclose_f32 for larger buffers",
               (long long)count, (long long)kMaxCount);
  unsigned long long *scratch = nullptr;
  int st = allclose_static_scratch(&scratch);
  if (st != B200_OK) return st;
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = (int)((count + kStaticBlockElems - 1) / kStaticBlockElems);
  unsigned long long *result = scratch + 2 * (kStaticMaxBlocks - 1);
  allclose_partial_kernel<<<blocks, 256, 0, s>>>((const float *)actual, (const float *)expected,
                                                 count, (float)rtol, (float)atol, equal_nan,
                                                 scratch);
  allclose_final_kernel<<<1, 256, 0, s>>>(scratch, blocks, result);
  B200_CUDA_OK(cudaGetLastError());
  unsigned long long host[2] = {0, 0};
  cudaError_t err = cudaMemcpyAsync(host, result, sizeof host, cudaMemcpyDeviceToHost, s);
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  if (err != cudaSuccess)
    return fail(B200_SYNC, "allclose (static scratch): %s", cudaGetErrorString(err));
  *bad_count = (int64_t)host[0];
  double e;
  memcpy(&e, &host[1], sizeof e);
  *max_abs_err = e;
  return B200_OK;
}

extern "C" int b200_reduce_slices_broadcast(const void *staging, uint32_t dtype,
                                            uint32_t out_dtype, int world, int64_t rows,
                                            int64_t cols, int64_t dst_row0, void *const *y_rank,
                                            void *stream) {
  using namespace b200;
  if (staging == nullptr || y_rank == nullptr) return fail(B200_USAGE, "null argument");
  B200_REQUIRE(world >= 1 && world <= 8, "world %d out of range", world);
  B200_REQUIRE((dtype == B200_DTYPE_BFLOAT16 || dtype == B200_DTYPE_FLOAT16) &&
               (out_dtype == B200_DTYPE_BFLOAT16 || out_dtype == B200_DTYPE_FLOAT16),
               "partials and result are f16 or bf16");
  B200_REQUIRE(rows >= 0 && cols > 0 && cols % 8 == 0 && cols < (1 << 30) && dst_row0 >= 0,
               "rows / cols out of range (cols must be a multiple of 8)");
  B200_REQUIRE((uintptr_t)staging % 16 == 0, "staging is not 16-byte aligned");
  void *y[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  for (int w = 0; w < world; ++w) {
    B200_REQUIRE(y_rank[w] != nullptr && (uintptr_t)y_rank[w] % 16 == 0,
                 "output pointer of rank %d is null or unaligned", w);
    y[w] = y_rank[w];
  }
  if (rows == 0) return B200_OK;
  const int64_t items = rows * (cols / 8);
  int64_t blocks = (items + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = (cudaStream_t)stream;
#define B200_RSB(T, O)                                                                         \
  reduce_slices_broadcast_kernel<T, O><<<(unsigned)blocks, 256, 0, s>>>(                       \
      (const T *)staging, world, rows, (int)cols, dst_row0, (O *)y[0], (O *)y[1], (O *)y[2],   \
      (O *)y[3], (O *)y[4], (O *)y[5], (O *)y[6], (O *)y[7])
  if (dtype == B200_DTYPE_BFLOAT16 && out_dtype == B200_DTYPE_BFLOAT16)
    B200_RSB(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == B200_DTYPE_FLOAT16 && out_dtype == B200_DTYPE_BFLOAT16)
    B200_RSB(__half, __nv_bfloat16);
  else if (dtype == B200_DTYPE_BFLOAT16)
    B200_RSB(__nv_bfloat16, __half);
  else
    B200_RSB(__half, __half);
#undef B200_RSB
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}
