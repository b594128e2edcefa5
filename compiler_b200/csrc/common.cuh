// Shared host/device helpers for the sm_100a operator library.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/b200ops.h"

namespace b200 {

// ---- host-side error reporting ------------------------------------------
// Detail text of the last non-OK status on this host thread.
char *last_error_buffer();  // 512 bytes, thread-local (api.cu)

inline int fail(int status, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return status;
}

#define B200_CUDA_OK(expr)                                                    \
  do {                                                                        \
    cudaError_t err__ = (expr);                                               \
    if (err__ != cudaSuccess)                                                 \
      return ::b200::fail(B200_RESOURCE, "%s: %s", #expr,                     \
                          cudaGetErrorString(err__));                         \
  } while (0)

#define B200_REQUIRE(cond, ...)                                               \
  do {                                                                        \
    if (!(cond)) return ::b200::fail(B200_REJECTED, __VA_ARGS__);             \
  } while (0)

inline size_t dtype_size(uint32_t dtype) {
  switch (dtype) {
    case B200_DTYPE_BOOL: case B200_DTYPE_INT8: case B200_DTYPE_UINT8: return 1;
    case B200_DTYPE_INT16: case B200_DTYPE_UINT16:
    case B200_DTYPE_FLOAT16: case B200_DTYPE_BFLOAT16: return 2;
    case B200_DTYPE_INT32: case B200_DTYPE_UINT32: case B200_DTYPE_FLOAT32: return 4;
    case B200_DTYPE_INT64: case B200_DTYPE_UINT64: case B200_DTYPE_FLOAT64: return 8;
    default: return 0;
  }
}

inline bool is_float_io(uint32_t dtype) {
  return dtype == B200_DTYPE_FLOAT16 || dtype == B200_DTYPE_BFLOAT16 ||
         dtype == B200_DTYPE_FLOAT32;
}

// Validates the generic part of a tensor descriptor.
inline int check_tensor(const b200_tensor *t, const char *name, uint32_t ndim) {
  if (t == nullptr) return fail(B200_USAGE, "%s: null descriptor", name);
  if (t->ndim != ndim)
    return fail(B200_REJECTED, "%s: ndim %u, expected %u", name, t->ndim, ndim);
  if (dtype_size(t->dtype) == 0)
    return fail(B200_REJECTED, "%s: unknown dtype code %u", name, t->dtype);
  int64_t count = 1;
  for (uint32_t i = 0; i < ndim; ++i) {
    if (t->shape[i] < 0)
      return fail(B200_REJECTED, "%s: negative extent in dim %u", name, i);
    count *= t->shape[i];
  }
  if (count > 0 && t->data == nullptr)
    return fail(B200_REJECTED, "%s: null data pointer", name);
  return B200_OK;
}

// Per-device status word written by kernels whose bounded waits expired.
unsigned int *device_status_word();  // device pointer for the current device

// Frees the decode-attention scratch kept for (current device, stream), if any (attn_decode.cu).
void release_stream_scratch(cudaStream_t stream);
// Frees the GEMM's split-wave scratch kept for (current device, stream), if any (gemm_sm100.cu).
void release_gemm_scratch(cudaStream_t stream);

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) !=
            cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---- device-side element conversion ---------------------------------------
template <typename T> struct io;
template <> struct io<float> {
  static __device__ __forceinline__ float load(float v) { return v; }
  static __device__ __forceinline__ float store(float v) { return v; }
};
template <> struct io<__half> {
  static __device__ __forceinline__ float load(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half store(float v) { return __float2half_rn(v); }
};
template <> struct io<__nv_bfloat16> {
  static __device__ __forceinline__ float load(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 store(float v) { return __float2bfloat16_rn(v); }
};

// 16-byte vector of T
template <typename T> struct vec16 {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 raw; T e[N]; };
};

__device__ __forceinline__ uint4 ld_stream16(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(void *p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
               :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ---- two fp32 lanes per instruction (sm_100 fma / add / mul .f32x2) ---------------------------
// Same arithmetic and rounding as the scalar forms, half the issue slots.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)),
        "l"(*reinterpret_cast<unsigned long long *>(&c)));
  return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)));
  return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long *>(&a)),
        "l"(*reinterpret_cast<unsigned long long *>(&b)));
  return *reinterpret_cast<float2 *>(&d);
}
__device__ __forceinline__ float2 splat(float v) { return make_float2(v, v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace b200
