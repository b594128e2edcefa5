// All-reduce of 16-bit partial results through NVSwitch (NVLS): the merge step of the
// tensor-parallel MLP.  Every rank holds its partial [rows, cols] in a buffer that is bound
// to one multicast address range; a load through that range (multimem.ld_reduce) returns the
// sum of all ranks' copies, added in the switch in fp32, and a store through it (multimem.st)
// writes all ranks' copies at once.  Rank r reduces rows [r*rows/world, (r+1)*rows/world) and
// publishes them, so each rank sends 1/world of the buffer up and receives the rest, and no
// partial ever crosses a link twice.  The reference's counterpart is the merge of per-worker
// partial slots behind a stage barrier (a100c/plan/stages.py:278-316); it has no multi-device
// form.  The caller separates the producer of the partials, this kernel and the consumer of
// the result with cross-rank barriers.
#include "common.cuh"

namespace b200 {
namespace {

template <bool BF16>
__device__ __forceinline__ uint4 multimem_ld_reduce(const void *mc) {
  uint4 v;
  if constexpr (BF16) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  } else {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  }
  return v;
}

__device__ __forceinline__ void multimem_st(void *mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               :: "l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// vecs 16-byte vectors starting at mc: four reduced loads in flight per thread, then the
// four stores.
template <bool BF16>
__global__ void __launch_bounds__(512)
multimem_allreduce_kernel(uint4 *mc, int64_t vecs) {
  constexpr int U = 4;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < vecs; i += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < vecs) v[u] = multimem_ld_reduce<BF16>(mc + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < vecs) multimem_st(mc + i + u * stride, v[u]);
  }
}

}  // namespace
}  // namespace b200

extern "C" int b200_multimem_allreduce(void *multicast_base, uint32_t dtype, int64_t offset,
                                       int64_t count, int rank, int world, int ctas,
                                       void *stream) {
  using namespace b200;
  if (multicast_base == nullptr) return fail(B200_USAGE, "null multicast pointer");
  B200_REQUIRE(dtype == B200_DTYPE_BFLOAT16 || dtype == B200_DTYPE_FLOAT16,
               "partials are f16 or bf16");
  B200_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world,
               "rank %d / world %d out of range", rank, world);
  B200_REQUIRE(offset >= 0 && count >= 0 && offset % 8 == 0 && count % (8 * world) == 0,
               "offset and count / world must be multiples of 8 elements (16 bytes)");
  B200_REQUIRE((uintptr_t)multicast_base % 16 == 0, "multicast pointer is not 16-byte aligned");
  if (count == 0) return B200_OK;
  const int64_t share = count / world;  // elements this rank reduces and publishes
  const int64_t vecs = share / 8;
  uint4 *first = reinterpret_cast<uint4 *>(
      static_cast<uint8_t *>(multicast_base) + (offset + (int64_t)rank * share) * 2);
  int64_t blocks = (vecs + 512 * 4 - 1) / (512 * 4);
  const int64_t cap = ctas > 0 ? ctas : (int64_t)sm_count() * 2;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == B200_DTYPE_BFLOAT16)
    multimem_allreduce_kernel<true><<<(unsigned)blocks, 512, 0, s>>>(first, vecs);
  else
    multimem_allreduce_kernel<false><<<(unsigned)blocks, 512, 0, s>>>(first, vecs);
  B200_CUDA_OK(cudaGetLastError());
  return B200_OK;
}
