// Self-test of the bounded device-side wait that every TMA / tcgen05 kernel of this library
// uses (sm100.cuh: mbar_wait).  One CTA waits on a barrier that nothing ever completes; the
// wait must give up after its time limit, record B200_TIMEOUT with its site in the device
// status word, release the other waiter of the CTA through the shared abort flag, and the
// kernel must return normally so that the context stays usable.
#include "common.cuh"
#include "sm100.cuh"

namespace b200 {
namespace {

constexpr uint32_t kSelftestSite = 31;

__global__ void __launch_bounds__(64) wait_selftest_kernel(unsigned int *status, unsigned int *result) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  using namespace sm100;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);  // one arrival expected; none will come
    mbar_init_fence();
    abort_flag = 0u;
  }
  __syncthreads();
  const WaitCtx ctx{&abort_flag, status};
  bool completed = true;
  // two waiters in different warps: the first to expire releases the other
  if ((threadIdx.x & 31) == 0) completed = mbar_wait(smem_u32(&bar), 0, ctx, kSelftestSite);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) atomicOr(result, completed ? 2u : 1u);  // 1 = gave up, as it must
}

}  // namespace
}  // namespace b200

extern "C" int b200_wait_selftest(unsigned int *gave_up, void *stream) {
  using namespace b200;
  if (gave_up == nullptr) return fail(B200_USAGE, "null out pointer");
  unsigned int *status = device_status_word();
  if (status == nullptr) return fail(B200_RESOURCE, "no status word on this device");
  unsigned int *result = nullptr;
  B200_CUDA_OK(cudaMalloc(&result, sizeof *result));
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t err = cudaMemsetAsync(result, 0, sizeof *result, s);
  if (err == cudaSuccess) {
    wait_selftest_kernel<<<1, 64, 0, s>>>(status, result);
    err = cudaGetLastError();
  }
  if (err == cudaSuccess) err = cudaStreamSynchronize(s);
  unsigned int host = 0;
  if (err == cudaSuccess) err = cudaMemcpy(&host, result, sizeof host, cudaMemcpyDeviceToHost);
  cudaFree(result);
  B200_CUDA_OK(err);
  *gave_up = host == 1u ? 1u : 0u;
  return B200_OK;
}
