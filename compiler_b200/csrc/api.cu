// Library-level entry points: status text, device query, memory / stream /
// event plumbing and the per-device status word.
#include "common.cuh"

#include <string.h>

namespace b200 {

char *last_error_buffer() {
  static thread_local char buffer[512] = {0};
  return buffer;
}

// One status word per device; kernels with bounded waits OR their failure
// code into it and the host reads it back after the stream has drained.
__device__ unsigned int g_device_status;

unsigned int *device_status_word() {
  static unsigned int *cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_device_status) != cudaSuccess) return nullptr;
    if (cudaMemset(ptr, 0, sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cached[dev] = (unsigned int *)ptr;
  }
  return cached[dev];
}

}  // namespace b200

using namespace b200;

extern "C" int b200_abi_version(void) { return B200_ABI_VERSION; }

extern "C" const char *b200_status_string(int status) {
  switch (status) {
    case B200_OK: return "ok";
    case B200_USAGE: return "usage: argument outside the contract";
    case B200_REJECTED: return "rejected: descriptor violates a precondition";
    case B200_RESOURCE: return "resource: allocation or CUDA runtime failure";
    case B200_REPEAT_MISMATCH: return "repeat mismatch: repeated launches differ";
    case B200_SYNC: return "sync: stream or device synchronisation failed";
    case B200_TIMEOUT: return "timeout: a bounded device-side wait expired";
    case B200_UNSUPPORTED: return "unsupported: no kernel for this request";
    default: return "unknown status";
  }
}

extern "C" const char *b200_last_error(void) { return last_error_buffer(); }

extern "C" int b200_device_query(int device, b200_device_props *out) {
  if (out == nullptr) return fail(B200_USAGE, "null props pointer");
  int count = 0;
  B200_CUDA_OK(cudaGetDeviceCount(&count));
  if (device < 0 || device >= count)
    return fail(B200_USAGE, "device %d out of range (%d visible)", device, count);
  cudaDeviceProp prop;
  B200_CUDA_OK(cudaGetDeviceProperties(&prop, device));
  memset(out, 0, sizeof *out);
  strncpy(out->name, prop.name, sizeof(out->name) - 1);
  out->cc_major = prop.major;
  out->cc_minor = prop.minor;
  out->sm_count = prop.multiProcessorCount;
  out->l2_bytes = prop.l2CacheSize;
  out->hbm_bytes = (int64_t)prop.totalGlobalMem;
  out->smem_per_block_optin = (int32_t)prop.sharedMemPerBlockOptin;
  int khz = 0;
  cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, device);
  out->clock_khz = khz;
  return B200_OK;
}

extern "C" int b200_set_device(int device) {
  B200_CUDA_OK(cudaSetDevice(device));
  return B200_OK;
}

extern "C" int b200_last_device_status(void *stream) {
  cudaError_t err = cudaStreamSynchronize((cudaStream_t)stream);
  if (err != cudaSuccess) return fail(B200_SYNC, "stream sync: %s", cudaGetErrorString(err));
  unsigned int *word = device_status_word();
  if (word == nullptr) return fail(B200_RESOURCE, "no status word on this device");
  unsigned int host = 0;
  B200_CUDA_OK(cudaMemcpy(&host, word, sizeof host, cudaMemcpyDeviceToHost));
  if (host != 0) {
    B200_CUDA_OK(cudaMemset(word, 0, sizeof host));
    return fail((int)(host & 0xff), "device status word 0x%08x (site %u)", host, host >> 8);
  }
  return B200_OK;
}

extern "C" int b200_malloc(void **out, size_t bytes) {
  if (out == nullptr) return fail(B200_USAGE, "null out pointer");
  *out = nullptr;
  B200_CUDA_OK(cudaMalloc(out, bytes ? bytes : 1));
  return B200_OK;
}
extern "C" int b200_free(void *ptr) {
  if (ptr != nullptr) B200_CUDA_OK(cudaFree(ptr));
  return B200_OK;
}
extern "C" int b200_malloc_host(void **out, size_t bytes) {
  if (out == nullptr) return fail(B200_USAGE, "null out pointer");
  *out = nullptr;
  B200_CUDA_OK(cudaMallocHost(out, bytes ? bytes : 1));
  return B200_OK;
}
extern "C" int b200_free_host(void *ptr) {
  if (ptr != nullptr) B200_CUDA_OK(cudaFreeHost(ptr));
  return B200_OK;
}
extern "C" int b200_memcpy_h2d(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return B200_OK;
  B200_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream));
  return B200_OK;
}
extern "C" int b200_memcpy_d2h(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return B200_OK;
  B200_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  return B200_OK;
}
extern "C" int b200_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream) {
  if (bytes == 0) return B200_OK;
  B200_CUDA_OK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream));
  return B200_OK;
}
extern "C" int b200_memset(void *dst, int value, size_t bytes, void *stream) {
  if (bytes == 0) return B200_OK;
  B200_CUDA_OK(cudaMemsetAsync(dst, value, bytes, (cudaStream_t)stream));
  return B200_OK;
}
extern "C" int b200_stream_create(void **out) {
  if (out == nullptr) return fail(B200_USAGE, "null out pointer");
  cudaStream_t s;
  B200_CUDA_OK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  *out = (void *)s;
  return B200_OK;
}
extern "C" int b200_stream_destroy(void *stream) {
  if (stream != nullptr) {
    b200::release_stream_scratch((cudaStream_t)stream);
    b200::release_gemm_scratch((cudaStream_t)stream);
    B200_CUDA_OK(cudaStreamDestroy((cudaStream_t)stream));
  }
  return B200_OK;
}
extern "C" int b200_stream_sync(void *stream) {
  cudaError_t err = cudaStreamSynchronize((cudaStream_t)stream);
  if (err != cudaSuccess) return fail(B200_SYNC, "stream sync: %s", cudaGetErrorString(err));
  return B200_OK;
}
extern "C" int b200_device_sync(void) {
  cudaError_t err = cudaDeviceSynchronize();
  if (err != cudaSuccess) return fail(B200_SYNC, "device sync: %s", cudaGetErrorString(err));
  return B200_OK;
}
extern "C" int b200_event_create(void **out) {
  if (out == nullptr) return fail(B200_USAGE, "null out pointer");
  cudaEvent_t e;
  B200_CUDA_OK(cudaEventCreate(&e));
  *out = (void *)e;
  return B200_OK;
}
extern "C" int b200_event_destroy(void *event) {
  if (event != nullptr) B200_CUDA_OK(cudaEventDestroy((cudaEvent_t)event));
  return B200_OK;
}
extern "C" int b200_event_record(void *event, void *stream) {
  B200_CUDA_OK(cudaEventRecord((cudaEvent_t)event, (cudaStream_t)stream));
  return B200_OK;
}
extern "C" int b200_event_elapsed_ms(void *start, void *stop, float *ms) {
  if (ms == nullptr) return fail(B200_USAGE, "null out pointer");
  cudaError_t err = cudaEventSynchronize((cudaEvent_t)stop);
  if (err != cudaSuccess) return fail(B200_SYNC, "event sync: %s", cudaGetErrorString(err));
  B200_CUDA_OK(cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return B200_OK;
}

// ---- CUDA graphs: a captured sequence of launches replayed with one call -----------------
extern "C" int b200_stream_wait_event(void *stream, void *event) {
  B200_CUDA_OK(cudaStreamWaitEvent((cudaStream_t)stream, (cudaEvent_t)event, 0));
  return B200_OK;
}
extern "C" int b200_graph_begin_capture(void *stream) {
  if (stream == nullptr) return b200::fail(B200_USAGE, "capture needs a created stream, not the default one");
  B200_CUDA_OK(cudaStreamBeginCapture((cudaStream_t)stream, cudaStreamCaptureModeThreadLocal));
  return B200_OK;
}
extern "C" int b200_graph_end_capture(void *stream, void **graph_exec) {
  if (graph_exec == nullptr) return b200::fail(B200_USAGE, "null out pointer");
  *graph_exec = nullptr;
  cudaGraph_t graph = nullptr;
  B200_CUDA_OK(cudaStreamEndCapture((cudaStream_t)stream, &graph));
  cudaGraphExec_t exec = nullptr;
  const cudaError_t err = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  B200_CUDA_OK(err);
  *graph_exec = (void *)exec;
  return B200_OK;
}
extern "C" int b200_graph_launch(void *graph_exec, void *stream) {
  if (graph_exec == nullptr) return b200::fail(B200_USAGE, "null graph");
  B200_CUDA_OK(cudaGraphLaunch((cudaGraphExec_t)graph_exec, (cudaStream_t)stream));
  return B200_OK;
}
extern "C" int b200_graph_destroy(void *graph_exec) {
  if (graph_exec != nullptr) B200_CUDA_OK(cudaGraphExecDestroy((cudaGraphExec_t)graph_exec));
  return B200_OK;
}
