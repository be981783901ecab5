// Status strings, version, mapped pinned allocation.
#include "jf_common.cuh"

namespace jf {
thread_local int32_t g_last_cuda_error = 0;

int num_sms() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return 148; }
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n > 0) return n;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    return 148;
  }
  cached[dev].store(n, std::memory_order_relaxed);
  return n;
}
}  // namespace jf

extern "C" const char* jf_status_string(jf_status_t st) {
  switch (st) {
    case JF_OK: return "ok";
    case JF_ERR_ARG: return "invalid argument (null pointer, bad shape or misaligned pointer)";
    case JF_ERR_UNSUPPORTED: return "request outside the supported envelope";
    case JF_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case JF_ERR_STATIC_LIMIT: return "request needs more scratch than the library's built-in static buffer holds";
    case JF_ERR_CUDA: return "CUDA call failed (see jf_last_cuda_error)";
    case JF_ERR_TIMEOUT: return "a bounded wait ran out";
    case JF_ERR_STATE: return "object used in the wrong state";
    default: return "unknown status";
  }
}

extern "C" int32_t jf_version(void) { return 100; }

extern "C" int32_t jf_last_cuda_error(void) { return jf::g_last_cuda_error; }

// Pinned host memory that the GPU can address directly, so a small result written by
// host threads is visible to a kernel without an explicit copy
// (alloc_mapped_pinned_pair, jetfire_vllm/csrc/cpu_topk_attn.cpp:958-1040).
extern "C" jf_status_t jf_alloc_mapped(uint64_t bytes, void** host_ptr, void** device_ptr) {
  if (!host_ptr || !device_ptr || bytes == 0) return JF_ERR_ARG;
  void* h = nullptr;
  JF_CUDA_TRY(cudaHostAlloc(&h, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
  void* d = nullptr;
  cudaError_t e = cudaHostGetDevicePointer(&d, h, 0);
  if (e != cudaSuccess) { cudaFreeHost(h); return jf::cuda_fail(e); }
  *host_ptr = h;
  *device_ptr = d;
  return JF_OK;
}

extern "C" jf_status_t jf_free_mapped(void* host_ptr) {
  if (!host_ptr) return JF_ERR_ARG;
  JF_CUDA_TRY(cudaFreeHost(host_ptr));
  return JF_OK;
}
