// Status strings, version, mapped pinned allocation.
#include <sys/mman.h>

#include <cstdlib>
#include <mutex>
#include <unordered_set>

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

// Asks the kernel to back [ptr, ptr + bytes) with 2 MB pages where it can (transparent huge pages
// in "madvise" mode serve only ranges that asked).  The host correction gathers 256-byte rows at
// random from mirrors of many gigabytes: with 4 KB pages nearly every row costs a page walk.
// Best before the memory is first touched.  JF_ERR_UNSUPPORTED if the system refuses.
extern "C" jf_status_t jf_advise_huge_pages(void* ptr, uint64_t bytes) {
  if (!ptr || bytes == 0) return JF_ERR_ARG;
  constexpr uintptr_t kHuge = 2u << 20;
  const uintptr_t lo = (reinterpret_cast<uintptr_t>(ptr) + kHuge - 1) & ~(kHuge - 1);
  const uintptr_t hi = (reinterpret_cast<uintptr_t>(ptr) + bytes) & ~(kHuge - 1);
  if (hi <= lo) return JF_OK;   // no whole huge page inside
#ifdef MADV_HUGEPAGE
  return madvise(reinterpret_cast<void*>(lo), hi - lo, MADV_HUGEPAGE) == 0 ? JF_OK : JF_ERR_UNSUPPORTED;
#else
  return JF_ERR_UNSUPPORTED;
#endif
}

namespace {
// allocations of jf_alloc_mapped that were made with the C allocator and registered (see below)
std::mutex g_reg_mu;
std::unordered_set<void*> g_registered;
constexpr uint64_t kHugeThreshold = 8ull << 20;
}  // namespace

// Pinned host memory that the GPU can address directly, so that what one side writes the other
// reads without an explicit copy (alloc_mapped_pinned_pair, jetfire_vllm/csrc/cpu_topk_attn.cpp:958-1040).
// Large blocks -- the host mirrors -- are allocated on a 2 MB boundary, advised to use huge pages
// (the host correction gathers rows from them at random), bound to a memory node if one is asked
// for, and then registered with the driver; small ones without a node, or a system that refuses
// any of these steps, get the driver's own allocation.
extern "C" jf_status_t jf_alloc_mapped_on_node(uint64_t bytes, int32_t node, void** host_ptr, void** device_ptr) {
  if (!host_ptr || !device_ptr || bytes == 0 || node < -1) return JF_ERR_ARG;
  void* h = nullptr;
  void* d = nullptr;
  if (bytes >= kHugeThreshold || node >= 0) {
    const uint64_t unit = bytes >= kHugeThreshold ? (2ull << 20) : 4096ull;
    const uint64_t rounded = (bytes + unit - 1) & ~(unit - 1);
    if (posix_memalign(&h, unit, rounded) == 0 && h) {
      if (bytes >= kHugeThreshold) jf_advise_huge_pages(h, rounded);
      if (node >= 0) jf_bind_memory_to_node(h, rounded, node);   // a refusal leaves first-touch placement
      if (cudaHostRegister(h, rounded, cudaHostRegisterMapped | cudaHostRegisterPortable) == cudaSuccess) {
        if (cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess) {
          std::lock_guard<std::mutex> lock(g_reg_mu);
          g_registered.insert(h);
          *host_ptr = h;
          *device_ptr = d;
          return JF_OK;
        }
        cudaHostUnregister(h);
      }
      cudaGetLastError();   // the driver's own allocation is tried next
      free(h);
      h = nullptr;
    }
  }
  JF_CUDA_TRY(cudaHostAlloc(&h, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
  cudaError_t e = cudaHostGetDevicePointer(&d, h, 0);
  if (e != cudaSuccess) { cudaFreeHost(h); return jf::cuda_fail(e); }
  *host_ptr = h;
  *device_ptr = d;
  return JF_OK;
}

extern "C" jf_status_t jf_alloc_mapped(uint64_t bytes, void** host_ptr, void** device_ptr) {
  return jf_alloc_mapped_on_node(bytes, -1, host_ptr, device_ptr);
}

extern "C" jf_status_t jf_free_mapped(void* host_ptr) {
  if (!host_ptr) return JF_ERR_ARG;
  bool registered = false;
  {
    std::lock_guard<std::mutex> lock(g_reg_mu);
    registered = g_registered.erase(host_ptr) != 0;
  }
  if (registered) {
    JF_CUDA_TRY(cudaHostUnregister(host_ptr));
    free(host_ptr);
    return JF_OK;
  }
  JF_CUDA_TRY(cudaFreeHost(host_ptr));
  return JF_OK;
}
