// jf_decode_fused_static: the fused decode step without a caller-provided workspace.
//
// Who this is for: code that drives the GPU but is not in a position to obtain device
// memory for scratch -- a plugin running inside a host that owns every allocation, a
// callback on a latency-critical path where an allocator call (and the implicit
// synchronisation cudaMalloc / cudaFree can bring) is not acceptable, or a process whose
// memory pool was sized in advance and is already spoken for.  Such a caller still hands
// in its inputs and outputs; only the scratch comes from here.
//
// The scratch is a fixed array in device global memory that is part of this library's
// image: every GPU on which the library is loaded carries JF_STATIC_SCRATCH_BYTES of it
// from load until the process exits, whether or not this entry point is ever called.
// Requests that need more are refused with JF_ERR_STATIC_LIMIT; nothing here calls
// cudaMalloc, cudaFree or any other allocating routine.
//
// Sharing: there is one array per device, used by every call.  It keeps whatever the last
// call left in it -- that is harmless, because each call rewrites every partial it later
// reads -- but two calls that overlap on the same
// GPU (different streams, or different host threads) write the same memory and race.
// Serialise them.
//
// First call on a device: the array's device address is looked up once per device
// (cudaGetSymbolAddress, with that device current) and remembered.  Make that first call
// outside of any stream capture.
#include "decode_common.cuh"

namespace {

static __device__ __align__(256) unsigned char g_static_scratch[JF_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {nullptr};
std::atomic<uint64_t> g_scratch_ready{0};

// In host code `g_static_scratch` is only a handle for the symbol, not an address a kernel
// could use; the address valid on the current device has to be asked for.
jf_status_t static_scratch(void** out) {
  int dev = 0;
  JF_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return JF_ERR_UNSUPPORTED;
  const uint64_t bit = 1ull << dev;
  if (!(g_scratch_ready.load(std::memory_order_acquire) & bit)) {
    void* p = nullptr;
    JF_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr) return JF_ERR_CUDA;
    g_scratch_addr[dev] = p;
    g_scratch_ready.fetch_or(bit, std::memory_order_release);
  }
  *out = g_scratch_addr[dev];
  return JF_OK;
}

}  // namespace

// For jf_decode_status: the status record of calls made through this entry point sits at the
// start of the built-in array (the kernels find it where a caller's workspace would hold it).
namespace jf {
jf_status_t static_scratch_address(void** out) { return static_scratch(out); }
}

extern "C" jf_status_t jf_decode_fused_static(const jf_decode_args* a, jf_stream_t stream) {
  if (!a) return JF_ERR_ARG;
  if (a->mode != JF_MODE_K3V2) return JF_ERR_UNSUPPORTED;  // see the header: K3V2 only
  const uint64_t need = jf_decode_workspace_bytes(a->mode, a->B, a->H_q, a->H_kv, a->max_S, a->top_k);
  if (need == 0) return JF_ERR_ARG;
  if (need > JF_STATIC_SCRATCH_BYTES) return JF_ERR_STATIC_LIMIT;
  void* scratch = nullptr;
  jf_status_t st = static_scratch(&scratch);
  if (st != JF_OK) return st;
  jf_decode_args local = *a;          // the caller's block is not modified
  local.workspace = scratch;
  local.workspace_bytes = JF_STATIC_SCRATCH_BYTES;
  return jf_decode_fused(&local, stream);
}
