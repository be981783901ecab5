// Stream-ordered append of new tokens' full-precision rows to a host mirror that the GPU
// cannot address (ordinary pageable host memory).
//
// Replaces the reference's pinned staging + host callback
// (jetfire_vllm/adapter/cache_store.py:616-640, create_shadow_append_submit_ctx /
// stream_submit_shadow_append, jetfire_vllm/csrc/cpu_topk_attn.cpp:1611-1665): three
// device-to-host copies and a callback there; here one kernel writes the rows, the slot list
// and the token count of a chunk into mapped pinned staging (coalesced 256-byte writes over
// the host link, no copy engine involved), and one callback scatters them to the mirror.  The
// stream orders everything: the callback runs after the kernel, the next chunk's kernel after
// the callback, and a correction submitted on the same stream (jf_stream_submit_cpu_topk_attn)
// after the rows it may select have landed.  Mirrors that live in mapped pinned memory need
// none of this: jf_pack_append_kv_mirror stores the rows from the packing kernel itself.
#include <atomic>
#include <cstring>
#include <new>

#include "jf_common.cuh"
#include "decode_common.cuh"

namespace jf {
namespace {

constexpr uint64_t kMirrorCtxTag = 0x4A464D4952524F52ull;  // "JFMIRROR"

struct StageHeader {
  int64_t n_tokens;   // written by the kernel: tokens of the chunk in the staging buffers
  int64_t pad[7];
};

struct MirrorCtx {
  uint64_t tag = kMirrorCtxTag;
  uint16_t* k_shadow = nullptr;
  uint16_t* v_shadow = nullptr;
  int32_t H_kv = 0;
  int64_t num_slots = 0, max_tokens = 0;
  // mapped pinned staging: header, slots[max_tokens], K rows, V rows ([t][h][128] each)
  void* stage_host = nullptr;
  void* stage_dev = nullptr;
  std::atomic<int64_t> rows_written{0}, rows_skipped{0}, chunks{0};
  StageHeader* header(void* base) const { return static_cast<StageHeader*>(base); }
  int64_t* slots(void* base) const { return reinterpret_cast<int64_t*>(static_cast<uint8_t*>(base) + sizeof(StageHeader)); }
  uint16_t* k_rows(void* base) const {
    return reinterpret_cast<uint16_t*>(reinterpret_cast<uint8_t*>(slots(base)) + align_bytes(max_tokens * 8));
  }
  uint16_t* v_rows(void* base) const { return k_rows(base) + max_tokens * H_kv * JF_HEAD_DIM; }
  static int64_t align_bytes(int64_t b) { return (b + 255) / 256 * 256; }
  int64_t stage_bytes() const {
    return static_cast<int64_t>(sizeof(StageHeader)) + align_bytes(max_tokens * 8) +
           2 * max_tokens * H_kv * JF_HEAD_DIM * 2;
  }
};

MirrorCtx* ctx_of(int64_t handle) {
  auto* c = reinterpret_cast<MirrorCtx*>(static_cast<intptr_t>(handle));
  return (c && c->tag == kMirrorCtxTag) ? c : nullptr;
}

// Half a warp per (token, kv-head) row, K and V sides on blockIdx.y: sixteen 16-byte loads,
// sixteen 16-byte stores into the staging rows.
__global__ void __launch_bounds__(256)
stage_rows_kernel(const uint16_t* __restrict__ key, const uint16_t* __restrict__ value, int64_t k_stride_t,
                  int64_t k_stride_h, int64_t v_stride_t, int64_t v_stride_h, const int64_t* __restrict__ slots_in,
                  int64_t T, int H, StageHeader* header, int64_t* slots_out, uint16_t* k_out, uint16_t* v_out) {
  const int sub = threadIdx.x & 15;
  const int64_t row = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 4;
  const bool v_side = blockIdx.y != 0;
  if (row < T * H) {
    const int64_t t = row / H;
    const int h = static_cast<int>(row - t * H);
    const uint16_t* src = v_side ? value + t * v_stride_t + h * v_stride_h : key + t * k_stride_t + h * k_stride_h;
    uint16_t* dst = (v_side ? v_out : k_out) + row * JF_HEAD_DIM;
    reinterpret_cast<uint4*>(dst)[sub] = __ldg(reinterpret_cast<const uint4*>(src) + sub);
    if (!v_side && h == 0 && sub == 0) slots_out[t] = slots_in[t];
  }
  if (!v_side && blockIdx.x == 0 && threadIdx.x == 0) header->n_tokens = T;
}

void CUDART_CB scatter_callback(void* ud) {
  auto* c = static_cast<MirrorCtx*>(ud);
  const int64_t T = c->header(c->stage_host)->n_tokens;
  if (T <= 0 || T > c->max_tokens) return;
  const int64_t* slots = c->slots(c->stage_host);
  const uint16_t* ks = c->k_rows(c->stage_host);
  const uint16_t* vs = c->v_rows(c->stage_host);
  const int64_t head_stride = c->num_slots * JF_HEAD_DIM;
  int64_t written = 0, skipped = 0;
  for (int64_t t = 0; t < T; ++t) {
    const int64_t slot = slots[t];
    if (slot < 0 || slot >= c->num_slots) { ++skipped; continue; }   // padding, as on the device side
    for (int h = 0; h < c->H_kv; ++h) {
      std::memcpy(c->k_shadow + h * head_stride + slot * JF_HEAD_DIM, ks + (t * c->H_kv + h) * JF_HEAD_DIM, JF_HEAD_DIM * 2);
      std::memcpy(c->v_shadow + h * head_stride + slot * JF_HEAD_DIM, vs + (t * c->H_kv + h) * JF_HEAD_DIM, JF_HEAD_DIM * 2);
    }
    ++written;
  }
  c->rows_written.fetch_add(written * c->H_kv, std::memory_order_relaxed);
  c->rows_skipped.fetch_add(skipped * c->H_kv, std::memory_order_relaxed);
  c->chunks.fetch_add(1, std::memory_order_release);
}

// The reference's own form of the staged append (create_shadow_append_submit_ctx /
// stream_submit_shadow_append, jetfire_vllm/csrc/cpu_topk_attn.cpp:1611-1665, 2186-2248): the
// caller owns pinned staging tensors k_append / v_append (T, H_kv, 128) and slots (T,) that its
// own stream-ordered copies fill; the callback scatters them into the mirror.
constexpr uint64_t kShadowCtxTag = 0x4A46534841444F57ull;  // "JFSHADOW"
struct ShadowAppendCtx {
  uint64_t tag = kShadowCtxTag;
  const uint16_t* k_append = nullptr;
  const uint16_t* v_append = nullptr;
  const int64_t* slots = nullptr;
  uint16_t* k_shadow = nullptr;
  uint16_t* v_shadow = nullptr;
  int64_t T = 0, num_slots = 0;
  int32_t H_kv = 0;
  std::atomic<int64_t> calls{0};
};

void CUDART_CB shadow_append_callback(void* ud) {
  auto* c = static_cast<ShadowAppendCtx*>(ud);
  const int64_t head_stride = c->num_slots * JF_HEAD_DIM;
  for (int64_t t = 0; t < c->T; ++t) {
    const int64_t slot = c->slots[t];
    if (slot < 0 || slot >= c->num_slots) continue;
    for (int h = 0; h < c->H_kv; ++h) {
      std::memcpy(c->k_shadow + h * head_stride + slot * JF_HEAD_DIM, c->k_append + (t * c->H_kv + h) * JF_HEAD_DIM, JF_HEAD_DIM * 2);
      std::memcpy(c->v_shadow + h * head_stride + slot * JF_HEAD_DIM, c->v_append + (t * c->H_kv + h) * JF_HEAD_DIM, JF_HEAD_DIM * 2);
    }
  }
  c->calls.fetch_add(1, std::memory_order_release);
}

}  // namespace
}  // namespace jf

extern "C" jf_status_t jf_shadow_append_ctx_create(const void* k_append, const void* v_append, const int64_t* slots,
                                                   int64_t T, int32_t H_kv, void* k_shadow, void* v_shadow,
                                                   int64_t num_slots, int64_t* handle) {
  using namespace jf;
  if (!k_append || !v_append || !slots || !k_shadow || !v_shadow || !handle || T < 0 || H_kv <= 0 || num_slots <= 0)
    return JF_ERR_ARG;
  auto* c = new (std::nothrow) ShadowAppendCtx();
  if (!c) return JF_ERR_STATE;
  c->k_append = static_cast<const uint16_t*>(k_append);
  c->v_append = static_cast<const uint16_t*>(v_append);
  c->slots = slots;
  c->k_shadow = static_cast<uint16_t*>(k_shadow);
  c->v_shadow = static_cast<uint16_t*>(v_shadow);
  c->T = T; c->H_kv = H_kv; c->num_slots = num_slots;
  *handle = static_cast<int64_t>(reinterpret_cast<intptr_t>(c));
  return JF_OK;
}

extern "C" jf_status_t jf_shadow_append_ctx_destroy(int64_t handle) {
  auto* c = reinterpret_cast<jf::ShadowAppendCtx*>(static_cast<intptr_t>(handle));
  if (!c || c->tag != jf::kShadowCtxTag) return JF_ERR_ARG;
  c->tag = 0;
  delete c;
  return JF_OK;
}

extern "C" jf_status_t jf_shadow_append_ctx_calls(int64_t handle, int64_t* calls) {
  auto* c = reinterpret_cast<jf::ShadowAppendCtx*>(static_cast<intptr_t>(handle));
  if (!c || c->tag != jf::kShadowCtxTag || !calls) return JF_ERR_ARG;
  *calls = c->calls.load(std::memory_order_acquire);
  return JF_OK;
}

extern "C" jf_status_t jf_stream_submit_shadow_append(jf_stream_t stream, int64_t handle) {
  using namespace jf;
  auto* c = reinterpret_cast<ShadowAppendCtx*>(static_cast<intptr_t>(handle));
  if (!c || c->tag != kShadowCtxTag) return JF_ERR_ARG;
  JF_CUDA_TRY(cudaLaunchHostFunc(static_cast<cudaStream_t>(stream), shadow_append_callback, c));
  return JF_OK;
}

// A 64-bit store to device-visible memory in stream order (stream_write_value64,
// jetfire_vllm/csrc/cpu_topk_attn.cpp:1293-1312): the reference clears its completion flag this
// way before it queues a correction.  The driver call is looked up at run time.
extern "C" jf_status_t jf_stream_write_value64(jf_stream_t stream, void* device_ptr, int64_t value) {
  using namespace jf;
  if (!device_ptr || (reinterpret_cast<uintptr_t>(device_ptr) & 7)) return JF_ERR_ARG;
  using Fn = int (*)(void*, unsigned long long, unsigned long long, unsigned int);
  static Fn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue64", &sym, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<Fn>(sym);
  }();
  if (!fn) return JF_ERR_UNSUPPORTED;
  const int r = fn(stream, static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(device_ptr)),
                   static_cast<unsigned long long>(value), 0u);
  if (r != 0) { g_last_cuda_error = r; return JF_ERR_CUDA; }
  return JF_OK;
}

namespace jf {
namespace {

// Clears the completion word, then raises the trigger word: both live in mapped pinned host memory.
// Everything queued on the stream before this kernel (the copies of the job's inputs to the host)
// has completed when it runs; the fence orders the two stores as the host sees them.
__global__ void signal_host_kernel(volatile long long* done, volatile long long* trigger) {
  if (threadIdx.x == 0) {
    *done = 0;
    __threadfence_system();
    *trigger = 1;
    __threadfence_system();
  }
}

// Polls a word in mapped pinned host memory until it is non-zero or the budget is used up; a wait
// that ran out is recorded in the status record (and the stream carries on).
__global__ void wait_host_flag_kernel(const volatile long long* flag, unsigned long long budget_ns, int32_t* status) {
  if (threadIdx.x != 0) return;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned long long polls = 0; polls < (1ull << 32); ++polls) {
    if (*flag != 0) {
      __threadfence_system();   // what the host wrote before the flag is read after it
      return;
    }
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - t0 > budget_ns) break;
    __nanosleep(polls < 64 ? 100 : 500);
  }
  if (status) report_status(status, JF_ERR_TIMEOUT);
}

}  // namespace
}  // namespace jf

// Queues a kernel that clears *done_dev and then sets *trigger_dev to 1 (device-visible addresses
// of two words in mapped pinned host memory): the GPU's half of starting a host correction without
// a host function in the stream.  The host's half is jf_submit_ctx_watch.
extern "C" jf_status_t jf_stream_signal_host(jf_stream_t stream, int64_t* done_dev, int64_t* trigger_dev) {
  using namespace jf;
  if (!done_dev || !trigger_dev || ((reinterpret_cast<uintptr_t>(done_dev) | reinterpret_cast<uintptr_t>(trigger_dev)) & 7))
    return JF_ERR_ARG;
  signal_host_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<volatile long long*>(done_dev),
                                                                      reinterpret_cast<volatile long long*>(trigger_dev));
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

// Queues a kernel that holds the stream until *flag_dev (mapped pinned host memory) is non-zero,
// for at most timeout_ms (1..60000); a wait that runs out writes JF_ERR_TIMEOUT to the workspace's
// status record (`status_record`: the start of the decode workspace; may be NULL) and lets the
// stream continue.  One thread polls; nothing else of the GPU is held.
extern "C" jf_status_t jf_stream_wait_host_flag(jf_stream_t stream, const int64_t* flag_dev, int32_t timeout_ms,
                                                void* status_record) {
  using namespace jf;
  if (!flag_dev || (reinterpret_cast<uintptr_t>(flag_dev) & 7) || timeout_ms <= 0 || timeout_ms > 60000) return JF_ERR_ARG;
  wait_host_flag_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const volatile long long*>(flag_dev), static_cast<unsigned long long>(timeout_ms) * 1000000ull,
      static_cast<int32_t*>(status_record));
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

extern "C" jf_status_t jf_mirror_append_ctx_create(void* k_shadow, void* v_shadow, int32_t H_kv, int64_t num_slots,
                                                   int64_t max_tokens, int64_t* handle) {
  using namespace jf;
  if (!k_shadow || !v_shadow || !handle || H_kv <= 0 || num_slots <= 0 || max_tokens <= 0) return JF_ERR_ARG;
  auto* c = new (std::nothrow) MirrorCtx();
  if (!c) return JF_ERR_STATE;
  c->k_shadow = static_cast<uint16_t*>(k_shadow);
  c->v_shadow = static_cast<uint16_t*>(v_shadow);
  c->H_kv = H_kv;
  c->num_slots = num_slots;
  c->max_tokens = max_tokens;
  jf_status_t st = jf_alloc_mapped(static_cast<uint64_t>(c->stage_bytes()), &c->stage_host, &c->stage_dev);
  if (st != JF_OK) { delete c; return st; }
  c->header(c->stage_host)->n_tokens = 0;
  *handle = static_cast<int64_t>(reinterpret_cast<intptr_t>(c));
  return JF_OK;
}

extern "C" jf_status_t jf_mirror_append_ctx_destroy(int64_t handle) {
  using namespace jf;
  MirrorCtx* c = ctx_of(handle);
  if (!c) return JF_ERR_ARG;
  c->tag = 0;
  jf_free_mapped(c->stage_host);
  delete c;
  return JF_OK;
}

extern "C" jf_status_t jf_mirror_append_ctx_stats(int64_t handle, int64_t* rows_written, int64_t* rows_skipped,
                                                  int64_t* chunks) {
  using namespace jf;
  MirrorCtx* c = ctx_of(handle);
  if (!c) return JF_ERR_ARG;
  if (chunks) *chunks = c->chunks.load(std::memory_order_acquire);
  if (rows_written) *rows_written = c->rows_written.load(std::memory_order_relaxed);
  if (rows_skipped) *rows_skipped = c->rows_skipped.load(std::memory_order_relaxed);
  return JF_OK;
}

extern "C" jf_status_t jf_stream_mirror_append(jf_stream_t stream_, int64_t handle, const void* key_tok,
                                               const void* value_tok, int64_t T, int64_t k_stride_t,
                                               int64_t k_stride_h, int64_t v_stride_t, int64_t v_stride_h,
                                               const int64_t* slots) {
  using namespace jf;
  MirrorCtx* c = ctx_of(handle);
  if (!c || !key_tok || !value_tok || !slots || T < 0) return JF_ERR_ARG;
  if (!aligned(key_tok, 16) || !aligned(value_tok, 16) || (k_stride_t % 8) || (k_stride_h % 8) || (v_stride_t % 8) ||
      (v_stride_h % 8))
    return JF_ERR_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  for (int64_t t0 = 0; t0 < T; t0 += c->max_tokens) {
    const int64_t n = (T - t0 < c->max_tokens) ? (T - t0) : c->max_tokens;
    const int64_t rows = n * c->H_kv;
    const unsigned ctas = static_cast<unsigned>((rows * 16 + 255) / 256);
    stage_rows_kernel<<<dim3(ctas, 2), 256, 0, stream>>>(
        static_cast<const uint16_t*>(key_tok) + t0 * k_stride_t, static_cast<const uint16_t*>(value_tok) + t0 * v_stride_t,
        k_stride_t, k_stride_h, v_stride_t, v_stride_h, slots + t0, n, c->H_kv, c->header(c->stage_dev),
        c->slots(c->stage_dev), c->k_rows(c->stage_dev), c->v_rows(c->stage_dev));
    JF_CUDA_TRY(cudaGetLastError());
    JF_CUDA_TRY(cudaLaunchHostFunc(stream, scatter_callback, c));
  }
  return JF_OK;
}

// Make an existing host allocation (for instance a mirror that a tensor library allocated)
// addressable by the GPU, so that jf_pack_append_kv_mirror can store into it.
extern "C" jf_status_t jf_map_host(void* host_ptr, uint64_t bytes, void** device_ptr) {
  using namespace jf;
  if (!host_ptr || !device_ptr || bytes == 0) return JF_ERR_ARG;
  JF_CUDA_TRY(cudaHostRegister(host_ptr, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable));
  void* d = nullptr;
  const cudaError_t e = cudaHostGetDevicePointer(&d, host_ptr, 0);
  if (e != cudaSuccess) { cudaHostUnregister(host_ptr); return cuda_fail(e); }
  *device_ptr = d;
  return JF_OK;
}

extern "C" jf_status_t jf_unmap_host(void* host_ptr) {
  using namespace jf;
  if (!host_ptr) return JF_ERR_ARG;
  JF_CUDA_TRY(cudaHostUnregister(host_ptr));
  return JF_OK;
}
