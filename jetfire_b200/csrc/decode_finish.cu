// finish (stand-alone): the finish stage for a selected list that is already in memory --
// the phase-by-phase API; the fused entry point runs the same code inside the select kernel.
//
// merge_correct: out = dtype(o_hat + W * float(o_new) - o_old_unnorm)
// (jetfire_vllm/csrc/blend.cu:202-226).  The normaliser stays the approximate softmax's:
// this is mass substitution, not a re-normalised merge.
#include "finish_tail.cuh"

namespace jf {

namespace {

struct FinishParams {
  const int64_t* block_table;
  const int32_t* seq_lens;
  const int64_t* topk_idx;
  int max_blocks;
};

// One CTA per (query head, batch element).
template <int MODE>
__global__ void __launch_bounds__(kSelThreads)
decode_finish_kernel(const FinishParams p, const TailParams tp) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  TailSmem<MODE>& tsm = *reinterpret_cast<TailSmem<MODE>*>(smem_raw);
  __shared__ float sm_m[kSelWarps];
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int hkv = h / tp.G, hi = h - hkv * tp.G;
  const int64_t bh = static_cast<int64_t>(b) * tp.H_q + h;
  const int64_t pbase = (static_cast<int64_t>(b) * tp.H_kv + hkv) * tp.splits;
  pdl_wait();
  SplitPre pre;
  split_preload(tp, pbase, hi, tid, pre);
  const int n = min(p.seq_lens[b], tp.max_S);
  const float M = block_max_of_splits(tp.part_m, pbase, hi, tp.splits, sm_m);
  const int64_t* sel = p.topk_idx + bh * tp.top_k;
  finish_tail<MODE>(tp, tsm, TailPrefetch{}, pre, M, n, b, h, p.block_table + static_cast<int64_t>(b) * p.max_blocks,
                    [&](int kk, int& pos, int& cidx) {
                      const int64_t v = sel[kk];
                      if (v < 0 || v >= n) return false;
                      pos = static_cast<int>(v);
                      cidx = -1;
                      return true;
                    });
}

template <int DT>
__global__ void merge_correct_kernel(const float* __restrict__ o_hat, const float* __restrict__ o_old,
                                     const float* __restrict__ W, const uint16_t* __restrict__ o_new,
                                     uint16_t* __restrict__ out, int total) {
  pdl_wait();
  pdl_trigger();  // the next kernel may start its prologue; it waits for this grid before reading
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float w = W[i / JF_HEAD_DIM];
  const float v = o_hat[i] + w * Elem<DT>::to_f32(o_new[i]) - o_old[i];
  out[i] = Elem<DT>::from_f32(v);
}

}  // namespace

}  // namespace jf

extern "C" jf_status_t jf_decode_finish(const jf_decode_args* a, jf_stream_t stream_) {
  using namespace jf;
  jf_status_t st = validate_decode_args(a);
  if (st != JF_OK) return st;
  if (!a->topk_idx || !a->o_hat || !a->o_old_unnorm || !a->W) return JF_ERR_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  Workspace ws = carve_workspace(a->workspace, a->mode, a->B, a->H_q, a->H_kv, a->max_S, a->top_k, true);
  FinishParams fp{};
  fp.block_table = a->block_table; fp.seq_lens = a->seq_lens; fp.topk_idx = a->topk_idx;
  fp.max_blocks = a->max_blocks;
  const TailParams tp = make_tail_params(a, ws);
  dim3 grid(a->H_q, a->B);
  if (a->mode == JF_MODE_K3V2) {
    JF_ENSURE_SMEM((decode_finish_kernel<JF_MODE_K3V2>), sizeof(TailSmem<JF_MODE_K3V2>));
    JF_CUDA_TRY(launch_pdl(decode_finish_kernel<JF_MODE_K3V2>, grid, dim3(kSelThreads), sizeof(TailSmem<JF_MODE_K3V2>), stream, fp, tp));
  } else {
    JF_ENSURE_SMEM((decode_finish_kernel<JF_MODE_K4V4>), sizeof(TailSmem<JF_MODE_K4V4>));
    JF_CUDA_TRY(launch_pdl(decode_finish_kernel<JF_MODE_K4V4>, grid, dim3(kSelThreads), sizeof(TailSmem<JF_MODE_K4V4>), stream, fp, tp));
  }
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

// scan, then select + finish in one kernel
extern "C" jf_status_t jf_decode_fused(const jf_decode_args* a, jf_stream_t stream) {
  jf_status_t st = jf_decode_scan(a, stream);
  if (st != JF_OK) return st;
  return jf::launch_select(a, static_cast<cudaStream_t>(stream), true);
}

extern "C" jf_status_t jf_decode_status(const jf_decode_args* a, jf_stream_t stream_) {
  using namespace jf;
  if (!a || !a->workspace) return JF_ERR_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  struct { unsigned long long tag; int32_t code; int32_t pad; } host{};
  JF_CUDA_TRY(cudaMemcpyAsync(&host, a->workspace, sizeof(host), cudaMemcpyDeviceToHost, stream));
  JF_CUDA_TRY(cudaStreamSynchronize(stream));
  if (host.tag != kStatusTag || host.code == 0) return JF_OK;
  JF_CUDA_TRY(cudaMemsetAsync(a->workspace, 0, sizeof(host), stream));
  JF_CUDA_TRY(cudaStreamSynchronize(stream));
  return static_cast<jf_status_t>(host.code);
}

extern "C" jf_status_t jf_merge_correct(const float* o_hat, const float* o_old_unnorm, const float* W,
                                        const void* o_new, void* out, int32_t dtype, int32_t B,
                                        int32_t H_q, jf_stream_t stream_) {
  using namespace jf;
  if (!o_hat || !o_old_unnorm || !W || !o_new || !out || B <= 0 || H_q <= 0) return JF_ERR_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int total = B * H_q * JF_HEAD_DIM;
  const int threads = 256, blocks = (total + threads - 1) / threads;
  if (dtype == JF_DTYPE_BF16)
    JF_CUDA_TRY(launch_pdl(merge_correct_kernel<JF_DTYPE_BF16>, dim3(blocks), dim3(threads), 0, stream, o_hat,
                           o_old_unnorm, W, static_cast<const uint16_t*>(o_new), static_cast<uint16_t*>(out), total));
  else if (dtype == JF_DTYPE_FP16)
    JF_CUDA_TRY(launch_pdl(merge_correct_kernel<JF_DTYPE_FP16>, dim3(blocks), dim3(threads), 0, stream, o_hat,
                           o_old_unnorm, W, static_cast<const uint16_t*>(o_new), static_cast<uint16_t*>(out), total));
  else
    return JF_ERR_UNSUPPORTED;
  return JF_OK;
}
