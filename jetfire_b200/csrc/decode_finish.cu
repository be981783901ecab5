// finish (stand-alone): the finish stage for a selected list that is already in memory --
// the phase-by-phase API; the fused entry point runs the same code inside the select kernel.
//
// merge_correct: out = dtype(o_hat + W * float(o_new) - o_old_unnorm)
// (jetfire_vllm/csrc/blend.cu:202-226).  The normaliser stays the approximate softmax's:
// this is mass substitution, not a re-normalised merge.
#include <cstring>

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
  SplitPre<kSelThreads> pre;
  split_preload<kSelThreads>(tp, pbase, hi, tid, pre);
  const int n = min(p.seq_lens[b], tp.max_S);
  const float M = block_max_of_splits(tp.part_m, pbase, hi, tp.splits, sm_m);
  const int64_t* sel = p.topk_idx + bh * tp.top_k;
  finish_tail<MODE, kSelThreads>(tp, tsm, TailPrefetch{}, pre, M, n, b, h, p.block_table + static_cast<int64_t>(b) * p.max_blocks,
                    [&](int kk, int& pos, int& cidx) {
                      const int64_t v = sel[kk];
                      if (v < 0 || v >= n) return false;
                      pos = static_cast<int>(v);
                      cidx = -1;
                      return true;
                    });
}

// Exact row maximum and 1 / sum exp(s - max) of a stored score row, as the reference's
// statistics-emitting select computes them (jetfire_vllm/csrc/int8tc_qk_scores.cu:1790-1800):
// an empty or all -inf row gives m = 0, and a non-positive sum gives 1/Z = 0.
// One CTA per (query head, batch element); sums in a fixed order.
__global__ void __launch_bounds__(256)
softmax_stats_kernel(const float* __restrict__ scores, const int32_t* __restrict__ seq_lens, float* __restrict__ out_m,
                     float* __restrict__ out_inv_z, int H_q, int max_S) {
  __shared__ float red[8];
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  const int n = max(0, min(seq_lens[b], max_S));
  const float* row = scores + (static_cast<int64_t>(b) * H_q + h) * max_S;
  float m = -INFINITY;
  for (int i = tid; i < n; i += 256) m = fmaxf(m, row[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, o));
  if (lane == 0) red[warp] = m;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < 8; ++w) m = fmaxf(m, red[w]);
  if (!isfinite(m)) m = 0.f;
  __syncthreads();
  float z = 0.f;
  for (int i = tid; i < n; i += 256) z += __expf(row[i] - m);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xFFFFFFFFu, z, o);
  if (lane == 0) red[warp] = z;
  __syncthreads();
  if (tid == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w];
    out_m[static_cast<int64_t>(b) * H_q + h] = m;
    out_inv_z[static_cast<int64_t>(b) * H_q + h] = t > 0.f ? 1.0f / t : 0.f;
  }
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

extern "C" jf_status_t jf_softmax_stats(const float* scores, const int32_t* seq_lens, float* softmax_m,
                                        float* softmax_inv_z, int32_t B, int32_t H_q, int32_t max_S,
                                        jf_stream_t stream_) {
  using namespace jf;
  if (!scores || !seq_lens || !softmax_m || !softmax_inv_z || B <= 0 || H_q <= 0 || max_S <= 0) return JF_ERR_ARG;
  JF_CUDA_TRY(launch_pdl(softmax_stats_kernel, dim3(H_q, B), dim3(256), 0, static_cast<cudaStream_t>(stream_), scores,
                         seq_lens, softmax_m, softmax_inv_z, static_cast<int>(H_q), static_cast<int>(max_S)));
  return JF_OK;
}

// scan, then select + finish in one kernel
extern "C" jf_status_t jf_decode_fused(const jf_decode_args* a, jf_stream_t stream) {
  if (a && a->scan_parts != JF_SCAN_ALL) return JF_ERR_ARG;   // the fused step needs both halves
  jf_status_t st = jf_decode_scan(a, stream);
  if (st != JF_OK) return st;
  return jf::launch_select(a, static_cast<cudaStream_t>(stream), true);
}

// select + finish in one kernel, after a scan that ran on its own (the second half of jf_decode_fused)
extern "C" jf_status_t jf_select_finish(const jf_decode_args* a, jf_stream_t stream) {
  if (a && a->scan_parts == JF_SCAN_K_ONLY) return JF_ERR_ARG;   // the finish stage needs the V side
  return jf::launch_select(a, static_cast<cudaStream_t>(stream), true);
}

extern "C" jf_status_t jf_decode_status(const jf_decode_args* a, jf_stream_t stream_) {
  using namespace jf;
  if (!a) return JF_ERR_ARG;
  // no workspace: the calls went through jf_decode_fused_static, whose record is in the built-in array
  void* record = a->workspace;
  if (!record) {
    const jf_status_t st = static_scratch_address(&record);
    if (st != JF_OK) return st;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  struct { unsigned long long tag; int32_t code; int32_t pad; } host{};
  JF_CUDA_TRY(cudaMemcpyAsync(&host, record, sizeof(host), cudaMemcpyDeviceToHost, stream));
  JF_CUDA_TRY(cudaStreamSynchronize(stream));
  if (host.tag != kStatusTag || host.code == 0) return JF_OK;
  JF_CUDA_TRY(cudaMemsetAsync(record, 0, sizeof(host), stream));
  JF_CUDA_TRY(cudaStreamSynchronize(stream));
  return static_cast<jf_status_t>(host.code);
}

// The same reading on a host copy of the record's first 16 bytes, for callers that bring the
// record over with a copy of their own in the stream (no synchronisation here, nothing cleared).
extern "C" jf_status_t jf_decode_status_of_copy(const void* record_copy) {
  if (!record_copy) return JF_ERR_ARG;
  struct { unsigned long long tag; int32_t code; int32_t pad; } host{};
  memcpy(&host, record_copy, sizeof(host));
  if (host.tag != jf::kStatusTag || host.code == 0) return JF_OK;
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
