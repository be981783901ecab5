// finish: merge the scan's split partials (log-sum-exp) into o_hat and the softmax
// statistics, then compute the approximate contribution of the selected set,
//   W = sum_{i in T} p_i,   o_old_unnorm[d] = sum_{i in T} (p_i * vscale_i,g(d)) * vcode_i,d
// (jetfire_vllm/csrc/int2_softmax_v.cu:738-788; V4: csrc/int4_softmax_v.cu:599-817).
//
// Weight swap for the selected set.  The scan's scores skip the reference's bf16 rounding
// of the dequantised key, so a weight can be off by ~1e-3 relative -- visible only on the
// few dominant positions, which are exactly the selected ones.  For every selected
// position the select kernel has the canonical score s_c; here the scan's weight
// exp(s_f - M) is replaced by exp(s_c - M) in the numerator, the normaliser and the
// selected-set terms, so that p_i of the selected set follows the reference arithmetic
// and the remaining (individually small) weights keep their approximate scores.
//
// merge_correct: out = dtype(o_hat + W * float(o_new) - o_old_unnorm)
// (jetfire_vllm/csrc/blend.cu:202-226).  The normaliser stays the approximate softmax's:
// this is mass substitution, not a re-normalised merge.
#include "decode_common.cuh"

namespace jf {

namespace {

constexpr int kFinishThreads = 512;
constexpr int kFinishWarps = kFinishThreads / 32;
constexpr int kSplitGroups = kFinishThreads / JF_HEAD_DIM;  // split partials are summed in 4 strided groups
constexpr int kChunk = 256;                                  // selected entries staged per round

struct FinishParams {
  const float* scores;
  const float* sel_canon;
  const float* part_o;
  const float* part_m;
  const float* part_l;
  const uint8_t* v_data;
  const uint16_t* v_scales;
  const int64_t* block_table;
  const int32_t* seq_lens;
  const int64_t* topk_idx;
  float* o_hat;
  float* o_old;
  float* W;
  float* softmax_m;
  float* softmax_inv_z;
  int64_t num_slots;
  int B, H_q, H_kv, G, max_S, max_blocks, splits, top_k;
};

// One CTA per (query head, batch element).  Everything is arranged as a few rounds of
// independent loads (the kernel is bound by L2 latency, not bandwidth): split statistics,
// then split partials in four strided groups, then per selected entry its slot / weights,
// then all V rows of a chunk into shared memory, then a warp per entry with lane l owning
// channels 4l..4l+3.  Summation orders are fixed (bit-reproducible).
template <int MODE>
__global__ void __launch_bounds__(kFinishThreads)
decode_finish_kernel(const FinishParams p) {
  constexpr int VW = (MODE == JF_MODE_K3V2) ? 8 : 16;  // 32-bit words per packed V row
  __shared__ int64_t sm_slot[kChunk];
  __shared__ float sm_wc[kChunk][2];   // canonical weight * v scale (per group)
  __shared__ float sm_dw[kChunk][2];   // (canonical - scan) weight * v scale
  __shared__ float sm_w[kChunk][2];    // canonical weight, weight difference
  __shared__ uint32_t sm_v[kChunk * VW];
  __shared__ float sm_red[kFinishWarps][JF_HEAD_DIM][2];
  __shared__ float sm_sum[kFinishWarps][2];
  __shared__ float sm_o[kSplitGroups][JF_HEAD_DIM];
  __shared__ float sm_z[kSplitGroups];
  __shared__ float sm_m[kFinishWarps];
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int hkv = h / p.G, hi = h - hkv * p.G;
  const int64_t bh = static_cast<int64_t>(b) * p.H_q + h;
  const int n = min(p.seq_lens[b], p.max_S);

  // ---- merged reference point: max over the splits ----
  const int64_t pbase = (static_cast<int64_t>(b) * p.H_kv + hkv) * p.splits;
  float M = kMinusBig;
  for (int s = tid; s < p.splits; s += kFinishThreads) M = fmaxf(M, p.part_m[(pbase + s) * kHeadsPad + hi]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
  if (lane == 0) sm_m[warp] = M;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < kFinishWarps; ++w) M = fmaxf(M, sm_m[w]);

  // ---- merge splits (unnormalised): thread (group, d) sums splits group, group + 4, ... ----
  {
    const int d = tid & (JF_HEAD_DIM - 1), grp = tid >> 7;
    float o = 0.f, Z = 0.f;
#pragma unroll 4
    for (int s = grp; s < p.splits; s += kSplitGroups) {
      const float w = ex2((p.part_m[(pbase + s) * kHeadsPad + hi] - M) * kLog2e);
      Z = fmaf(p.part_l[(pbase + s) * kHeadsPad + hi], w, Z);
      o = fmaf(p.part_o[((pbase + s) * kHeadsPad + hi) * JF_HEAD_DIM + d], w, o);
    }
    sm_o[grp][d] = o;
    if (d == 0) sm_z[grp] = Z;
  }

  // ---- selected set: canonical weights, and their difference to the scan's ----
  const ModeInfo mi = mode_info(MODE);
  const uint8_t* v_rows = p.v_data + static_cast<int64_t>(hkv) * p.num_slots * mi.v_row;
  const uint16_t* v_sc = p.v_scales + static_cast<int64_t>(hkv) * p.num_slots * mi.ng;
  const int64_t* bt = p.block_table + static_cast<int64_t>(b) * p.max_blocks;
  const float* srow = p.scores + bh * p.max_S;
  const int64_t* sel = p.topk_idx + bh * p.top_k;
  const float* canon = p.sel_canon + bh * p.top_k;
  float a_old[4] = {0.f, 0.f, 0.f, 0.f}, a_dw[4] = {0.f, 0.f, 0.f, 0.f};
  float wsum = 0.f, dz = 0.f;
  const int qg = (MODE == JF_MODE_K3V2) ? (lane >> 4) : 0;  // quant group of channels 4l..4l+3
  for (int k0 = 0; k0 < p.top_k; k0 += kChunk) {
    const int kend = min(kChunk, p.top_k - k0);
    if (tid < kChunk) {
      const int kk = k0 + tid;
      int64_t slot = -1;
      float wc = 0.f, dw = 0.f, vs0 = 0.f, vs1 = 0.f;
      if (kk < p.top_k && n > 0) {
        const int64_t pos = sel[kk];
        if (pos >= 0 && pos < n) {
          const int64_t blk = bt[pos >> 4];
          if (blk >= 0 && blk < (p.num_slots >> 4)) {
            slot = blk * 16 + (pos & 15);
            wc = ex2((canon[kk] - M) * kLog2e);
            dw = wc - ex2((srow[pos] - M) * kLog2e);
            if (MODE == JF_MODE_K3V2) {
              const uint32_t sw = __ldg(reinterpret_cast<const uint32_t*>(v_sc + slot * 2));
              vs0 = __uint_as_float(sw << 16);
              vs1 = __uint_as_float(sw & 0xFFFF0000u);
            } else {
              vs0 = vs1 = bf16_bits_to_f32(__ldg(v_sc + slot));
            }
          }
        }
      }
      sm_slot[tid] = slot;
      sm_w[tid][0] = wc; sm_w[tid][1] = dw;
      sm_wc[tid][0] = wc * vs0; sm_wc[tid][1] = wc * vs1;
      sm_dw[tid][0] = dw * vs0; sm_dw[tid][1] = dw * vs1;
    }
    __syncthreads();
    for (int idx = tid; idx < kend * VW; idx += kFinishThreads) {
      const int c = idx / VW, w = idx - c * VW;
      const int64_t slot = sm_slot[c];
      sm_v[idx] = (slot >= 0) ? __ldg(reinterpret_cast<const uint32_t*>(v_rows + slot * (VW * 4)) + w) : 0u;
    }
    __syncthreads();
    for (int j = warp; j < kend; j += kFinishWarps) {
      if (sm_slot[j] < 0) continue;  // warp-uniform
      float c[4];
      if (MODE == JF_MODE_K3V2) {
        const uint32_t byte = reinterpret_cast<const uint8_t*>(sm_v + j * VW)[lane];
#pragma unroll
        for (int e = 0; e < 4; ++e) c[e] = static_cast<float>(static_cast<int>((byte >> ((3 - e) * 2)) & 3u) - 2);
      } else {
        const uint32_t two = reinterpret_cast<const uint16_t*>(sm_v + j * VW)[lane];
        c[0] = static_cast<float>(static_cast<int>((two >> 4) & 15u) - 8);
        c[1] = static_cast<float>(static_cast<int>(two & 15u) - 8);
        c[2] = static_cast<float>(static_cast<int>((two >> 12) & 15u) - 8);
        c[3] = static_cast<float>(static_cast<int>((two >> 8) & 15u) - 8);
      }
      const float fw = sm_wc[j][qg], fd = sm_dw[j][qg];
#pragma unroll
      for (int e = 0; e < 4; ++e) { a_old[e] = fmaf(fw, c[e], a_old[e]); a_dw[e] = fmaf(fd, c[e], a_dw[e]); }
      wsum += sm_w[j][0];
      dz += sm_w[j][1];
    }
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) { sm_red[warp][4 * lane + e][0] = a_old[e]; sm_red[warp][4 * lane + e][1] = a_dw[e]; }
  if (lane == 0) { sm_sum[warp][0] = wsum; sm_sum[warp][1] = dz; }
  __syncthreads();
  if (tid < JF_HEAD_DIM) {
    float acc_old = 0.f, acc_dw = 0.f, ws = 0.f, dzs = 0.f, o = 0.f, Z = 0.f;
#pragma unroll
    for (int w = 0; w < kFinishWarps; ++w) {
      acc_old += sm_red[w][tid][0]; acc_dw += sm_red[w][tid][1];
      ws += sm_sum[w][0]; dzs += sm_sum[w][1];
    }
#pragma unroll
    for (int gI = 0; gI < kSplitGroups; ++gI) { o += sm_o[gI][tid]; Z += sm_z[gI]; }
    Z += dzs;
    const bool live = (Z > 0.f) && (n > 0);
    const float inv_z = live ? (1.0f / Z) : 0.f;
    p.o_hat[bh * JF_HEAD_DIM + tid] = (o + acc_dw) * inv_z;
    p.o_old[bh * JF_HEAD_DIM + tid] = acc_old * inv_z;
    if (tid == 0) {
      p.W[bh] = ws * inv_z;
      if (p.softmax_m) p.softmax_m[bh] = live ? M : 0.f;
      if (p.softmax_inv_z) p.softmax_inv_z[bh] = inv_z;
    }
  }
}

template <int DT>
__global__ void merge_correct_kernel(const float* __restrict__ o_hat, const float* __restrict__ o_old,
                                     const float* __restrict__ W, const uint16_t* __restrict__ o_new,
                                     uint16_t* __restrict__ out, int total) {
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
  fp.scores = a->scores ? a->scores : ws.scores;
  fp.sel_canon = ws.sel_canon;
  fp.part_o = ws.part_o; fp.part_m = ws.part_m; fp.part_l = ws.part_l;
  fp.v_data = a->v_data; fp.v_scales = static_cast<const uint16_t*>(a->v_scales);
  fp.block_table = a->block_table; fp.seq_lens = a->seq_lens; fp.topk_idx = a->topk_idx;
  fp.o_hat = a->o_hat; fp.o_old = a->o_old_unnorm; fp.W = a->W;
  fp.softmax_m = a->softmax_m; fp.softmax_inv_z = a->softmax_inv_z;
  fp.num_slots = a->num_slots;
  fp.B = a->B; fp.H_q = a->H_q; fp.H_kv = a->H_kv; fp.G = a->H_q / a->H_kv;
  fp.max_S = a->max_S; fp.max_blocks = a->max_blocks;
  fp.splits = scan_splits(a->mode, a->q_dtype, a->B, a->H_kv, a->max_S);
  fp.top_k = a->top_k;
  dim3 grid(a->H_q, a->B);
  if (a->mode == JF_MODE_K3V2) decode_finish_kernel<JF_MODE_K3V2><<<grid, kFinishThreads, 0, stream>>>(fp);
  else decode_finish_kernel<JF_MODE_K4V4><<<grid, kFinishThreads, 0, stream>>>(fp);
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

extern "C" jf_status_t jf_decode_fused(const jf_decode_args* a, jf_stream_t stream) {
  jf_status_t st = jf_decode_scan(a, stream);
  if (st != JF_OK) return st;
  st = jf_topk_select(a, stream);
  if (st != JF_OK) return st;
  return jf_decode_finish(a, stream);
}

extern "C" jf_status_t jf_decode_status(const jf_decode_args* a, jf_stream_t stream_) {
  using namespace jf;
  if (!a || !a->workspace) return JF_ERR_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int32_t host = 0;
  JF_CUDA_TRY(cudaMemcpyAsync(&host, a->workspace, sizeof(host), cudaMemcpyDeviceToHost, stream));
  JF_CUDA_TRY(cudaStreamSynchronize(stream));
  return host == 0 ? JF_OK : static_cast<jf_status_t>(host);
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
    merge_correct_kernel<JF_DTYPE_BF16><<<blocks, threads, 0, stream>>>(
        o_hat, o_old_unnorm, W, static_cast<const uint16_t*>(o_new), static_cast<uint16_t*>(out), total);
  else if (dtype == JF_DTYPE_FP16)
    merge_correct_kernel<JF_DTYPE_FP16><<<blocks, threads, 0, stream>>>(
        o_hat, o_old_unnorm, W, static_cast<const uint16_t*>(o_new), static_cast<uint16_t*>(out), total);
  else
    return JF_ERR_UNSUPPORTED;
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}
