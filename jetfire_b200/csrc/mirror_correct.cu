// Top-k correction on the GPU over the HOST mirror: exact attention over the selected rows, read
// straight from the full-precision mirror in mapped pinned host memory, for a range of the
// (sequence, query head) rows.
//
// The host correction (cpu_correction.cpp; the reference's cpu_topk_attn,
// jetfire_vllm/csrc/cpu_topk_attn.cpp:316-479) is what bounds a decode step end to end: the
// workers gather two 256-byte rows per selected entry at random from a cold mirror, and the GPU
// and its host link idle meanwhile.  This kernel takes a share of the rows off the workers: the
// slots are already on the device, each selected K and V row is one coalesced 256-byte read over
// the link, and the result lands in the device's o_new directly.  Same arithmetic as the host
// path -- s = (q . k) * scale in fp32, softmax over the valid entries, o = sum p * v in fp32,
// rounded once to the 16-bit type; invalid slots count as -inf, a row without a valid entry or
// with a non-positive / non-finite normaliser gives zeros -- in a different summation order, so
// the results agree to rounding, not bit for bit.  The reference has no counterpart on its
// release path (its GPU-side correction, csrc/fused_correction.cu, reads a device-resident copy).
#include "jf_common.cuh"

namespace jf {
namespace {

constexpr int kMcThreads = 256;
constexpr int kMcWarps = kMcThreads / 32;
constexpr int kMcUnroll = 4;   // rows a warp has in flight over the link

template <typename SlotT>
__device__ __forceinline__ int64_t mirror_row(const SlotT* ts, int k, int K, int64_t num_slots) {
  if (k >= K) return -1;
  const int64_t s = static_cast<int64_t>(ts[k]);
  return (s < 0 || s >= num_slots) ? -1 : s;
}

// One block per row; a warp reads a whole 256-byte mirror row per load (8 bytes a lane).
template <int DT, typename SlotT>
__global__ void __launch_bounds__(kMcThreads)
mirror_correct_kernel(const uint16_t* __restrict__ q, const uint16_t* __restrict__ k_mirror,
                      const uint16_t* __restrict__ v_mirror, const SlotT* __restrict__ ts, uint16_t* __restrict__ o_new,
                      int H_q, int H_kv, int64_t num_slots, int K, float scale, int64_t row_begin) {
  extern __shared__ float mc_smem[];          // scores[K] | partial[kMcWarps][128] | red[kMcWarps] x 2
  float* scores = mc_smem;
  float* partial = mc_smem + ((K + 3) & ~3);
  float* red = partial + kMcWarps * JF_HEAD_DIM;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t bh = row_begin + blockIdx.x;
  const int h = static_cast<int>(bh % H_q);
  const int hkv = h / (H_q / H_kv);
  const SlotT* row_ts = ts + bh * K;
  const uint16_t* kbase = k_mirror + static_cast<int64_t>(hkv) * num_slots * JF_HEAD_DIM;
  const uint16_t* vbase = v_mirror + static_cast<int64_t>(hkv) * num_slots * JF_HEAD_DIM;

  float qf[4];
  {
    const uint2 qq = *reinterpret_cast<const uint2*>(q + bh * JF_HEAD_DIM + 4 * lane);
    qf[0] = Elem<DT>::to_f32(static_cast<uint16_t>(qq.x & 0xFFFFu));
    qf[1] = Elem<DT>::to_f32(static_cast<uint16_t>(qq.x >> 16));
    qf[2] = Elem<DT>::to_f32(static_cast<uint16_t>(qq.y & 0xFFFFu));
    qf[3] = Elem<DT>::to_f32(static_cast<uint16_t>(qq.y >> 16));
  }

  // ---- scores ----
  float my_max = -INFINITY;
  for (int k0 = warp * kMcUnroll; k0 < K; k0 += kMcWarps * kMcUnroll) {
    int64_t slot[kMcUnroll];
    uint2 raw[kMcUnroll];
#pragma unroll
    for (int u = 0; u < kMcUnroll; ++u) {
      slot[u] = mirror_row(row_ts, k0 + u, K, num_slots);
      raw[u] = make_uint2(0u, 0u);
      if (slot[u] >= 0) raw[u] = *reinterpret_cast<const uint2*>(kbase + slot[u] * JF_HEAD_DIM + 4 * lane);
    }
#pragma unroll
    for (int u = 0; u < kMcUnroll; ++u) {
      float d = qf[0] * Elem<DT>::to_f32(static_cast<uint16_t>(raw[u].x & 0xFFFFu));
      d = fmaf(qf[1], Elem<DT>::to_f32(static_cast<uint16_t>(raw[u].x >> 16)), d);
      d = fmaf(qf[2], Elem<DT>::to_f32(static_cast<uint16_t>(raw[u].y & 0xFFFFu)), d);
      d = fmaf(qf[3], Elem<DT>::to_f32(static_cast<uint16_t>(raw[u].y >> 16)), d);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xFFFFFFFFu, d, o);
      const float s = slot[u] >= 0 ? d * scale : -INFINITY;
      if (k0 + u < K) {
        if (lane == 0) scores[k0 + u] = s;
        my_max = fmaxf(my_max, s);
      }
    }
  }
  if (lane == 0) red[warp] = my_max;
  __syncthreads();
  float row_max = red[0];
#pragma unroll
  for (int w = 1; w < kMcWarps; ++w) row_max = fmaxf(row_max, red[w]);
  uint16_t* out = o_new + bh * JF_HEAD_DIM;
  if (!(row_max > -INFINITY) || !(row_max < INFINITY)) {   // no valid entry, or a NaN / +inf score: zeros
    if (threadIdx.x < JF_HEAD_DIM) out[threadIdx.x] = 0;
    return;
  }

  // ---- weights and the weighted sum of the V rows ----
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  float my_sum = 0.f;
  for (int k0 = warp * kMcUnroll; k0 < K; k0 += kMcWarps * kMcUnroll) {
    int64_t slot[kMcUnroll];
    uint2 raw[kMcUnroll];
#pragma unroll
    for (int u = 0; u < kMcUnroll; ++u) {
      slot[u] = mirror_row(row_ts, k0 + u, K, num_slots);
      raw[u] = make_uint2(0u, 0u);
      if (slot[u] >= 0) raw[u] = *reinterpret_cast<const uint2*>(vbase + slot[u] * JF_HEAD_DIM + 4 * lane);
    }
#pragma unroll
    for (int u = 0; u < kMcUnroll; ++u) {
      if (k0 + u >= K || slot[u] < 0) continue;
      const float p = __expf(scores[k0 + u] - row_max);
      my_sum += p;
      acc[0] = fmaf(p, Elem<DT>::to_f32(static_cast<uint16_t>(raw[u].x & 0xFFFFu)), acc[0]);
      acc[1] = fmaf(p, Elem<DT>::to_f32(static_cast<uint16_t>(raw[u].x >> 16)), acc[1]);
      acc[2] = fmaf(p, Elem<DT>::to_f32(static_cast<uint16_t>(raw[u].y & 0xFFFFu)), acc[2]);
      acc[3] = fmaf(p, Elem<DT>::to_f32(static_cast<uint16_t>(raw[u].y >> 16)), acc[3]);
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) partial[warp * JF_HEAD_DIM + 4 * lane + c] = acc[c];
  if (lane == 0) red[kMcWarps + warp] = my_sum;   // every lane of a warp saw the same weights
  __syncthreads();
  if (threadIdx.x < JF_HEAD_DIM) {
    float denom = 0.f, v = 0.f;
#pragma unroll
    for (int w = 0; w < kMcWarps; ++w) {
      denom += red[kMcWarps + w];
      v += partial[w * JF_HEAD_DIM + threadIdx.x];
    }
    const bool ok = denom > 0.f && denom < INFINITY;
    out[threadIdx.x] = ok ? Elem<DT>::from_f32(v / denom) : static_cast<uint16_t>(0);
  }
}

template <int DT, typename SlotT>
jf_status_t launch_mirror_correct(const void* q, const void* km, const void* vm, const void* ts, void* o_new, int H_q,
                                  int H_kv, int64_t num_slots, int K, float scale, int64_t row_begin, int64_t rows,
                                  cudaStream_t stream) {
  const size_t smem = (static_cast<size_t>((K + 3) & ~3) + kMcWarps * JF_HEAD_DIM + 2 * kMcWarps) * sizeof(float);
  mirror_correct_kernel<DT, SlotT><<<static_cast<unsigned>(rows), kMcThreads, smem, stream>>>(
      static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(km), static_cast<const uint16_t*>(vm),
      static_cast<const SlotT*>(ts), static_cast<uint16_t*>(o_new), H_q, H_kv, num_slots, K, scale, row_begin);
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

}  // namespace
}  // namespace jf

extern "C" jf_status_t jf_gpu_topk_attn_rows(const void* q, const void* k_mirror_dev, const void* v_mirror_dev,
                                             const void* topk_slots, int32_t slots_are_i32, void* o_new, int32_t dtype,
                                             int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots, int32_t K, float scale,
                                             int64_t row_begin, int64_t row_end, jf_stream_t stream_) {
  using namespace jf;
  if (!q || !k_mirror_dev || !v_mirror_dev || !topk_slots || !o_new) return JF_ERR_ARG;
  if (B <= 0 || H_q <= 0 || H_kv <= 0 || K <= 0 || num_slots <= 0 || H_q % H_kv != 0) return JF_ERR_ARG;
  if (row_begin < 0 || row_end < row_begin || row_end > static_cast<int64_t>(B) * H_q) return JF_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_mirror_dev) | reinterpret_cast<uintptr_t>(v_mirror_dev)) & 7)
    return JF_ERR_ARG;
  if (K > JF_MAX_TOP_K) return JF_ERR_UNSUPPORTED;
  if (row_end == row_begin) return JF_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int64_t rows = row_end - row_begin;
  if (dtype == JF_DTYPE_BF16) {
    return slots_are_i32 ? launch_mirror_correct<JF_DTYPE_BF16, int32_t>(q, k_mirror_dev, v_mirror_dev, topk_slots, o_new, H_q, H_kv, num_slots, K, scale, row_begin, rows, stream)
                         : launch_mirror_correct<JF_DTYPE_BF16, int64_t>(q, k_mirror_dev, v_mirror_dev, topk_slots, o_new, H_q, H_kv, num_slots, K, scale, row_begin, rows, stream);
  }
  if (dtype == JF_DTYPE_FP16) {
    return slots_are_i32 ? launch_mirror_correct<JF_DTYPE_FP16, int32_t>(q, k_mirror_dev, v_mirror_dev, topk_slots, o_new, H_q, H_kv, num_slots, K, scale, row_begin, rows, stream)
                         : launch_mirror_correct<JF_DTYPE_FP16, int64_t>(q, k_mirror_dev, v_mirror_dev, topk_slots, o_new, H_q, H_kv, num_slots, K, scale, row_begin, rows, stream);
  }
  return JF_ERR_UNSUPPORTED;
}
