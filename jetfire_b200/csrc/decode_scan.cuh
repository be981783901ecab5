// Pieces shared by the per-mode scan kernels: parameters, ring-slot geometry, the CTA-level
// merge of the four warps' partials.
#pragma once

#include "decode_common.cuh"

namespace jf {

template <int MODE> struct Tile;
template <> struct Tile<JF_MODE_K3V2> {
  // A warp's ring is made of two-page slots: [K page A | K page B | V page A | V page B |
  // K scales A, B | V scales A, B]; two pages whose blocks are neighbours in the cache are
  // fetched with one bulk copy per array.
  static constexpr int kKRow = 48, kVRow = 32, kNG = 2;
  static constexpr int kKPage = 768, kVPage = 512, kSPage = 64;   // bytes per page and array
  static constexpr int kVOff = 1536, kKsOff = 2560, kVsRel = 128; // slot-relative; V scales from the K scales
  static constexpr int kSlotBytes = 2816;
  static constexpr int kPageTx = 1408;    // bytes that land per page
  static constexpr int kSlots = 4;        // two-page slots per warp: eight pages in flight
};
template <> struct Tile<JF_MODE_K4V4> {
  // A warp's ring is made of two-page slots: [K page A | K page B | V page A | V page B |
  // K scales A, B | V scales A, B].  Two pages whose blocks are neighbours in the cache are
  // fetched as one 32-row tensor copy per tensor and one 64-byte copy per scale array; the
  // tiles are written by swizzled tensor copies and sit on 1024-byte boundaries.
  static constexpr int kKRow = 64, kVRow = 64, kNG = 1;
  static constexpr int kPageBytes = 1024;                 // K (or V) data of one page
  static constexpr int kVOff = 2048;                      // V page, from the K page of the same half
  static constexpr int kScaleOff = 4096;                  // K scales of half 0, from the slot base
  static constexpr int kVsOff = 64;                       // V scales, from the K scales of the same half
  static constexpr int kSlotBytes = 4608;
  static constexpr int kPageTx = 2112;                    // bytes that land per page
  static constexpr int kSlots = 2;                        // two-page slots per warp (4 CTAs = 16 warps per SM)
};

struct ScanParams {
  const void* q;
  const uint8_t* k_data;
  const uint16_t* k_scales;
  const uint8_t* v_data;
  const uint16_t* v_scales;
  const int64_t* block_table;
  const int32_t* seq_lens;
  float* scores;
  float* pmax;          // K3V2: largest score of every pair of pages, [B][H_q][np_stride] (see the select kernel)
  float* part_o;
  float* part_m;
  float* part_l;
  float* part_smax;
  int32_t* status;
  int64_t num_slots;
  int B, H_q, H_kv, G, max_S, max_blocks, splits, pages_per_split;
  int pages_per_warp;   // a warp's contiguous share of a split: ceil(pages_per_split / kScanWarps)
  float attn_scale;
  int q_dtype;
  int kv_shift;         // cache head = KV head >> kv_shift (see head_geom)
  int np_stride;        // entries per row of pmax
  // K4V4: work is cut into two-page tiles (see scan_k4v4_kernel)
  int n_tiles, tiles_per_split, tiles_per_warp, ref_chunk;
  int tile_base[9];
};

constexpr uint32_t kMagic = 0x64006400u;  // fp16 1024.0 in both halves
constexpr int kBtChunk = 16;              // block-table entries fetched per load (one per lane of a half-warp)

template <int DT>
__device__ __forceinline__ float load_q(const void* q, int64_t idx) {
  return Elem<DT>::to_f32(reinterpret_cast<const uint16_t*>(q)[idx]);
}


// Bytes of shared memory the merge needs (per-warp output tiles + statistics).
constexpr int kMergeBytes = (kScanWarps * kHeadsPad * JF_HEAD_DIM + 3 * kScanWarps * kHeadsPad) * 4;

// CTA-level merge, fixed summation order (bit-reproducible, no atomics).  Before the call
// every warp has written its un-permuted output tile to sm_o[warp][head][d]; l0/l1 are
// the lane's partial softmax sums for heads 2*tig and 2*tig+1, m_ref0/1 its reference
// points, smax0/1 the largest K group scales it saw.
__device__ __forceinline__ void cta_merge_store(const ScanParams& p, uint8_t* smem, float l0, float l1,
                                                float m_ref0, float m_ref1, float smax0, float smax1,
                                                int split, int hkv, int b) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  float* sm_o = reinterpret_cast<float*>(smem);               // [4 warps][8][128]
  float* sm_m = sm_o + kScanWarps * kHeadsPad * JF_HEAD_DIM;  // [4][8]
  float* sm_l = sm_m + kScanWarps * kHeadsPad;                // [4][8]
  float* sm_s = sm_l + kScanWarps * kHeadsPad;                // [4][2]
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l0 += __shfl_xor_sync(0xFFFFFFFFu, l0, o);
    l1 += __shfl_xor_sync(0xFFFFFFFFu, l1, o);
  }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    smax0 = fmaxf(smax0, __shfl_xor_sync(0xFFFFFFFFu, smax0, o));
    smax1 = fmaxf(smax1, __shfl_xor_sync(0xFFFFFFFFu, smax1, o));
  }
  if (g == 0) {
    sm_m[warp * 8 + 2 * tig] = m_ref0; sm_m[warp * 8 + 2 * tig + 1] = m_ref1;
    sm_l[warp * 8 + 2 * tig] = l0;     sm_l[warp * 8 + 2 * tig + 1] = l1;
  }
  if (lane == 0) { sm_s[warp * 2] = smax0; sm_s[warp * 2 + 1] = smax1; }
  __syncthreads();
  const int64_t pidx = (static_cast<int64_t>(b) * p.H_kv + hkv) * p.splits + split;
  float* po = p.part_o + pidx * (kHeadsPad * JF_HEAD_DIM);
  for (int i = threadIdx.x; i < kHeadsPad * JF_HEAD_DIM; i += blockDim.x) {
    const int h = i >> 7;
    float M = kMinusBig;
#pragma unroll
    for (int w = 0; w < kScanWarps; ++w) M = fmaxf(M, sm_m[w * 8 + h]);
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < kScanWarps; ++w)
      acc = fmaf(sm_o[w * (kHeadsPad * JF_HEAD_DIM) + i], ex2((sm_m[w * 8 + h] - M) * kLog2e), acc);
    po[i] = acc;
  }
  if (threadIdx.x < kHeadsPad) {
    const int h = threadIdx.x;
    float M = kMinusBig;
    for (int w = 0; w < kScanWarps; ++w) M = fmaxf(M, sm_m[w * 8 + h]);
    float L = 0.f;
    for (int w = 0; w < kScanWarps; ++w) L += sm_l[w * 8 + h] * ex2((sm_m[w * 8 + h] - M) * kLog2e);
    p.part_m[pidx * kHeadsPad + h] = M;
    p.part_l[pidx * kHeadsPad + h] = L;
  }
  if (threadIdx.x < 2) {
    float s = 0.f;
    for (int w = 0; w < kScanWarps; ++w) s = fmaxf(s, sm_s[w * 2 + threadIdx.x]);
    p.part_smax[pidx * 2 + threadIdx.x] = s;
  }
}

// Online-softmax step shared by the modes: the reference point may lag the true maximum
// by less than 4 (so exp stays below e^4 and the fp16 P operand cannot overflow); the
// exact warp-wide maximum is only taken when a score runs ahead of it.
template <int NT>
__device__ __forceinline__ void softmax_step(float s0, float s1, float s2, float s3, float& m_ref0, float& m_ref1,
                                             float& l0, float& l1, float (&oacc)[NT][4], float& p0, float& p1,
                                             float& p2, float& p3) {
  float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
  const bool need = (mx0 > m_ref0 + 4.0f) || (mx1 > m_ref1 + 4.0f);
  if (__any_sync(0xFFFFFFFFu, need)) {
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, o));
    }
    const float n0 = fmaxf(m_ref0, mx0), n1 = fmaxf(m_ref1, mx1);
    const float f0 = ex2((m_ref0 - n0) * kLog2e), f1 = ex2((m_ref1 - n1) * kLog2e);
    l0 *= f0; l1 *= f1;
#pragma unroll
    for (int i = 0; i < NT; ++i) { oacc[i][0] *= f0; oacc[i][1] *= f1; oacc[i][2] *= f0; oacc[i][3] *= f1; }
    m_ref0 = n0; m_ref1 = n1;
  }
  const float mb0 = m_ref0 * kLog2e, mb1 = m_ref1 * kLog2e;
  p0 = ex2(fmaf(s0, kLog2e, -mb0)); p1 = ex2(fmaf(s1, kLog2e, -mb1));
  p2 = ex2(fmaf(s2, kLog2e, -mb0)); p3 = ex2(fmaf(s3, kLog2e, -mb1));
  l0 += p0 + p2;
  l1 += p1 + p3;
}

// parts: 0 = scores and output partials, 1 = scores and softmax sums only, 2 = output partials from
// stored scores; int8p: the reference's batch > 1 weight rounding
jf_status_t launch_scan_k4v4(ScanParams sp, bool int8p, int parts, dim3 grid, cudaStream_t stream);

}  // namespace jf
