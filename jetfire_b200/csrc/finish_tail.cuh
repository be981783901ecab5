// Finish stage shared by the fused select+finish kernel and the stand-alone finish kernel:
// merge the scan's split partials (log-sum-exp) into o_hat and the softmax statistics, and
// compute the approximate contribution of the selected set from the scan's own scores,
//   W = sum_{i in T} p_i,   o_old_unnorm[d] = sum_{i in T} (p_i * vscale_i,g(d)) * vcode_i,d
// (jetfire_vllm/csrc/int2_softmax_v.cu:738-788; V4: csrc/int4_softmax_v.cu:599-817), as the
// reference's Stage B does with the scores of its Stage A: what the later merge subtracts
// is exactly what the approximate pass added for these positions.
//
// Every summation order is fixed (no floating-point atomics) and does not depend on the block
// size: a block of NT threads plays the 1024 thread-items and the 32 warps of the widest
// block one after the other, so every kernel that runs this code gives the same bits.
//
// The selected set's sum runs on the tensor cores like the scan's P.V: sixteen staged entries
// are a "page" (their packed V rows lie one after the other in shared memory), the masked code
// fields go to mma.sync.m16n8k16 as subnormal fp16 numbers without arithmetic, the weights
// (times the V group scale, rounded to fp16 as the scan rounds its P operand) are the other
// operand -- one column of it; the codes' offset leaves through a sum-of-weights tile.
#pragma once

#include "decode_common.cuh"

namespace jf {

constexpr int kSelThreads = 1024;                        // widest block; the unit of the fixed orders below
constexpr int kSelWarps = kSelThreads / 32;
constexpr int kSplitGroups = kSelThreads / JF_HEAD_DIM;  // split partials are summed in 8 strided groups
constexpr int kSplitPre = 4;                             // partials per thread fetched ahead of use (all its items together)
constexpr int kTailChunk = 256;                          // selected entries staged per round
constexpr int kTailPerWarp = kTailChunk / kSelWarps;

struct TailParams {
  const float* scores;
  const float* part_o;
  const float* part_m;
  const float* part_l;
  const uint8_t* v_data;
  const uint16_t* v_scales;
  float* o_hat;
  float* o_old;
  float* W;
  float* softmax_m;
  float* softmax_inv_z;
  int64_t num_slots;
  int H_q, H_kv, G, max_S, splits, top_k;
  int kv_shift;   // cache head = KV head >> kv_shift (see head_geom)
};

template <int MODE>
struct TailSmem {
  static constexpr int VW = (MODE == JF_MODE_K3V2) ? 8 : 16;  // 32-bit words per packed V row
  uint32_t v[kTailChunk * VW];                                 // first: 16-byte aligned
  int64_t slot[kTailChunk];
  int cidx[kTailChunk];      // candidate index in the prefetched arrays, or -1
  float wv[kTailChunk][2];   // weight * v scale (per group)
  float red[kSelWarps][JF_HEAD_DIM];
  float sum[kSelWarps];
  float o[kSplitGroups][JF_HEAD_DIM];
  float z[kSplitGroups];
};

// The first kSplitPre split partials of thread (group, d), loaded before they are needed so
// that their latency hides behind other work.
// Thread-item `it` = (group it >> 7, channel it & 127) of the 1024; a thread of an NT-wide block
// owns items tid, tid + NT, ... and preloads the first kSplitPre * NT / 1024 splits of each.
template <int NT>
struct SplitPre {
  static constexpr int kItems = kSelThreads / NT, kPer = kSplitPre / kItems;
  float m[kItems][kPer], l[kItems][kPer], o[kItems][kPer];
};

template <int NT>
__device__ __forceinline__ void split_preload(const TailParams& p, int64_t pbase, int hi, int tid, SplitPre<NT>& r) {
#pragma unroll
  for (int k = 0; k < SplitPre<NT>::kItems; ++k) {
    const int it = tid + k * NT;
    const int d = it & (JF_HEAD_DIM - 1), grp = it >> 7;
#pragma unroll
    for (int i = 0; i < SplitPre<NT>::kPer; ++i) {
      const int s = grp + i * kSplitGroups;
      r.m[k][i] = kMinusBig; r.l[k][i] = 0.f; r.o[k][i] = 0.f;
      if (s < p.splits) {
        const int64_t e = (pbase + s) * kHeadsPad + hi;
        r.m[k][i] = p.part_m[e];
        r.l[k][i] = p.part_l[e];
        r.o[k][i] = p.part_o[e * JF_HEAD_DIM + d];
      }
    }
  }
}

// code - bias as a float without an integer-to-float conversion: 2^23 + code is the float
// with `code` in its low mantissa bits.
__device__ __forceinline__ float small_code_to_f32(uint32_t code, float bias) {
  return __uint_as_float(0x4B000000u | code) - (8388608.0f + bias);
}

// What the fused kernel already holds in shared memory per candidate (null pointers in the
// stand-alone kernel): slot, scan score, V scales, packed V row.  The values are the ones
// the stand-alone kernel reads from global memory, so both give the same bits.
struct TailPrefetch {
  const int64_t* slot;
  const float* score;
  const uint32_t* vsc;    // K3: both group scales; K4: the aligned pair of scales that holds this slot's
  const uint32_t* vrows;
};

// `src(kk, pos, cidx)` yields the kk-th selected entry (rank order): its position and its
// index in the prefetched arrays (-1: none); false if there is no such entry.  M = max over
// the splits of the scan's reference points.  n = sequence length.
template <int MODE, int NT, typename Src>
__device__ __forceinline__ void finish_tail(const TailParams& p, TailSmem<MODE>& sm, const TailPrefetch& pf,
                                            const SplitPre<NT>& pre, float M, int n, int b, int h, const int64_t* bt,
                                            Src src) {
  constexpr int VW = TailSmem<MODE>::VW;
  constexpr int kW = NT / 32;                 // warps of this block
  constexpr int kPre = SplitPre<NT>::kPer;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hkv = h / p.G, hi = h - hkv * p.G;
  const int64_t bh = static_cast<int64_t>(b) * p.H_q + h;
  const int64_t pbase = (static_cast<int64_t>(b) * p.H_kv + hkv) * p.splits;

  // ---- merge splits (unnormalised): thread (group, d) sums splits group, group + 8, ... ----
#pragma unroll
  for (int k = 0; k < SplitPre<NT>::kItems; ++k) {
    const int it = tid + k * NT;
    const int d = it & (JF_HEAD_DIM - 1), grp = it >> 7;
    float o = 0.f, Z = 0.f;
#pragma unroll
    for (int i = 0; i < kPre; ++i) {
      if (grp + i * kSplitGroups < p.splits) {
        const float w = ex2((pre.m[k][i] - M) * kLog2e);
        Z = fmaf(pre.l[k][i], w, Z);
        o = fmaf(pre.o[k][i], w, o);
      }
    }
    // the remaining splits four at a time: the twelve loads first (with many splits -- few
    // (sequence, KV head) pairs on the GPU -- one load after the other made this the longest part
    // of the stage), then the sums in the same ascending order as before
    for (int s = grp + kPre * kSplitGroups; s < p.splits; s += 4 * kSplitGroups) {
      float pm[4], pl[4], po[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int su = s + u * kSplitGroups;
        pm[u] = kMinusBig; pl[u] = 0.f; po[u] = 0.f;
        if (su < p.splits) {
          const int64_t e = (pbase + su) * kHeadsPad + hi;
          pm[u] = p.part_m[e];
          pl[u] = p.part_l[e];
          po[u] = p.part_o[e * JF_HEAD_DIM + d];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (s + u * kSplitGroups < p.splits) {
          const float w = ex2((pm[u] - M) * kLog2e);
          Z = fmaf(pl[u], w, Z);
          o = fmaf(po[u], w, o);
        }
      }
    }
    sm.o[grp][d] = o;
    if (d == 0) sm.z[grp] = Z;
  }

  // ---- selected set: weights from the scan's scores ----
  const ModeInfo mi = mode_info(MODE);
  const uint8_t* v_rows = p.v_data + static_cast<int64_t>(hkv >> p.kv_shift) * p.num_slots * mi.v_row;
  const uint16_t* v_sc = p.v_scales + static_cast<int64_t>(hkv >> p.kv_shift) * p.num_slots * mi.ng;
  const float* srow = p.scores + bh * p.max_S;
  constexpr int kVW = kSelWarps / kW;   // warps of the widest block this warp plays: warp, warp + kW, ...
  for (int i = tid; i < kSelWarps * JF_HEAD_DIM; i += NT) (&sm.red[0][0])[i] = 0.f;
  if (tid < kSelWarps) sm.sum[tid] = 0.f;
  __syncthreads();
  for (int k0 = 0; k0 < p.top_k; k0 += kTailChunk) {
    const int kend = min(kTailChunk, p.top_k - k0);
    if (tid < kTailChunk) {
      int64_t slot = -1;
      float w = 0.f, vs0 = 0.f, vs1 = 0.f;
      int pos = -1, cidx = -1;
      if (tid < kend && n > 0 && src(k0 + tid, pos, cidx) && pos >= 0 && pos < n) {
        float approx = 0.f;
        uint32_t sw = 0u;
        if (cidx >= 0) {
          slot = pf.slot[cidx];
          approx = pf.score[cidx];
          sw = pf.vsc[cidx];
          if (MODE == JF_MODE_K4V4) sw = (slot & 1) ? (sw >> 16) : (sw & 0xFFFFu);  // the pair that holds the scale
        } else {
          const int64_t blk = bt[pos >> 4];
          approx = srow[pos];  // independent of the block-table lookup
          if (blk >= 0 && blk < (p.num_slots >> 4)) {
            slot = blk * 16 + (pos & 15);
            if (MODE == JF_MODE_K3V2) sw = __ldg(reinterpret_cast<const uint32_t*>(v_sc + slot * 2));
            else sw = __ldg(v_sc + slot);
          }
        }
        if (slot >= 0) {
          w = ex2((approx - M) * kLog2e);
          if (MODE == JF_MODE_K3V2) {
            vs0 = __uint_as_float(sw << 16);
            vs1 = __uint_as_float(sw & 0xFFFF0000u);
          } else {
            vs0 = vs1 = __uint_as_float(sw << 16);
          }
        }
      }
      sm.slot[tid] = slot;
      sm.cidx[tid] = cidx;
      sm.wv[tid][0] = w * vs0; sm.wv[tid][1] = w * vs1;
      // the weights' sum: whole warps are here (kTailChunk is a multiple of 32); fixed order
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xFFFFFFFFu, w, o);
      if (lane == 0) sm.sum[warp] += w;
    }
    __syncthreads();
    // packed V rows, one 16-byte load per thread
    for (int u = tid; u < kend * (VW / 4); u += NT) {
      const int c = u / (VW / 4), part = u - c * (VW / 4);
      const int64_t slot = sm.slot[c];
      const int cidx = sm.cidx[c];
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (slot >= 0) {
        if (cidx >= 0) v = reinterpret_cast<const uint4*>(pf.vrows)[cidx * (VW / 4) + part];
        else v = __ldg(reinterpret_cast<const uint4*>(v_rows + slot * (VW * 4)) + part);
      }
      reinterpret_cast<uint4*>(sm.v)[u] = v;
    }
    __syncthreads();
    // Work item (group of 16 staged entries, quarter of the channels) -> warp item & 31 of the
    // widest block; its four output tiles and the sum-of-weights tile are added to the warp's own
    // row of sm.red (no other warp touches it).
    {
      const int g = lane >> 2, tig = lane & 3;
      constexpr int kGroups = kTailChunk / 16;
      constexpr int kParts = (MODE == JF_MODE_K3V2) ? 2 : 4;          // channel ranges per group: 64 / 32 channels
      static_assert(kGroups * kParts <= 2 * kSelWarps, "work items per round");
#pragma unroll
      for (int k = 0; k < kVW * (kGroups * kParts / kSelWarps); ++k) {
        const int item = warp + k * kW;                  // 0 .. kGroups * kParts - 1
        const int grp = item % kGroups, part = item / kGroups;
        if (16 * grp >= kend) continue;                  // warp-uniform: no live entry in the group
        const int e0 = 16 * grp;
        float t[5][4];
#pragma unroll
        for (int i = 0; i < 5; ++i) t[i][0] = t[i][1] = t[i][2] = t[i][3] = 0.f;
        float* red = sm.red[item & (kSelWarps - 1)];
        if (MODE == JF_MODE_K3V2) {
          // as the scan's V path (k-slots 2tig, 2tig+1, 2tig+8, 2tig+9 <-> entries tig, tig+4, tig+8, tig+12)
          const int qh = part;
          const uint8_t* page = reinterpret_cast<const uint8_t*>(sm.v + e0 * VW) + 16 * qh + 2 * g;
          const uint32_t Ha = *reinterpret_cast<const uint16_t*>(page + tig * 32);
          const uint32_t Hb = *reinterpret_cast<const uint16_t*>(page + (tig + 4) * 32);
          const uint32_t Hc = *reinterpret_cast<const uint16_t*>(page + (tig + 8) * 32);
          const uint32_t Hd = *reinterpret_cast<const uint16_t*>(page + (tig + 12) * 32);
          uint32_t b0 = 0u, b1 = 0u;
          if (g == 0) {   // the one column of the weight operand
            b0 = pack_f16x2_sat(sm.wv[e0 + tig][qh], sm.wv[e0 + tig + 4][qh]);
            b1 = pack_f16x2_sat(sm.wv[e0 + tig + 8][qh], sm.wv[e0 + tig + 12][qh]);
          }
          const uint32_t XA = Ha | (Hb << 16), XB = Hc | (Hd << 16);
          const uint32_t XA2 = XA >> 10, XB2 = XB >> 10;
          constexpr uint32_t m0 = 0x00030003u;
          mma_f16_16816(t[0], XA & m0, XA & (m0 << 2), XB & m0, XB & (m0 << 2), b0, b1);
          mma_f16_16816(t[1], XA & (m0 << 4), XA & (m0 << 6), XB & (m0 << 4), XB & (m0 << 6), b0, b1);
          mma_f16_16816(t[2], XA & (m0 << 8), XA2 & m0, XB & (m0 << 8), XB2 & m0, b0, b1);
          mma_f16_16816(t[3], XA2 & (m0 << 2), XA2 & (m0 << 4), XB2 & (m0 << 2), XB2 & (m0 << 4), b0, b1);
          mma_f16_16816(t[4], 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, b0, b1);
          if (tig == 0) {   // column 0: rows g (fields 2ml) and g + 8 (fields 2ml + 1)
#pragma unroll
            for (int ml = 0; ml < 4; ++ml) {
              const int fa = 2 * ml, fb = 2 * ml + 1;
              // bit position of field f in its 16-bit half (after the shift by 10 for f >= 5) and its channel
              const int pa = fa <= 4 ? 2 * fa : 2 * fa - 10, pb = fb <= 4 ? 2 * fb : 2 * fb - 10;
              const int da = 64 * qh + 8 * g + 4 * (fa >> 2) + 3 - (fa & 3), db = 64 * qh + 8 * g + 4 * (fb >> 2) + 3 - (fb & 3);
              red[da] += fmaf(t[ml][0], 16777216.0f / static_cast<float>(1 << pa), -2.0f * t[4][0]);
              red[db] += fmaf(t[ml][2], 16777216.0f / static_cast<float>(1 << pb), -2.0f * t[4][2]);
            }
          }
        } else {
          // as the K4V4 scan's V path: k-slots 2tig, 2tig+1 (+8) <-> entries tokA, tokB (+8)
          const int wi = part & 1, bp = part >> 1;
          const int tokA = ((2 * tig >> 2) & 1) | (((2 * tig >> 1) & 1) << 2) | ((2 * tig & 1) << 1);
          const int tokB = (((2 * tig + 1) >> 2) & 1) | ((((2 * tig + 1) >> 1) & 1) << 2) | (((2 * tig + 1) & 1) << 1);
          const uint8_t* page = reinterpret_cast<const uint8_t*>(sm.v + e0 * VW) + 8 * g + 4 * wi;   // channels 16g + 8wi ..
          const uint32_t wa = *reinterpret_cast<const uint32_t*>(page + tokA * 64);
          const uint32_t wb = *reinterpret_cast<const uint32_t*>(page + tokB * 64);
          const uint32_t wc = *reinterpret_cast<const uint32_t*>(page + (tokA + 8) * 64);
          const uint32_t wd = *reinterpret_cast<const uint32_t*>(page + (tokB + 8) * 64);
          uint32_t b0 = 0u, b1 = 0u;
          if (g == 0) {
            b0 = pack_f16x2_sat(sm.wv[e0 + tokA][0], sm.wv[e0 + tokB][0]);
            b1 = pack_f16x2_sat(sm.wv[e0 + tokA + 8][0], sm.wv[e0 + tokB + 8][0]);
          }
          const uint32_t sel = bp ? 0x7632u : 0x5410u;
          const uint32_t XA = prmt(wa, wb, sel), XB = prmt(wc, wd, sel);
          const uint32_t XA2 = XA >> 8, XB2 = XB >> 8;
          constexpr uint32_t m0 = 0x000F000Fu;
          mma_f16_16816(t[0], XA & m0, XA & (m0 << 4), XB & m0, XB & (m0 << 4), b0, b1);
          mma_f16_16816(t[1], XA2 & m0, XA2 & (m0 << 4), XB2 & m0, XB2 & (m0 << 4), b0, b1);
          mma_f16_16816(t[4], 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, b0, b1);
          if (tig == 0) {   // low nibble -> row g (odd channel), high nibble -> row g + 8 (even channel)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int dlo = 16 * g + 8 * wi + 4 * bp + 2 * e + 1;
              red[dlo] += fmaf(t[e][0], 16777216.0f, -8.0f * t[4][0]);
              red[dlo - 1] += fmaf(t[e][2], 1048576.0f, -8.0f * t[4][2]);
            }
          }
        }
      }
    }
    __syncthreads();
  }
  __syncthreads();
  if (tid < JF_HEAD_DIM) {
    float acc_old = 0.f, ws = 0.f, o = 0.f, Z = 0.f;
#pragma unroll
    for (int w = 0; w < kSelWarps; ++w) { acc_old += sm.red[w][tid]; ws += sm.sum[w]; }
#pragma unroll
    for (int gI = 0; gI < kSplitGroups; ++gI) { o += sm.o[gI][tid]; Z += sm.z[gI]; }
    const bool live = (Z > 0.f) && (n > 0);
    const float inv_z = live ? (1.0f / Z) : 0.f;
    p.o_hat[bh * JF_HEAD_DIM + tid] = o * inv_z;
    p.o_old[bh * JF_HEAD_DIM + tid] = acc_old * inv_z;
    if (tid == 0) {
      p.W[bh] = ws * inv_z;
      if (p.softmax_m) p.softmax_m[bh] = live ? M : 0.f;
      if (p.softmax_inv_z) p.softmax_inv_z[bh] = inv_z;
    }
  }
}

// Shared by both kernels: the merged reference point M = max over the splits, block-wide.
// `red` = 32 floats of shared memory.  Ends with a barrier.  For a block of kSelThreads threads.
__device__ __forceinline__ float block_max_of_splits(const float* part_m, int64_t pbase, int hi, int splits, float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float M = kMinusBig;
  for (int s = tid; s < splits; s += kSelThreads) M = fmaxf(M, part_m[(pbase + s) * kHeadsPad + hi]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xFFFFFFFFu, M, o));
  if (lane == 0) red[warp] = M;
  __syncthreads();
#pragma unroll
  for (int w = 0; w < kSelWarps; ++w) M = fmaxf(M, red[w]);
  return M;
}

struct Workspace;
TailParams make_tail_params(const jf_decode_args* a, const Workspace& ws);
jf_status_t launch_select(const jf_decode_args* a, cudaStream_t stream, bool fused);

}  // namespace jf
