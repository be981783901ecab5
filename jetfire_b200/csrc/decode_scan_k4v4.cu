// K4V4 (INT4 K, INT4 V, group 128) flavour of the fused decode scan.
//
// Scores follow the reference's INT8 tensor-core arithmetic exactly
// (jetfire_vllm/csrc/int8tc_qk_scores.cu:272-290, 445-487): the query is quantised to INT8
// per 32-channel block with qs = max(amax/127, 1e-12) and qi = clamp(rn(q * (1/qs))); per
// block an exact int32 dot of qi with (code - 8); then s = fma(float(acc_c), qs_c, s) for
// c = 0..3, * k_scale, * attn_scale.  Integer MMA is exact, so these scores are bit-equal
// to what a CPU computes in the same order and the selection needs no re-scoring band.
// The nibbles are fed to mma.sync.m16n8k32 as *unsigned* bytes against the signed query
// (mixed u8 x s8), the "-8" being folded into the accumulator's start value
// -8 * sum(qi) per block.
//
// P.V runs in fp16 like K3V2 (the reference's INT8 quantisation of P for batch > 1,
// csrc/int8tc_softmax_v_fused.cu:1203-1311, is less accurate than its own fp32 path and is
// not reproduced; distances to both are measured in the tests).
//
// Pages are 64-byte rows; read straight, eight rows of a fragment would hit only two
// bank groups.  K and V pages are therefore fetched with tiled tensor copies
// (cp.async.bulk.tensor.2d) using the 64-byte swizzle, which XORs the 16-byte chunk index
// with bits 1..2 of the row index -- fragment loads then touch all banks once.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <unordered_map>

#include "decode_scan.cuh"

namespace jf {

namespace {

using T4 = Tile<JF_MODE_K4V4>;

// token held by MMA row r (0..7); rows r + 8 hold token + 8.  Chosen so that both the K
// fragment loads (8 rows) and the V fragment loads (4 tokens x 8 lanes) are conflict-free
// under the 64-byte swizzle.
__device__ __forceinline__ constexpr int row_token(int r) {
  return ((r >> 2) & 1) | (((r >> 1) & 1) << 2) | ((r & 1) << 1);
}

// A V nibble as an fp16 operand without any arithmetic: the masked field, read as fp16, is the
// subnormal code * 2^POS * 2^-24 (exponent bits zero), which the tensor core multiplies exactly.
// The codes' offset of 8 is not removed per element: the accumulators collect sum(P * code),
// one extra MMA per page against a row of ones collects sum(P), and the epilogue forms
// 2^(24 - POS) * acc - 8 * sum(P).  (fp32 accumulation; the accumulated terms are about three
// times larger than with the offset removed, far inside the output tolerance.)
template <int POS>
__device__ __forceinline__ uint32_t v4_field(uint32_t v) {
  constexpr uint32_t m = (15u << POS) | (15u << (POS + 16));
  return v & m;
}
constexpr uint32_t kOnesF16x2 = 0x3C003C00u;

__device__ __forceinline__ void mma_u8s8_cd(int (&d)[4], const int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%11,%12,%13};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

__device__ __forceinline__ void tma_load_2d_u32(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar,
                                                uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar), "l"(policy)
      : "memory");
}

template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds16(uint32_t addr) {
  uint32_t v;  // a 32-bit destination is zero-extended by the 16-bit load
  asm volatile("ld.shared.u16 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}

// The integer accumulators start at -8 * sum(qi) + kAccMagic (the bits of the float 1.5 * 2^23):
// the sum the MMA returns, read as a float, is then 1.5 * 2^23 + acc exactly (|acc| < 2^22: at
// most 32 * 127 * 15), and one subtraction gives float(acc) -- the same value an int-to-float
// conversion returns, on the FMA pipe instead of the conversion unit.
constexpr int kAccMagic = 0x4B400000;
__device__ __forceinline__ float acc_to_f32(int acc_biased) { return __int_as_float(acc_biased) - 12582912.0f; }

// Shared memory of a CTA: the warps' rings, their barriers (one per two-page slot), the query
// exchange buffer, the parked tile descriptors.
constexpr int kRingBytes = kScanWarps * T4::kSlots * T4::kSlotBytes;
constexpr int kBarOff = kRingBytes;
constexpr int kQxOff = kBarOff + 64;                                            // 4 warps x 2 barriers
constexpr int kBtOff = kQxOff + kScanWarps * 6 * 32 * 4;
constexpr int kSmemBytes = kBtOff + kScanWarps * 2 * kBtChunk * 16 + 1024;      // tile descriptors + alignment slack
static_assert(kScanWarps * T4::kSlots * 8 <= 64 && kRingBytes >= kMergeBytes && kBtOff % 16 == 0, "layout");

struct K4State {
  uint32_t qb[4][2];          // INT8 query fragments (B operand of the K MMA)
  float qs_h0[4], qs_h1[4];   // block scales of the heads this lane's score columns belong to
  int init[4][4];             // -8 * sum(qi) + kAccMagic per block for those heads, laid out as the MMA's C operand
  float oacc[9][4];           // output tiles 0..7; tile 8: sum of the P operand per head (see v4_field)
  float m_ref0, m_ref1, l0, l1;
  uint32_t k_off[4];          // swizzled byte offsets of this lane's K words, per 32-channel block
  uint32_t v_offA, v_offB;    // swizzled byte offsets of this lane's V words for tokens tA, tB
  uint32_t s_off;             // byte offset of this lane's scale entries
};

// One tile: two 16-token pages (the second may be absent) processed together, written out so
// that the two pages' instruction streams interleave (the asm statements keep their program
// order): all shared-memory loads first, the integer MMAs of both pages alternating, one
// softmax step over both pages' scores (one reference-point check instead of two), then the
// P.V MMAs of both pages into the same accumulator tiles.  A warp is one long dependent chain
// per page; with four warps per scheduler that chain, not the instruction count, set the pace.
//
// `sbA / sbB` = shared-memory addresses of the pages' K tiles (V tiles follow at kVOff),
// `ssA / ssB` = of their K scales (V scales follow at kVsOff).
// kMasked: `mask` holds, per page, the range [lo, hi) of its 16 tokens that belong to this tile
//   (the last page of a sequence, a page whose block id was invalid, a page cut by a boundary of
//   the reference's splits, an absent second page); tokens outside score -inf and weigh nothing.
// kInt8P: the weights follow the reference's batch > 1 Stage B for this mode
//   (jetfire_vllm/csrc/int8tc_softmax_v_fused.cu:1203-1235): per tile of 32 tokens and query
//   head, pv = p * v_scale is rounded to 127 levels of the tile's largest pv before it meets V.
//   (The reference then multiplies integers and rescales; here the rounded pv goes on as a
//   16-bit float -- the same numbers up to 2^-12 relative.)  The reference normalises p before
//   rounding and this kernel after (online softmax), which changes neither the levels nor the
//   rounding except for ties at the last float bit.
// kParts: 0 = scores and output partials; 1 = scores and softmax sums only (no V);
//   2 = output partials from scores read back from memory (no K).
template <bool kInt8P, bool kMasked, int kParts>
__device__ __forceinline__ void k4v4_tile(K4State& st, uint32_t sbA, uint32_t sbB, uint32_t ssA, uint32_t ssB,
                                          int mask, int t0, float attn, float* spA0, float* spA1, bool st0, bool st1,
                                          bool want_pm, float* pm, int lane) {
  constexpr bool kDoK = kParts != 2, kDoV = kParts != 1;
  bool aLo = true, aHi = true, bLo = true, bHi = true;   // is this lane's token of page A / B (rows g, g + 8) in the tile
  if (kMasked) {
    const int loA = mask & 31, hiA = (mask >> 5) & 31, loB = (mask >> 10) & 31, hiB = (mask >> 15) & 31;
    aLo = t0 >= loA && t0 < hiA;  aHi = t0 + 8 >= loA && t0 + 8 < hiA;
    bLo = t0 >= loB && t0 < hiB;  bHi = t0 + 8 >= loB && t0 + 8 < hiB;
  }
  float* spB0 = spA0 + 16;
  float* spB1 = spA1 + 16;
  float sA[4] = {0.f, 0.f, 0.f, 0.f}, sB[4] = {0.f, 0.f, 0.f, 0.f};
  const uint32_t saA = ssA + st.s_off, saB = ssB + st.s_off;
  if (kDoK) {
    uint32_t kwA[4][2], kwB[4][2];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t a = sbA + st.k_off[c], b = sbB + st.k_off[c];
      kwA[c][0] = lds32<0>(a); kwA[c][1] = lds32<512>(a);
      kwB[c][0] = lds32<0>(b); kwB[c][1] = lds32<512>(b);
    }
    const uint32_t ksA0 = lds16<0>(saA), ksA1 = lds16<16>(saA), ksB0 = lds16<0>(saB), ksB1 = lds16<16>(saB);
    int accA[4][4], accB[4][4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t a0 = kwA[c][0], a1 = kwA[c][1], b0 = kwB[c][0], b1 = kwB[c][1];
      mma_u8s8_cd(accA[c], st.init[c], (a0 >> 4) & 0x0F0F0F0Fu, (a1 >> 4) & 0x0F0F0F0Fu, a0 & 0x0F0F0F0Fu, a1 & 0x0F0F0F0Fu,
                  st.qb[c][0], st.qb[c][1]);
      mma_u8s8_cd(accB[c], st.init[c], (b0 >> 4) & 0x0F0F0F0Fu, (b1 >> 4) & 0x0F0F0F0Fu, b0 & 0x0F0F0F0Fu, b1 & 0x0F0F0F0Fu,
                  st.qb[c][0], st.qb[c][1]);
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      sA[0] = __fmaf_rn(acc_to_f32(accA[c][0]), st.qs_h0[c], sA[0]);
      sB[0] = __fmaf_rn(acc_to_f32(accB[c][0]), st.qs_h0[c], sB[0]);
      sA[1] = __fmaf_rn(acc_to_f32(accA[c][1]), st.qs_h1[c], sA[1]);
      sB[1] = __fmaf_rn(acc_to_f32(accB[c][1]), st.qs_h1[c], sB[1]);
      sA[2] = __fmaf_rn(acc_to_f32(accA[c][2]), st.qs_h0[c], sA[2]);
      sB[2] = __fmaf_rn(acc_to_f32(accB[c][2]), st.qs_h0[c], sB[2]);
      sA[3] = __fmaf_rn(acc_to_f32(accA[c][3]), st.qs_h1[c], sA[3]);
      sB[3] = __fmaf_rn(acc_to_f32(accB[c][3]), st.qs_h1[c], sB[3]);
    }
    const float kA0 = __uint_as_float(ksA0 << 16), kA1 = __uint_as_float(ksA1 << 16);
    const float kB0 = __uint_as_float(ksB0 << 16), kB1 = __uint_as_float(ksB1 << 16);
    sA[0] = __fmul_rn(__fmul_rn(sA[0], kA0), attn); sB[0] = __fmul_rn(__fmul_rn(sB[0], kB0), attn);
    sA[1] = __fmul_rn(__fmul_rn(sA[1], kA0), attn); sB[1] = __fmul_rn(__fmul_rn(sB[1], kB0), attn);
    sA[2] = __fmul_rn(__fmul_rn(sA[2], kA1), attn); sB[2] = __fmul_rn(__fmul_rn(sB[2], kB1), attn);
    sA[3] = __fmul_rn(__fmul_rn(sA[3], kA1), attn); sB[3] = __fmul_rn(__fmul_rn(sB[3], kB1), attn);
  } else {
    // the scores an earlier scan stored (heads past the group stay at 0: their columns are dropped)
    if (st0) {
      if (aLo) sA[0] = spA0[0];
      if (aHi) sA[2] = spA0[8];
      if (bLo) sB[0] = spB0[0];
      if (bHi) sB[2] = spB0[8];
    }
    if (st1) {
      if (aLo) sA[1] = spA1[0];
      if (aHi) sA[3] = spA1[8];
      if (bLo) sB[1] = spB1[0];
      if (bHi) sB[3] = spB1[8];
    }
  }
  // V words and scales of both pages: requested now, used after the softmax
  uint2 WaA, WbA, WcA, WdA, WaB, WbB, WcB, WdB;
  float vsA0 = 0.f, vsA1 = 0.f, vsB0 = 0.f, vsB1 = 0.f;
  if (kDoV) {
    const uint32_t vA0 = sbA + st.v_offA, vA1 = sbA + st.v_offB, vB0 = sbB + st.v_offA, vB1 = sbB + st.v_offB;
    WaA = lds64<0>(vA0); WbA = lds64<0>(vA1); WcA = lds64<512>(vA0); WdA = lds64<512>(vA1);
    WaB = lds64<0>(vB0); WbB = lds64<0>(vB1); WcB = lds64<512>(vB0); WdB = lds64<512>(vB1);
    vsA0 = __uint_as_float(lds16<T4::kVsOff>(saA) << 16); vsA1 = __uint_as_float(lds16<T4::kVsOff + 16>(saA) << 16);
    vsB0 = __uint_as_float(lds16<T4::kVsOff>(saB) << 16); vsB1 = __uint_as_float(lds16<T4::kVsOff + 16>(saB) << 16);
  }
  if (kMasked) {
    if (!aLo) { sA[0] = sA[1] = -INFINITY; vsA0 = 0.f; }
    if (!aHi) { sA[2] = sA[3] = -INFINITY; vsA1 = 0.f; }
    if (!bLo) { sB[0] = sB[1] = -INFINITY; vsB0 = 0.f; }
    if (!bHi) { sB[2] = sB[3] = -INFINITY; vsB1 = 0.f; }
  }
  if (kDoK) {
    if (kMasked) {
      if (st0 && aLo) spA0[0] = sA[0];
      if (st0 && aHi) spA0[8] = sA[2];
      if (st0 && bLo) spB0[0] = sB[0];
      if (st0 && bHi) spB0[8] = sB[2];
      if (st1 && aLo) spA1[0] = sA[1];
      if (st1 && aHi) spA1[8] = sA[3];
      if (st1 && bLo) spB1[0] = sB[1];
      if (st1 && bHi) spB1[8] = sB[3];
    } else {
      if (st0) { spA0[0] = sA[0]; spA0[8] = sA[2]; spB0[0] = sB[0]; spB0[8] = sB[2]; }
      if (st1) { spA1[0] = sA[1]; spA1[8] = sA[3]; spB1[0] = sB[1]; spB1[8] = sB[3]; }
    }
  }

  if (kDoK && want_pm) {
    // Largest score of each page per head, for the select kernel's threshold.  Four values per lane
    // (page A / B x head 2tig / 2tig+1) are reduced over the eight lanes that hold a head's tokens
    // while the lanes trade them away: lane bit 4 keeps one head, bit 3 one page, bit 2 is reduced
    // in full -- four shuffles per tile.  A page that a split boundary cuts belongs to two tiles:
    // both store +inf for it ("fetch it always"), which is exact for the select kernel's purposes.
    float a0 = fmaxf(sA[0], sA[2]), a1 = fmaxf(sA[1], sA[3]), b0 = fmaxf(sB[0], sB[2]), b1 = fmaxf(sB[1], sB[3]);
    if (kMasked) {
      if (mask & (1 << 22)) a0 = a1 = INFINITY;
      if (mask & (1 << 23)) b0 = b1 = INFINITY;
    }
    const bool hb = (lane & 16) != 0, pb = (lane & 8) != 0;
    const float ka = fmaxf(hb ? a1 : a0, __shfl_xor_sync(0xFFFFFFFFu, hb ? a0 : a1, 16));   // page A, this lane's head
    const float kb = fmaxf(hb ? b1 : b0, __shfl_xor_sync(0xFFFFFFFFu, hb ? b0 : b1, 16));   // page B
    float v = fmaxf(pb ? kb : ka, __shfl_xor_sync(0xFFFFFFFFu, pb ? ka : kb, 8));
    v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, 4));
    if (pm && (!kMasked || !pb || ((mask >> 20) & 3) == 2)) *pm = v;   // lanes with bit 2 clear of a live head; page B only if present
  }

  // ---- one online-softmax step over both pages (same arithmetic per score as softmax_step) ----
  float pA[4], pB[4];
  {
    float mx0 = fmaxf(fmaxf(sA[0], sA[2]), fmaxf(sB[0], sB[2])), mx1 = fmaxf(fmaxf(sA[1], sA[3]), fmaxf(sB[1], sB[3]));
    const bool need = (mx0 > st.m_ref0 + 4.0f) || (mx1 > st.m_ref1 + 4.0f);
    if (__any_sync(0xFFFFFFFFu, need)) {
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xFFFFFFFFu, mx0, o));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xFFFFFFFFu, mx1, o));
      }
      const float n0 = fmaxf(st.m_ref0, mx0), n1 = fmaxf(st.m_ref1, mx1);
      const float f0 = ex2((st.m_ref0 - n0) * kLog2e), f1 = ex2((st.m_ref1 - n1) * kLog2e);
      st.l0 *= f0; st.l1 *= f1;
      if (kDoV) {
#pragma unroll
        for (int i = 0; i < 9; ++i) { st.oacc[i][0] *= f0; st.oacc[i][1] *= f1; st.oacc[i][2] *= f0; st.oacc[i][3] *= f1; }
      }
      st.m_ref0 = n0; st.m_ref1 = n1;
    }
    const float mb0 = st.m_ref0 * kLog2e, mb1 = st.m_ref1 * kLog2e;
    pA[0] = ex2(fmaf(sA[0], kLog2e, -mb0)); pB[0] = ex2(fmaf(sB[0], kLog2e, -mb0));
    pA[1] = ex2(fmaf(sA[1], kLog2e, -mb1)); pB[1] = ex2(fmaf(sB[1], kLog2e, -mb1));
    pA[2] = ex2(fmaf(sA[2], kLog2e, -mb0)); pB[2] = ex2(fmaf(sB[2], kLog2e, -mb0));
    pA[3] = ex2(fmaf(sA[3], kLog2e, -mb1)); pB[3] = ex2(fmaf(sB[3], kLog2e, -mb1));
    st.l0 += (pA[0] + pA[2]) + (pB[0] + pB[2]);
    st.l1 += (pA[1] + pA[3]) + (pB[1] + pB[3]);
  }
  if (!kDoV) return;

  // ---- (P * vscale).V for both pages ----
  float wA[4] = {pA[0] * vsA0, pA[1] * vsA0, pA[2] * vsA1, pA[3] * vsA1};
  float wB[4] = {pB[0] * vsB0, pB[1] * vsB0, pB[2] * vsB1, pB[3] * vsB1};
  if (kInt8P) {
    // largest pv of the tile per query head: this lane's four tokens, then the eight lanes that
    // hold the other tokens of the same head pair
    float a0 = fmaxf(fmaxf(wA[0], wA[2]), fmaxf(wB[0], wB[2])), a1 = fmaxf(fmaxf(wA[1], wA[3]), fmaxf(wB[1], wB[3]));
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      a0 = fmaxf(a0, __shfl_xor_sync(0xFFFFFFFFu, a0, o));
      a1 = fmaxf(a1, __shfl_xor_sync(0xFFFFFFFFu, a1, o));
    }
    const float sc0 = a0 * (1.0f / 127.0f), sc1 = a1 * (1.0f / 127.0f);
    const float in0 = sc0 > 0.f ? __frcp_rn(sc0) : 0.f, in1 = sc1 > 0.f ? __frcp_rn(sc1) : 0.f;
    // round to nearest (ties to even) by adding and removing 1.5 * 2^23: 0 <= pv / scale <= 127
    constexpr float kRnd = 12582912.0f;
    wA[0] = (fmaf(wA[0], in0, kRnd) - kRnd) * sc0; wA[1] = (fmaf(wA[1], in1, kRnd) - kRnd) * sc1;
    wA[2] = (fmaf(wA[2], in0, kRnd) - kRnd) * sc0; wA[3] = (fmaf(wA[3], in1, kRnd) - kRnd) * sc1;
    wB[0] = (fmaf(wB[0], in0, kRnd) - kRnd) * sc0; wB[1] = (fmaf(wB[1], in1, kRnd) - kRnd) * sc1;
    wB[2] = (fmaf(wB[2], in0, kRnd) - kRnd) * sc0; wB[3] = (fmaf(wB[3], in1, kRnd) - kRnd) * sc1;
  }
  const uint32_t A0 = movmatrix_trans(pack_f16x2_sat(wA[0], wA[1]));
  const uint32_t B0 = movmatrix_trans(pack_f16x2_sat(wB[0], wB[1]));
  const uint32_t A1 = movmatrix_trans(pack_f16x2_sat(wA[2], wA[3]));
  const uint32_t B1 = movmatrix_trans(pack_f16x2_sat(wB[2], wB[3]));
  const uint32_t waA[2] = {WaA.x, WaA.y}, wbA[2] = {WbA.x, WbA.y}, wcA[2] = {WcA.x, WcA.y}, wdA[2] = {WdA.x, WdA.y};
  const uint32_t waB[2] = {WaB.x, WaB.y}, wbB[2] = {WbB.x, WbB.y}, wcB[2] = {WcB.x, WcB.y}, wdB[2] = {WdB.x, WdB.y};
#pragma unroll
  for (int wi = 0; wi < 2; ++wi) {
#pragma unroll
    for (int bp = 0; bp < 2; ++bp) {
      const uint32_t sel = bp ? 0x7632u : 0x5410u;
      const uint32_t XA = prmt(waA[wi], wbA[wi], sel), XB = prmt(wcA[wi], wdA[wi], sel);
      const uint32_t YA = prmt(waB[wi], wbB[wi], sel), YB = prmt(wcB[wi], wdB[wi], sel);
      const uint32_t XA2 = XA >> 8, XB2 = XB >> 8, YA2 = YA >> 8, YB2 = YB >> 8;
      const int mt = 4 * wi + 2 * bp;
      // low nibble -> output row g, high nibble -> output row g + 8
      mma_f16_16816(st.oacc[mt], v4_field<0>(XA), v4_field<4>(XA), v4_field<0>(XB), v4_field<4>(XB), A0, A1);
      mma_f16_16816(st.oacc[mt + 1], v4_field<0>(XA2), v4_field<4>(XA2), v4_field<0>(XB2), v4_field<4>(XB2), A0, A1);
      mma_f16_16816(st.oacc[mt], v4_field<0>(YA), v4_field<4>(YA), v4_field<0>(YB), v4_field<4>(YB), B0, B1);
      mma_f16_16816(st.oacc[mt + 1], v4_field<0>(YA2), v4_field<4>(YA2), v4_field<0>(YB2), v4_field<4>(YB2), B0, B1);
    }
  }
  mma_f16_16816(st.oacc[8], kOnesF16x2, kOnesF16x2, kOnesF16x2, kOnesF16x2, A0, A1);
  mma_f16_16816(st.oacc[8], kOnesF16x2, kOnesF16x2, kOnesF16x2, kOnesF16x2, B0, B1);
}

constexpr int kFullTile = (16 << 5) | (16 << 15) | (2 << 20);   // both pages whole

}  // namespace

// Work is cut into tiles of two pages.  kInt8P = false: tile T is pages 2T, 2T + 1 of the
// sequence.  kInt8P = true: tiles are the reference's -- positions are cut into 8 splits of
// ceil(max_S / 8), and inside a split the 32-token tiles start at the split's first 16-token
// block (jetfire_vllm/csrc/int8tc_softmax_v_fused.cu:62, 1049-1053); a block that a split boundary
// cuts belongs to two tiles, each with its own tokens.  p.tile_base[s] = first tile of split s.
// A CTA takes a contiguous range of tiles, each of its warps a contiguous quarter of it.
template <bool kInt8P, int kParts>
__global__ void __launch_bounds__(kScanWarps * 32, 4)
scan_k4v4_kernel(const ScanParams p, const __grid_constant__ CUtensorMap k_map,
                 const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap k_map2,
                 const __grid_constant__ CUtensorMap v_map2) {
  constexpr bool kDoK = kParts != 2, kDoV = kParts != 1;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // swizzled tiles must sit on 512-byte boundaries: align by hand (1 KB of slack is allocated)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;  // uniform by construction
  const int g = lane >> 2, tig = lane & 3;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;

  const uint32_t smem_base = smem_u32(smem);
  const uint32_t slots0 = smem_base + warp * (T4::kSlots * T4::kSlotBytes);
  const uint32_t bars0 = smem_base + kBarOff + warp * (T4::kSlots * 8);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kBarOff) + warp * T4::kSlots;

  if (lane == 0) {
    for (int s = 0; s < T4::kSlots; ++s) mbar_init(&bars[s], 1);
    // the tensor maps are kernel parameters, not results of the previous kernel: fetch them now
    if (kDoK) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&k_map2)) : "memory");
    if (kDoV) asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&v_map2)) : "memory");
  }
  fence_barrier_init();
  __syncwarp();
  pdl_wait();  // nothing above reads global memory

  // The first loads (sequence length, the block-table entries of the first tiles, the query) do
  // not depend on one another: all are issued here, so the prologue pays one memory latency before
  // the first copies can start, and the query arithmetic then runs while those copies are in flight.
  const int t_first = split * p.tiles_per_split + warp * p.tiles_per_warp;          // this warp's tiles
  const int t_end = min(min(t_first + p.tiles_per_warp, (split + 1) * p.tiles_per_split), p.n_tiles);
  const int64_t* bt_row = p.block_table + static_cast<int64_t>(b) * p.max_blocks;
  const int len = min(p.seq_lens[b], p.max_S);
  const int64_t n_blocks_phys = p.num_slots >> 4;
  const int head_row0 = static_cast<int>(static_cast<int64_t>(hkv >> p.kv_shift) * p.num_slots);  // first cache row of this KV head

  // Tile T of the warp (tile t_first + T of the row): its first page and the token ranges of its
  // pages, packed as lo_A | hi_A << 5 | lo_B << 10 | hi_B << 15 | pages << 20 | cut flags << 22; 0 = no such tile
  // (past the warp's range or past the sequence; such tiles are a suffix of the range).
  auto tile_geom = [&](int T, int& pageA) -> int {
    const int gT = t_first + T;
    pageA = 0;
    if (gT >= t_end) return 0;
    int s_lo = 0, s_hi = len;
    pageA = 2 * gT;
    if (kInt8P) {
      int s = 0, base = 0;
#pragma unroll
      for (int i = 1; i < 8; ++i)
        if (gT >= p.tile_base[i]) { s = i; base = p.tile_base[i]; }
      s_lo = s * p.ref_chunk;
      s_hi = min(s_lo + p.ref_chunk, len);
      pageA = (s_lo >> 4) + 2 * (gT - base);
    }
    const int blk_end = (s_hi + 15) >> 4;
    if (s_lo >= s_hi || pageA >= blk_end) return 0;
    const int pa = pageA * 16;
    const int two = (pageA + 1 < blk_end) ? 1 : 0;
    const int loA = max(s_lo - pa, 0), hiA = min(s_hi - pa, 16);
    const int hiB = two ? min(s_hi - pa - 16, 16) : 0;
    // bits 22 / 23: page A / B is cut by a split boundary (another tile holds its other tokens)
    const int cutA = (loA > 0 || (hiA < 16 && pa + hiA < len)) ? 1 : 0;
    const int cutB = (two && hiB < 16 && pa + 16 + hiB < len) ? 1 : 0;
    return loA | (hiA << 5) | (hiB << 15) | ((1 + two) << 20) | (cutA << 22) | (cutB << 23);
  };
  // Descriptors are worked out sixteen tiles at a time by sixteen lanes, a whole chunk ahead of
  // their use (a global load issued while megabytes of page copies are queued in the memory
  // system takes several microseconds; fetched a tile or two ahead, those loads stalled the
  // loop), and parked in shared memory: x / y = first cache row of page A / B, z = the token
  // ranges, w = page A's index in the sequence.
  int4* desc_s = reinterpret_cast<int4*>(smem + kBtOff) + warp * (2 * kBtChunk);
  struct Pending { int64_t ba, bb; int pageA, mask; };
  auto desc_load = [&](int chunk) -> Pending {
    Pending r{-1, -1, 0, 0};
    if (lane < kBtChunk) {
      r.mask = tile_geom(chunk * kBtChunk + lane, r.pageA);
      if (r.mask) {
        if (r.pageA < p.max_blocks) r.ba = bt_row[r.pageA];
        if (((r.mask >> 20) & 3) == 2 && r.pageA + 1 < p.max_blocks) r.bb = bt_row[r.pageA + 1];
      }
    }
    return r;
  };
  // an invalid block id reads block 0 and counts no live token
  auto desc_make = [&](const Pending& r) -> int4 {
    int mask = r.mask;
    const bool badA = r.ba < 0 || r.ba >= n_blocks_phys, badB = r.bb < 0 || r.bb >= n_blocks_phys;
    if (badA) mask &= ~0x3FF;
    if (badB) mask &= ~(0x3FF << 10);
    const int rowA = head_row0 + static_cast<int>(badA ? 0 : r.ba) * 16;
    const int rowB = ((mask >> 20) & 3) == 2 ? head_row0 + static_cast<int>(badB ? 0 : r.bb) * 16 : -1;
    return make_int4(rowA, rowB, mask, r.pageA);
  };
  Pending pend = desc_load(0);
  // warp w prepares the query's 32-channel block w for the whole CTA (see below)
  uint4 q_raw = make_uint4(0u, 0u, 0u, 0u);
  if (kDoK && g < p.G) {   // the 8 channels 32 w + 8 tig + {0..7} are 16 contiguous bytes
    const int64_t qbase = (static_cast<int64_t>(b) * p.H_q + hkv * p.G + g) * JF_HEAD_DIM;
    q_raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + qbase + 32 * warp + 8 * tig));
  }

  // One elected lane issues a tile's copies: per page a tensor copy for K and one for V and two
  // scale copies; two pages whose blocks are neighbours in the cache take one 32-row tensor copy
  // per tensor and one 64-byte copy per scale array.  Everything lands on the slot's barrier.
  // The packed cache is read once per call: fetched as first-to-evict, it leaves the scores
  // this kernel writes (and the next kernel reads) in L2.
  const uint64_t stream_policy = l2_policy_evict_first();
  constexpr uint32_t kTxPage = (kDoK ? 1056u : 0u) + (kDoV ? 1056u : 0u);
  auto refill = [&](int sl, int4 d) {
    if (elect_one()) {
      const uint32_t bar = bars0 + sl * 8;
      const uint32_t dst = slots0 + sl * T4::kSlotBytes;
      const int ra = d.x, rb = d.y;
      const bool two = rb >= 0;
      if (two && rb == ra + 16) {
        mbar_expect_tx_u32(bar, 2 * kTxPage);
        if (kDoK) {
          tma_load_2d_u32(dst, &k_map2, 0, ra, bar, stream_policy);
          bulk_g2s_u32(dst + T4::kScaleOff, p.k_scales + ra, 64, bar);
        }
        if (kDoV) {
          tma_load_2d_u32(dst + T4::kVOff, &v_map2, 0, ra, bar, stream_policy);
          bulk_g2s_u32(dst + T4::kScaleOff + T4::kVsOff, p.v_scales + ra, 64, bar);
        }
      } else {
        mbar_expect_tx_u32(bar, two ? 2 * kTxPage : kTxPage);
        if (kDoK) {
          tma_load_2d_u32(dst, &k_map, 0, ra, bar, stream_policy);
          bulk_g2s_u32(dst + T4::kScaleOff, p.k_scales + ra, 32, bar);
        }
        if (kDoV) {
          tma_load_2d_u32(dst + T4::kVOff, &v_map, 0, ra, bar, stream_policy);
          bulk_g2s_u32(dst + T4::kScaleOff + T4::kVsOff, p.v_scales + ra, 32, bar);
        }
        if (two) {
          if (kDoK) {
            tma_load_2d_u32(dst + T4::kPageBytes, &k_map, 0, rb, bar, stream_policy);
            bulk_g2s_u32(dst + T4::kScaleOff + 32, p.k_scales + rb, 32, bar);
          }
          if (kDoV) {
            tma_load_2d_u32(dst + T4::kPageBytes + T4::kVOff, &v_map, 0, rb, bar, stream_policy);
            bulk_g2s_u32(dst + T4::kScaleOff + T4::kVsOff + 32, p.v_scales + rb, 32, bar);
          }
        }
      }
    }
  };

  // chunk 0 to shared memory, chunk 1 requested, the ring filled
  if (lane < kBtChunk) desc_s[lane] = desc_make(pend);
  int stored = 0;   // chunks 0..stored are in shared memory; chunk stored + 1 is in `pend`
  pend = desc_load(1);
  __syncwarp();
  {
#pragma unroll
    for (int sl = 0; sl < T4::kSlots; ++sl) {
      const int4 d = desc_s[sl];
      if (d.z) refill(sl, d);
    }
  }

  // ---- query: INT8 per 32-channel block.  Lane (head n = g, tig) owns channels
  //      32c + 8 tig + {0..7}; even channels meet the high nibbles, odd the low ones.
  //      The four warps need identical fragments: warp w quantises block c = w and the CTA
  //      exchanges the results through shared memory (a quarter of the arithmetic per warp). ----
  K4State st;
  if (kDoK) {
    static_assert(kScanWarps == 4, "one warp per 32-channel query block");
    uint32_t* qx = reinterpret_cast<uint32_t*>(smem + kQxOff);  // [c][6][32]
    {
      float v[8];
      float amax = 0.f;
      const uint32_t rw[4] = {q_raw.x, q_raw.y, q_raw.z, q_raw.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint16_t bits = static_cast<uint16_t>((j & 1) ? (rw[j >> 1] >> 16) : (rw[j >> 1] & 0xFFFFu));
        v[j] = p.q_dtype == JF_DTYPE_FP16 ? Elem<JF_DTYPE_FP16>::to_f32(bits) : Elem<JF_DTYPE_BF16>::to_f32(bits);
        amax = fmaxf(amax, fabsf(v[j]));
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
      const float qs = fmaxf(__fdiv_rn(amax, 127.0f), 1e-12f);
      const float inv = __fdiv_rn(1.0f, qs);
      int qi[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        qi[j] = max(-128, min(127, __float2int_rn(__fmul_rn(v[j], inv))));
        sum += qi[j];
      }
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 1);
      sum += __shfl_xor_sync(0xFFFFFFFFu, sum, 2);
      uint32_t* mine = qx + warp * (6 * 32) + lane;
      mine[0] = (qi[0] & 255) | ((qi[2] & 255) << 8) | ((qi[4] & 255) << 16) | ((qi[6] & 255) << 24);
      mine[32] = (qi[1] & 255) | ((qi[3] & 255) << 8) | ((qi[5] & 255) << 16) | ((qi[7] & 255) << 24);
      mine[64] = __float_as_uint(__shfl_sync(0xFFFFFFFFu, qs, 8 * tig));
      mine[96] = __float_as_uint(__shfl_sync(0xFFFFFFFFu, qs, 8 * tig + 4));
      mine[128] = static_cast<uint32_t>(-8 * __shfl_sync(0xFFFFFFFFu, sum, 8 * tig));
      mine[160] = static_cast<uint32_t>(-8 * __shfl_sync(0xFFFFFFFFu, sum, 8 * tig + 4));
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t* src = qx + c * (6 * 32) + lane;
      st.qb[c][0] = src[0];
      st.qb[c][1] = src[32];
      st.qs_h0[c] = __uint_as_float(src[64]);
      st.qs_h1[c] = __uint_as_float(src[96]);
      st.init[c][0] = st.init[c][2] = static_cast<int>(src[128]) + kAccMagic;
      st.init[c][1] = st.init[c][3] = static_cast<int>(src[160]) + kAccMagic;
    }
  }
#pragma unroll
  for (int i = 0; i < 9; ++i) { st.oacc[i][0] = st.oacc[i][1] = st.oacc[i][2] = st.oacc[i][3] = 0.f; }
  st.m_ref0 = kMinusBig; st.m_ref1 = kMinusBig; st.l0 = 0.f; st.l1 = 0.f;
  bool failed = false;

  const int t0 = row_token(g);                 // token of MMA row g (row g + 8 -> t0 + 8)
  {
    const int ksw = (t0 >> 1) & 3;             // swizzle term of rows t0 and t0 + 8
    const int tA = row_token(2 * tig), tB = row_token(2 * tig + 1);  // tokens of P.V k-slots
    const int vchunk = g >> 1, vsub = 8 * (g & 1);
#pragma unroll
    for (int c = 0; c < 4; ++c) st.k_off[c] = t0 * 64 + 4 * tig + ((c ^ ksw) << 4);
    st.v_offA = T4::kVOff + tA * 64 + ((vchunk ^ ((tA >> 1) & 3)) << 4) + vsub;
    st.v_offB = T4::kVOff + tB * 64 + ((vchunk ^ ((tB >> 1) & 3)) << 4) + vsub;
    st.s_off = t0 * 2;
  }
  const int h0 = hkv * p.G + 2 * tig;
  float* sp0 = p.scores + (static_cast<int64_t>(b) * p.H_q + h0) * p.max_S + t0;
  float* sp1 = sp0 + p.max_S;
  const bool st0 = (2 * tig) < p.G, st1 = (2 * tig + 1) < p.G;
  const float attn = p.attn_scale;
  // page maxima: after the tile's exchange the lanes with bit 2 clear hold them -- bit 4: head
  // 2tig / 2tig+1, bit 3: page A / B
  const int pm_head = 2 * tig + (lane >> 4);
  const bool want_pm = kDoK && p.pmax != nullptr;   // the same for the whole grid
  float* pm_row = (want_pm && (lane & 4) == 0 && pm_head < p.G)
                      ? p.pmax + (static_cast<int64_t>(b) * p.H_q + hkv * p.G + pm_head) * p.np_stride + ((lane >> 3) & 1)
                      : nullptr;

  // A round takes one slot: one tile.  Tiles of two whole pages go through the unmasked path.
  int sl = 0;
  uint32_t parity = 0u;
  for (int it = 0; it < p.tiles_per_warp; ++it) {
    // the tile's parked descriptor is still resident: a chunk is overwritten 16 tiles after its
    // last entry was issued
    const int4 d = desc_s[it & (2 * kBtChunk - 1)];
    if (d.z == 0) break;
    if (!mbar_wait(&bars[sl], parity)) {
      if (desc_s[(it + 1) & (2 * kBtChunk - 1)].z) mbar_wait(&bars[sl ^ 1], parity ^ static_cast<uint32_t>(sl), 1000000ull);
      failed = true;
      break;
    }
    const uint32_t sb = slots0 + sl * T4::kSlotBytes, ss = sb + T4::kScaleOff;
    float* spA0 = sp0 + static_cast<int64_t>(d.w) * 16;
    float* spA1 = sp1 + static_cast<int64_t>(d.w) * 16;
    if (d.z == kFullTile)
      k4v4_tile<kInt8P, false, kParts>(st, sb, sb + T4::kPageBytes, ss, ss + 32, d.z, t0, attn, spA0, spA1, st0, st1,
                                       want_pm, pm_row ? pm_row + d.w : nullptr, lane);
    else
      k4v4_tile<kInt8P, true, kParts>(st, sb, sb + T4::kPageBytes, ss, ss + 32, d.z, t0, attn, spA0, spA1, st0, st1,
                                      want_pm, pm_row ? pm_row + d.w : nullptr, lane);
    __syncwarp();
    // the refill below reads the descriptor of tile it + kSlots: bring its chunk in first
    if (((it + T4::kSlots) >> 4) > stored) {
      ++stored;
      if (lane < kBtChunk) desc_s[(stored & 1) * kBtChunk + lane] = desc_make(pend);
      pend = desc_load(stored + 1);
      __syncwarp();
    }
    const int4 dn = desc_s[(it + T4::kSlots) & (2 * kBtChunk - 1)];
    if (it + T4::kSlots < p.tiles_per_warp && dn.z) refill(sl, dn);
    sl ^= 1;
    if (sl == 0) parity ^= 1u;
  }

  pdl_trigger();  // the next kernel may start its prologue; it waits for this grid before reading
  if (failed && lane == 0) report_status(p.status, JF_ERR_TIMEOUT);
  if (kDoK && threadIdx.x == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) p.status[4] = want_pm ? kPageMaxTag : 0;

  __syncthreads();
  {
    float* wo = reinterpret_cast<float*>(smem) + warp * (kHeadsPad * JF_HEAD_DIM);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const int wi = mt >> 2, bp = (mt >> 1) & 1, e = mt & 1;
      const int dlo = 16 * g + 8 * wi + 4 * bp + 2 * e + 1;  // low nibble of the byte: odd channel
      const int dhi = dlo - 1;                               // high nibble: even channel
      // 2^(24 - POS) * sum(P * field) - 8 * sum(P): the codes' offset leaves here (see v4_field)
      wo[(2 * tig) * JF_HEAD_DIM + dlo] = fmaf(st.oacc[mt][0], 16777216.0f, -8.0f * st.oacc[8][0]);
      wo[(2 * tig + 1) * JF_HEAD_DIM + dlo] = fmaf(st.oacc[mt][1], 16777216.0f, -8.0f * st.oacc[8][1]);
      wo[(2 * tig) * JF_HEAD_DIM + dhi] = fmaf(st.oacc[mt][2], 1048576.0f, -8.0f * st.oacc[8][2]);
      wo[(2 * tig + 1) * JF_HEAD_DIM + dhi] = fmaf(st.oacc[mt][3], 1048576.0f, -8.0f * st.oacc[8][3]);
    }
  }
  cta_merge_store(p, smem, st.l0, st.l1, st.m_ref0, st.m_ref1, 0.f, 0.f, split, hkv, b);
}

// ---- tensor maps -----------------------------------------------------------------------
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qr) != cudaSuccess ||
        qr != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeFn>(sym);
  }();
  return fn;
}

struct MapKey {
  const void* base;
  uint64_t rows;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (std::hash<uint64_t>()(k.rows * 64 + k.box_rows) * 1000003u);
  }
};

// (rows x 64 bytes) view of a packed tensor, box = one 16-row page or two (32 rows), 64-byte swizzle.
jf_status_t page_map(const void* base, uint64_t rows, uint32_t box_rows, CUtensorMap* out) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  std::lock_guard<std::mutex> lock(mu);
  const MapKey key{base, rows, box_rows};
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return JF_OK; }
  EncodeFn fn = encode_fn();
  if (!fn) return JF_ERR_CUDA;
  const cuuint64_t dims[2] = {64, rows};
  const cuuint64_t strides[1] = {64};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMap m;
  const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { g_last_cuda_error = static_cast<int32_t>(r); return JF_ERR_CUDA; }
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return JF_OK;
}

}  // namespace

template <bool kInt8P, int kParts>
jf_status_t launch_variant(const ScanParams& sp, dim3 grid, cudaStream_t stream, const CUtensorMap& k_map,
                           const CUtensorMap& v_map, const CUtensorMap& k_map2, const CUtensorMap& v_map2) {
  const size_t smem = kSmemBytes;
  JF_ENSURE_SMEM((scan_k4v4_kernel<kInt8P, kParts>), smem);
  JF_CUDA_TRY(launch_pdl(scan_k4v4_kernel<kInt8P, kParts>, grid, dim3(kScanWarps * 32), smem, stream, sp, k_map, v_map,
                         k_map2, v_map2));
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

// `sp` arrives with everything but the tile geometry filled in.
jf_status_t launch_scan_k4v4(ScanParams sp, bool int8p, int parts, dim3 grid, cudaStream_t stream) {
  const uint64_t rows = static_cast<uint64_t>(sp.H_kv >> sp.kv_shift) * static_cast<uint64_t>(sp.num_slots);
  if (rows > 0x7FFFFFFFull) return JF_ERR_UNSUPPORTED;
  // tiles of the longest row this call can see (the kernel drops those past a row's own length)
  if (int8p && parts != 1) {
    sp.ref_chunk = (sp.max_S + 7) / 8;
    int n = 0;
    for (int s = 0; s < 8; ++s) {
      sp.tile_base[s] = n;
      const int lo = s * sp.ref_chunk, hi = std::min(lo + sp.ref_chunk, sp.max_S);
      if (lo < hi) n += ((hi + 15) / 16 - lo / 16 + 1) / 2;
    }
    sp.tile_base[8] = n;
    sp.n_tiles = n;
  } else {
    int8p = false;   // the tiling only matters where weights meet V
    sp.ref_chunk = sp.max_S;
    sp.n_tiles = ((sp.max_S + 15) / 16 + 1) / 2;
    for (int s = 0; s <= 8; ++s) sp.tile_base[s] = s ? sp.n_tiles : 0;
  }
  sp.tiles_per_split = (sp.n_tiles + sp.splits - 1) / sp.splits;
  sp.tiles_per_warp = (sp.tiles_per_split + kScanWarps - 1) / kScanWarps;
  // a tensor map of a tensor the call does not read is never used by the kernel; the other one stands in
  const void* k_base = sp.k_data ? static_cast<const void*>(sp.k_data) : static_cast<const void*>(sp.v_data);
  const void* v_base = sp.v_data ? static_cast<const void*>(sp.v_data) : static_cast<const void*>(sp.k_data);
  CUtensorMap k_map, v_map, k_map2, v_map2;
  jf_status_t st = page_map(k_base, rows, 16, &k_map);
  if (st == JF_OK) st = page_map(v_base, rows, 16, &v_map);
  if (st == JF_OK) st = page_map(k_base, rows, 32, &k_map2);
  if (st == JF_OK) st = page_map(v_base, rows, 32, &v_map2);
  if (st != JF_OK) return st;
  if (parts == 1) return launch_variant<false, 1>(sp, grid, stream, k_map, v_map, k_map2, v_map2);
  if (parts == 2) {
    return int8p ? launch_variant<true, 2>(sp, grid, stream, k_map, v_map, k_map2, v_map2)
                 : launch_variant<false, 2>(sp, grid, stream, k_map, v_map, k_map2, v_map2);
  }
  return int8p ? launch_variant<true, 0>(sp, grid, stream, k_map, v_map, k_map2, v_map2)
               : launch_variant<false, 0>(sp, grid, stream, k_map, v_map, k_map2, v_map2);
}

}  // namespace jf
