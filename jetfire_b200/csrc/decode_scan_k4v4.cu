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
// exchange buffer, the parked block-table entries.
constexpr int kPagesInFlight = 2 * T4::kSlots;                                  // per warp
constexpr int kRingBytes = kScanWarps * T4::kSlots * T4::kSlotBytes;
constexpr int kBarOff = kRingBytes;
constexpr int kQxOff = kBarOff + 64;                                            // 4 warps x 2 barriers
constexpr int kBtOff = kQxOff + kScanWarps * 6 * 32 * 4;
constexpr int kSmemBytes = kBtOff + kScanWarps * 2 * kBtChunk * 8 + 1024;       // + alignment slack
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

// One 16-token page; kPartial as in the K3V2 kernel.
// `sb` = shared-memory address of the page's K tile (its V tile follows at kVOff), `ss` = of its
// K scales (its V scales follow at kVsOff).
template <bool kPartial>
__device__ __forceinline__ void k4v4_page(K4State& st, uint32_t sb, uint32_t ss, int t0, int valid, float attn,
                                          float* sp0, float* sp1, bool st0, bool st1) {
  // ---------------- K: nibbles -> u8 fragments, exact integer Q.K^T per block ----------------
  // all shared-memory reads of the page are issued up front
  uint32_t kw[4][2];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t a = sb + st.k_off[c];
    kw[c][0] = lds32<0>(a); kw[c][1] = lds32<512>(a);
  }
  const uint32_t sa = ss + st.s_off;
  const uint32_t ksb0 = lds16<0>(sa), ksb1 = lds16<16>(sa), vsb0 = lds16<T4::kVsOff>(sa), vsb1 = lds16<T4::kVsOff + 16>(sa);
  const uint32_t aA = sb + st.v_offA, aB = sb + st.v_offB;
  const uint2 Wa = lds64<0>(aA), Wb = lds64<0>(aB), Wc = lds64<512>(aA), Wd = lds64<512>(aB);
  int acc[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t w0 = kw[c][0], w1 = kw[c][1];
    mma_u8s8_cd(acc[c], st.init[c], (w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu, w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu,
                st.qb[c][0], st.qb[c][1]);
  }
  const float ks0 = __uint_as_float(ksb0 << 16), ks1 = __uint_as_float(ksb1 << 16);
  float vs0 = __uint_as_float(vsb0 << 16), vs1 = __uint_as_float(vsb1 << 16);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    s0 = __fmaf_rn(acc_to_f32(acc[c][0]), st.qs_h0[c], s0);
    s1 = __fmaf_rn(acc_to_f32(acc[c][1]), st.qs_h1[c], s1);
    s2 = __fmaf_rn(acc_to_f32(acc[c][2]), st.qs_h0[c], s2);
    s3 = __fmaf_rn(acc_to_f32(acc[c][3]), st.qs_h1[c], s3);
  }
  s0 = __fmul_rn(__fmul_rn(s0, ks0), attn);
  s1 = __fmul_rn(__fmul_rn(s1, ks0), attn);
  s2 = __fmul_rn(__fmul_rn(s2, ks1), attn);
  s3 = __fmul_rn(__fmul_rn(s3, ks1), attn);
  if (kPartial) {
    const bool lo = t0 < valid, hi = t0 + 8 < valid;
    if (!lo) { s0 = s1 = -INFINITY; vs0 = 0.f; }
    if (!hi) { s2 = s3 = -INFINITY; vs1 = 0.f; }
    if (st0 && lo) sp0[0] = s0;
    if (st0 && hi) sp0[8] = s2;
    if (st1 && lo) sp1[0] = s1;
    if (st1 && hi) sp1[8] = s3;
  } else {
    if (st0) { sp0[0] = s0; sp0[8] = s2; }
    if (st1) { sp1[0] = s1; sp1[8] = s3; }
  }

  // ---------------- online softmax ----------------
  float p0, p1, p2, p3;
  softmax_step(s0, s1, s2, s3, st.m_ref0, st.m_ref1, st.l0, st.l1, st.oacc, p0, p1, p2, p3);

  // ---------------- V: nibbles -> fp16 fragments, (P * vscale).V ----------------
  const uint32_t B0 = movmatrix_trans(pack_f16x2_sat(p0 * vs0, p1 * vs0));  // tokens tA, tB
  const uint32_t B1 = movmatrix_trans(pack_f16x2_sat(p2 * vs1, p3 * vs1));  // tokens tA+8, tB+8
  const uint32_t wa[2] = {Wa.x, Wa.y}, wb[2] = {Wb.x, Wb.y}, wc[2] = {Wc.x, Wc.y}, wd[2] = {Wd.x, Wd.y};
#pragma unroll
  for (int wi = 0; wi < 2; ++wi) {
#pragma unroll
    for (int bp = 0; bp < 2; ++bp) {
      const uint32_t sel = bp ? 0x7632u : 0x5410u;
      const uint32_t XA = prmt(wa[wi], wb[wi], sel), XB = prmt(wc[wi], wd[wi], sel);
      const uint32_t XA2 = XA >> 8, XB2 = XB >> 8;
      const int mt = 4 * wi + 2 * bp;
      // low nibble -> output row g, high nibble -> output row g + 8
      mma_f16_16816(st.oacc[mt], v4_field<0>(XA), v4_field<4>(XA), v4_field<0>(XB), v4_field<4>(XB), B0, B1);
      mma_f16_16816(st.oacc[mt + 1], v4_field<0>(XA2), v4_field<4>(XA2), v4_field<0>(XB2), v4_field<4>(XB2), B0, B1);
    }
  }
  mma_f16_16816(st.oacc[8], kOnesF16x2, kOnesF16x2, kOnesF16x2, kOnesF16x2, B0, B1);
}

// Two full 16-token pages at once, written out so that the two pages' instruction streams
// interleave (the asm statements keep their program order): all shared-memory loads first,
// the integer MMAs of both pages alternating, one softmax step over both pages' scores (one
// reference-point check instead of two), then the P.V MMAs of both pages into the same
// accumulator tiles.  A warp is one long dependent chain per page; with four warps per
// scheduler that chain, not the instruction count, set the pace.
__device__ __forceinline__ void k4v4_page_pair(K4State& st, uint32_t sbA, uint32_t sbB, uint32_t ssA, uint32_t ssB,
                                               float attn, float* spA0, float* spA1, float* spB0, float* spB1,
                                               bool st0, bool st1) {
  uint32_t kwA[4][2], kwB[4][2];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t a = sbA + st.k_off[c], b = sbB + st.k_off[c];
    kwA[c][0] = lds32<0>(a); kwA[c][1] = lds32<512>(a);
    kwB[c][0] = lds32<0>(b); kwB[c][1] = lds32<512>(b);
  }
  const uint32_t saA = ssA + st.s_off, saB = ssB + st.s_off;
  const uint32_t ksA0 = lds16<0>(saA), ksA1 = lds16<16>(saA), vsA0b = lds16<T4::kVsOff>(saA), vsA1b = lds16<T4::kVsOff + 16>(saA);
  const uint32_t ksB0 = lds16<0>(saB), ksB1 = lds16<16>(saB), vsB0b = lds16<T4::kVsOff>(saB), vsB1b = lds16<T4::kVsOff + 16>(saB);
  int accA[4][4], accB[4][4];
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t a0 = kwA[c][0], a1 = kwA[c][1], b0 = kwB[c][0], b1 = kwB[c][1];
    mma_u8s8_cd(accA[c], st.init[c], (a0 >> 4) & 0x0F0F0F0Fu, (a1 >> 4) & 0x0F0F0F0Fu, a0 & 0x0F0F0F0Fu, a1 & 0x0F0F0F0Fu,
                st.qb[c][0], st.qb[c][1]);
    mma_u8s8_cd(accB[c], st.init[c], (b0 >> 4) & 0x0F0F0F0Fu, (b1 >> 4) & 0x0F0F0F0Fu, b0 & 0x0F0F0F0Fu, b1 & 0x0F0F0F0Fu,
                st.qb[c][0], st.qb[c][1]);
  }
  // V words of both pages: requested now, used after the softmax
  const uint32_t vA0 = sbA + st.v_offA, vA1 = sbA + st.v_offB, vB0 = sbB + st.v_offA, vB1 = sbB + st.v_offB;
  const uint2 WaA = lds64<0>(vA0), WbA = lds64<0>(vA1), WcA = lds64<512>(vA0), WdA = lds64<512>(vA1);
  const uint2 WaB = lds64<0>(vB0), WbB = lds64<0>(vB1), WcB = lds64<512>(vB0), WdB = lds64<512>(vB1);
  float sA[4] = {0.f, 0.f, 0.f, 0.f}, sB[4] = {0.f, 0.f, 0.f, 0.f};
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
  {
    const float kA0 = __uint_as_float(ksA0 << 16), kA1 = __uint_as_float(ksA1 << 16);
    const float kB0 = __uint_as_float(ksB0 << 16), kB1 = __uint_as_float(ksB1 << 16);
    sA[0] = __fmul_rn(__fmul_rn(sA[0], kA0), attn); sB[0] = __fmul_rn(__fmul_rn(sB[0], kB0), attn);
    sA[1] = __fmul_rn(__fmul_rn(sA[1], kA0), attn); sB[1] = __fmul_rn(__fmul_rn(sB[1], kB0), attn);
    sA[2] = __fmul_rn(__fmul_rn(sA[2], kA1), attn); sB[2] = __fmul_rn(__fmul_rn(sB[2], kB1), attn);
    sA[3] = __fmul_rn(__fmul_rn(sA[3], kA1), attn); sB[3] = __fmul_rn(__fmul_rn(sB[3], kB1), attn);
  }
  if (st0) { spA0[0] = sA[0]; spA0[8] = sA[2]; spB0[0] = sB[0]; spB0[8] = sB[2]; }
  if (st1) { spA1[0] = sA[1]; spA1[8] = sA[3]; spB1[0] = sB[1]; spB1[8] = sB[3]; }

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
#pragma unroll
      for (int i = 0; i < 9; ++i) { st.oacc[i][0] *= f0; st.oacc[i][1] *= f1; st.oacc[i][2] *= f0; st.oacc[i][3] *= f1; }
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

  // ---- (P * vscale).V for both pages ----
  const float vsA0 = __uint_as_float(vsA0b << 16), vsA1 = __uint_as_float(vsA1b << 16);
  const float vsB0 = __uint_as_float(vsB0b << 16), vsB1 = __uint_as_float(vsB1b << 16);
  const uint32_t A0 = movmatrix_trans(pack_f16x2_sat(pA[0] * vsA0, pA[1] * vsA0));
  const uint32_t B0 = movmatrix_trans(pack_f16x2_sat(pB[0] * vsB0, pB[1] * vsB0));
  const uint32_t A1 = movmatrix_trans(pack_f16x2_sat(pA[2] * vsA1, pA[3] * vsA1));
  const uint32_t B1 = movmatrix_trans(pack_f16x2_sat(pB[2] * vsB1, pB[3] * vsB1));
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
      mma_f16_16816(st.oacc[mt], v4_field<0>(XA), v4_field<4>(XA), v4_field<0>(XB), v4_field<4>(XB), A0, A1);
      mma_f16_16816(st.oacc[mt + 1], v4_field<0>(XA2), v4_field<4>(XA2), v4_field<0>(XB2), v4_field<4>(XB2), A0, A1);
      mma_f16_16816(st.oacc[mt], v4_field<0>(YA), v4_field<4>(YA), v4_field<0>(YB), v4_field<4>(YB), B0, B1);
      mma_f16_16816(st.oacc[mt + 1], v4_field<0>(YA2), v4_field<4>(YA2), v4_field<0>(YB2), v4_field<4>(YB2), B0, B1);
    }
  }
  mma_f16_16816(st.oacc[8], kOnesF16x2, kOnesF16x2, kOnesF16x2, kOnesF16x2, A0, A1);
  mma_f16_16816(st.oacc[8], kOnesF16x2, kOnesF16x2, kOnesF16x2, kOnesF16x2, B0, B1);
}

}  // namespace

template <int DT>
__global__ void __launch_bounds__(kScanWarps * 32, 4)
scan_k4v4_kernel(const ScanParams p, const __grid_constant__ CUtensorMap k_map,
                 const __grid_constant__ CUtensorMap v_map, const __grid_constant__ CUtensorMap k_map2,
                 const __grid_constant__ CUtensorMap v_map2) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // swizzled tiles must sit on 512-byte boundaries: align by hand (1 KB of slack is allocated)
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  JF_PHASE(0);
  const int cta_lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  JF_CTA_STAMP(cta_lin, 0);
#ifdef JF_PHASE_TIMING
  if (threadIdx.x == 0 && cta_lin < 1024) {
    unsigned smid__;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid__));
    g_cta_t[cta_lin * 8 + 5] = smid__;
  }
#endif
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
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&k_map2)) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&v_map2)) : "memory");
  }
  fence_barrier_init();
  __syncwarp();
  pdl_wait();  // nothing above reads global memory
  JF_PHASE(1);
  JF_CTA_STAMP(cta_lin, 1);

  // The first loads (sequence length, the block-table entries of the first ring of pages, the
  // query) do not depend on one another: all are issued here, so the prologue pays one
  // memory latency before the first copies can start, and the query arithmetic then runs
  // while those copies are in flight.
  // Warp w owns a contiguous quarter of the split's pages, so its block-table entries are
  // contiguous too: sixteen lanes fetch sixteen entries with one load, a whole chunk ahead of
  // its use, and park them in shared memory (kBtChunk entries per half of a two-chunk buffer).
  // A load issued while megabytes of page copies are queued in the memory system takes several
  // microseconds; fetched one entry at a time, a page or two ahead, those loads stalled the loop.
  const int pg_first = split * p.pages_per_split + warp * p.pages_per_warp;
  const int64_t* bt_w = p.block_table + static_cast<int64_t>(b) * p.max_blocks + pg_first;
  const int bt_avail = p.max_blocks - pg_first;   // entries of the row from this warp's first page on
  const int len_raw = p.seq_lens[b];
  // what is parked per page: the first cache row of its block (the tensor copies' y coordinate)
  // and how many of its 16 tokens are live -- worked out by sixteen lanes at once when a chunk
  // arrives, so that issuing a page's copies is a shared-memory read and the copies
  int2* bt_s = reinterpret_cast<int2*>(smem + kBtOff) + warp * (2 * kBtChunk);
  auto bt_load = [&](int chunk) -> int64_t {   // lanes 0..15: entry 16 * chunk + lane (never read when out of range)
    const int e = chunk * kBtChunk + lane;
    return (lane < kBtChunk && e < bt_avail) ? bt_w[e] : -1;
  };
  int64_t bt_pend = bt_load(0);
  // warp w prepares the query's 32-channel block w for the whole CTA (see below)
  uint4 q_raw = make_uint4(0u, 0u, 0u, 0u);
  if (g < p.G) {   // the 8 channels 32 w + 8 tig + {0..7} are 16 contiguous bytes
    const int64_t qbase = (static_cast<int64_t>(b) * p.H_q + hkv * p.G + g) * JF_HEAD_DIM;
    q_raw = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + qbase + 32 * warp + 8 * tig));
  }
  const int len = min(len_raw, p.max_S);
  const int n_pages = (len + 15) >> 4;
  const int my_n = max(0, min(min(pg_first + p.pages_per_warp, (split + 1) * p.pages_per_split), n_pages) - pg_first);

  const int64_t n_blocks_phys = p.num_slots >> 4;
  const int64_t head_row0 = static_cast<int64_t>(hkv) * p.num_slots;  // first cache row of this KV head
  const int last_pg = (len & 15) ? (n_pages - 1) : -1;   // the only page that can be partial

  // One elected lane issues the page's two tensor copies (K, V) and two scale copies.
  // The packed cache is read once per call: fetched as first-to-evict, it leaves the scores
  // this kernel writes (and the next kernel reads) in L2.
  const uint64_t stream_policy = l2_policy_evict_first();
  // entry e of this warp (page pg_first + e) from its block id: an invalid block id reads
  // block 0 and counts no live token; the sequence's last page may be partial
  auto bt_entry = [&](int64_t blk64, int e) -> int2 {
    const int pg = pg_first + e;
    const bool bad = blk64 < 0 || blk64 >= n_blocks_phys;
    const int valid = bad ? 0 : (pg == last_pg ? len - pg * 16 : 16);
    return make_int2(static_cast<int>(head_row0 + (bad ? 0 : blk64) * 16), valid);
  };
  // By one elected lane: the copies of one or two pages into slot `sl`.  Two pages whose blocks
  // are neighbours in the cache take one 32-row tensor copy per tensor and one 64-byte copy per
  // scale array; otherwise each page takes its own four copies.  Either way everything lands on
  // the slot's barrier.
  auto refill = [&](int sl, int2 ent_a, int2 ent_b, bool two) {
    if (elect_one()) {
      const uint32_t bar = bars0 + sl * 8;
      const uint32_t dst = slots0 + sl * T4::kSlotBytes;
      const int ra = ent_a.x, rb = ent_b.x;
      if (two && rb == ra + 16) {
        mbar_expect_tx_u32(bar, 2 * T4::kPageTx);
        tma_load_2d_u32(dst, &k_map2, 0, ra, bar, stream_policy);
        tma_load_2d_u32(dst + T4::kVOff, &v_map2, 0, ra, bar, stream_policy);
        bulk_g2s_u32(dst + T4::kScaleOff, p.k_scales + ra, 64, bar);
        bulk_g2s_u32(dst + T4::kScaleOff + T4::kVsOff, p.v_scales + ra, 64, bar);
      } else {
        mbar_expect_tx_u32(bar, two ? 2 * T4::kPageTx : T4::kPageTx);
        tma_load_2d_u32(dst, &k_map, 0, ra, bar, stream_policy);
        tma_load_2d_u32(dst + T4::kVOff, &v_map, 0, ra, bar, stream_policy);
        bulk_g2s_u32(dst + T4::kScaleOff, p.k_scales + ra, 32, bar);
        bulk_g2s_u32(dst + T4::kScaleOff + T4::kVsOff, p.v_scales + ra, 32, bar);
        if (two) {
          tma_load_2d_u32(dst + T4::kPageBytes, &k_map, 0, rb, bar, stream_policy);
          tma_load_2d_u32(dst + T4::kPageBytes + T4::kVOff, &v_map, 0, rb, bar, stream_policy);
          bulk_g2s_u32(dst + T4::kScaleOff + 32, p.k_scales + rb, 32, bar);
          bulk_g2s_u32(dst + T4::kScaleOff + T4::kVsOff + 32, p.v_scales + rb, 32, bar);
        }
      }
    }
  };

  // chunk 0 to shared memory, chunk 1 requested, the ring filled
  if (lane < kBtChunk) bt_s[lane] = bt_entry(bt_pend, lane);
  int bt_stored = 0;   // chunks 0..bt_stored are in shared memory; chunk bt_stored + 1 is in bt_pend
  bt_pend = bt_load(1);
  __syncwarp();
  {
#pragma unroll
    for (int sl = 0; sl < T4::kSlots; ++sl)
      if (2 * sl < my_n) refill(sl, bt_s[2 * sl], bt_s[2 * sl + 1], 2 * sl + 1 < my_n);
  }

  // ---- query: INT8 per 32-channel block.  Lane (head n = g, tig) owns channels
  //      32c + 8 tig + {0..7}; even channels meet the high nibbles, odd the low ones.
  //      The four warps need identical fragments: warp w quantises block c = w and the CTA
  //      exchanges the results through shared memory (a quarter of the arithmetic per warp). ----
  K4State st;
  {
    static_assert(kScanWarps == 4, "one warp per 32-channel query block");
    uint32_t* qx = reinterpret_cast<uint32_t*>(smem + kQxOff);  // [c][6][32]
    {
      float v[8];
      float amax = 0.f;
      const uint32_t rw[4] = {q_raw.x, q_raw.y, q_raw.z, q_raw.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[j] = Elem<DT>::to_f32(static_cast<uint16_t>((j & 1) ? (rw[j >> 1] >> 16) : (rw[j >> 1] & 0xFFFFu)));
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
  float* sp0 = p.scores + (static_cast<int64_t>(b) * p.H_q + h0) * p.max_S + t0 +
               static_cast<int64_t>(pg_first) * 16;
  float* sp1 = sp0 + p.max_S;
  const bool st0 = (2 * tig) < p.G, st1 = (2 * tig + 1) < p.G;
  const float attn = p.attn_scale;

  JF_PHASE(2);
  JF_CTA_STAMP(cta_lin, 2);
  // A round takes one slot: two pages (one at the end of the range).  Two full pages go through
  // the interleaved pair path; a partial or invalid page is processed on its own.
  int sl = 0;
  uint32_t parity = 0u;
  for (int it = 0; it < my_n; it += 2) {
    const bool two = it + 1 < my_n;
    // live tokens of the pages, from their parked entries (still resident: a chunk is
    // overwritten 16 pages after its last entry was issued)
    const int live_a = bt_s[it & (2 * kBtChunk - 1)].y, live_b = bt_s[(it + 1) & (2 * kBtChunk - 1)].y;
    if (!mbar_wait(&bars[sl], parity)) {
      if (it + 2 < my_n) mbar_wait(&bars[sl ^ 1], parity ^ static_cast<uint32_t>(sl), 1000000ull);
      failed = true;
      break;
    }
    if (it == 0) JF_PHASE(3);
    const uint32_t sb = slots0 + sl * T4::kSlotBytes, ss = sb + T4::kScaleOff;
    if (two && live_a == 16 && live_b == 16) {
      k4v4_page_pair(st, sb, sb + T4::kPageBytes, ss, ss + 32, attn, sp0, sp1, sp0 + 16, sp1 + 16, st0, st1);
    } else {
      if (live_a != 16) k4v4_page<true>(st, sb, ss, t0, live_a, attn, sp0, sp1, st0, st1);
      else k4v4_page<false>(st, sb, ss, t0, 16, attn, sp0, sp1, st0, st1);
      if (two) {
        if (live_b != 16) k4v4_page<true>(st, sb + T4::kPageBytes, ss + 32, t0, live_b, attn, sp0 + 16, sp1 + 16, st0, st1);
        else k4v4_page<false>(st, sb + T4::kPageBytes, ss + 32, t0, 16, attn, sp0 + 16, sp1 + 16, st0, st1);
      }
    }
    __syncwarp();
    // the refill below reads entries up to it + kPagesInFlight + 1: bring their chunk in first
    if (((it + kPagesInFlight + 1) >> 4) > bt_stored) {
      ++bt_stored;
      if (lane < kBtChunk) bt_s[(bt_stored & 1) * kBtChunk + lane] = bt_entry(bt_pend, bt_stored * kBtChunk + lane);
      bt_pend = bt_load(bt_stored + 1);
      __syncwarp();
    }
    const int e0 = it + kPagesInFlight;   // first page to fetch into the slot just freed
    if (e0 < my_n) refill(sl, bt_s[e0 & (2 * kBtChunk - 1)], bt_s[(e0 + 1) & (2 * kBtChunk - 1)], e0 + 1 < my_n);
    sp0 += 32;
    sp1 += 32;
    sl ^= 1;
    if (sl == 0) parity ^= 1u;
  }

  JF_PHASE(4);
  JF_CTA_STAMP(cta_lin, 3);
  JF_PHASE_VAL(10, my_n);
  pdl_trigger();  // the next kernel may start its prologue; it waits for this grid before reading
  if (failed && lane == 0) report_status(p.status, JF_ERR_TIMEOUT);

  __syncthreads();
  JF_PHASE(5);
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
  JF_PHASE(6);
  JF_CTA_STAMP(cta_lin, 4);
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

#ifdef JF_PHASE_TIMING
extern "C" int jf_debug_scan_times(unsigned long long* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_phase_t, sizeof(g_phase_t)));
}
extern "C" int jf_debug_scan_cta_times(unsigned long long* out) {   // [1024][8] globaltimer stamps
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_cta_t, sizeof(g_cta_t)));
}
#endif

jf_status_t launch_scan_k4v4(const ScanParams& sp, int q_dtype, dim3 grid, cudaStream_t stream) {
  const uint64_t rows = static_cast<uint64_t>(sp.H_kv) * static_cast<uint64_t>(sp.num_slots);
  if (rows > 0x7FFFFFFFull) return JF_ERR_UNSUPPORTED;
  CUtensorMap k_map, v_map, k_map2, v_map2;
  jf_status_t st = page_map(sp.k_data, rows, 16, &k_map);
  if (st == JF_OK) st = page_map(sp.v_data, rows, 16, &v_map);
  if (st == JF_OK) st = page_map(sp.k_data, rows, 32, &k_map2);
  if (st == JF_OK) st = page_map(sp.v_data, rows, 32, &v_map2);
  if (st != JF_OK) return st;
  const size_t smem = kSmemBytes;
  if (q_dtype == JF_DTYPE_BF16) {
    JF_ENSURE_SMEM(scan_k4v4_kernel<JF_DTYPE_BF16>, smem);
    JF_CUDA_TRY(launch_pdl(scan_k4v4_kernel<JF_DTYPE_BF16>, grid, dim3(kScanWarps * 32), smem, stream, sp, k_map, v_map,
                           k_map2, v_map2));
  } else {
    JF_ENSURE_SMEM(scan_k4v4_kernel<JF_DTYPE_FP16>, smem);
    JF_CUDA_TRY(launch_pdl(scan_k4v4_kernel<JF_DTYPE_FP16>, grid, dim3(kScanWarps * 32), smem, stream, sp, k_map, v_map,
                           k_map2, v_map2));
  }
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

}  // namespace jf
