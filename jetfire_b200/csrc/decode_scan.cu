// Fused low-bit decode-attention scan for sm_100a.
//
// One pass over the packed KV cache computes, for all query heads of a KV head at once
// (so every packed byte is read from HBM once per step):
//   approximate scores  s = attn_scale * sum_g  scale_g * (q . codes_g)       -> scratch
//   online softmax      p = exp(s - m_ref)                                   (registers)
//   output partial      O += (p * vscale) . vcodes                           (registers)
// Replaces the reference's Stage A score kernels (jetfire_vllm/csrc/int3_qk_scores.cu:
// 103-312, csrc/int8tc_qk_scores.cu:133-488) and Stage B softmax.V kernels
// (csrc/int2_softmax_v.cu:101-144, 601-789; csrc/int8tc_softmax_v_fused.cu:1017-1401),
// which materialise scores and weights in HBM and read V once per *query* head.
//
// Data movement: a 16-token page of the cache is contiguous per tensor (768 B of INT3 K,
// 512 B of INT2 V, 64 + 64 B of bf16 scales for K3V2), so a page is fetched with four
// bulk-async copies (TMA, non-tensor form) into a per-warp ring of two-page slots in shared
// memory, completion counted on the slot's mbarrier; two pages in neighbouring cache blocks
// share their copies.  A page is exactly one MMA M tile.  Block-table entries are fetched
// sixteen at a time, a chunk ahead of their use, and parked in shared memory together with
// what the copies need, so that the loop never waits for a global load and the warp-uniform
// work per page stays small.
//
// Compute: tokens sit on the MMA M axis and the (<= 8) query heads on N = 8.  Packed codes
// are expanded in registers straight into the A fragments of mma.sync.m16n8k16 (the
// dequantised tile never goes through shared memory).  A masked 2-/3-/4-bit field, read as a
// 16-bit float, is a subnormal number code * 2^pos * 2^-24 (fp16) or * 2^-133 (bf16): V fields go
// to the tensor core as they are (one AND per two codes), K fields take one bf16x2 fma that
// applies offset, group scale and the reference's bf16 rounding together.  The power-of-two
// factors are undone on the other operand (K: folded into Q) or on the output row (V); the V
// group scale is folded into P, the V codes' offset leaves through a sum(P) tile at the end.
#include "decode_scan.cuh"

namespace jf {

namespace {

// Bit position at which code x (0..7) of an INT3 group is picked up (see the unpack in the
// kernel): the 3-bit field has to sit inside the 7-bit bf16 mantissa, i.e. at 0..4.
__device__ __forceinline__ constexpr int k3_pos(int x) {
  return x == 0 ? 0 : x == 1 ? 3 : x == 2 ? 0 : x == 3 ? 4 : x == 4 ? 1 : x == 5 ? 0 : x == 6 ? 3 : 0;
}
// bit position of 2-bit field f (0..7, bit offset 2f of a 16-bit half row word)
__device__ __forceinline__ constexpr int v2_pos(int f) { return f <= 4 ? 2 * f : 2 * f - 10; }
// head-dim index inside the 8-wide chunk for field f: bytes are little-endian in the
// 16-bit load, codes MSB-first inside a byte
__device__ __forceinline__ constexpr int v2_dlocal(int f) { return 4 * (f >> 2) + 3 - (f & 3); }


// Shared-memory loads with a 32-bit address and an immediate offset: one instruction each,
// no 64-bit pointer arithmetic in the loop.
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
// lo | (hi << 16) for two 16-bit values, as an integer multiply-add (runs on the FMA pipe,
// which has twice the throughput of the logic pipe that PRMT/SHL/LOP3 share)
__device__ __forceinline__ uint32_t join16(uint32_t lo, uint32_t hi) {
  uint32_t d;
  asm("mad.lo.u32 %0, %1, 65536, %2;" : "=r"(d) : "r"(hi), "r"(lo));
  return d;
}

// Dequantised K in the reference's rounding, times a power of two, in ONE bf16x2 fma per two
// codes.  The masked 3-bit field, read as bf16, is the subnormal f * 2^POS * 2^-133 (exponent
// bits zero).  With S = scale * 2^100 and C = -4 * 2^POS * 2^-133 * S = -scale * 2^(POS - 31)
// (both exact: powers of two times the scale),
//   fma(field, S, C) = bf16_rn((f - 4) * scale * 2^(POS - 33)) = 2^(POS - 33) * bf16_rn((f - 4) * scale):
// the fma rounds once, and a power of two commutes with the rounding -- which is
// jetfire_vllm/csrc/int3_qk_scores.cu:94-99.  The factor 2^(POS - 33) is undone by the query
// operand.  (An 8-bit scale times a 3-bit integer needs at most 10 bits: exact before rounding.)
struct K3Scale {
  uint32_t S;     // scale * 2^100, both halves
  uint32_t C[5];  // -scale * 2^(POS - 31) for POS = 0..4, both halves (POS 2 is unused)
};
__device__ __forceinline__ K3Scale k3_scale(uint32_t scale2) {
  K3Scale k;
  k.S = mul_bf16x2(scale2, 0x71807180u);        // 2^100
  k.C[0] = mul_bf16x2(scale2, 0xB000B000u);     // -2^-31
  k.C[1] = mul_bf16x2(scale2, 0xB080B080u);     // -2^-30
  k.C[2] = 0u;
  k.C[3] = mul_bf16x2(scale2, 0xB180B180u);     // -2^-28
  k.C[4] = mul_bf16x2(scale2, 0xB200B200u);     // -2^-27
  return k;
}
template <int POS>
__device__ __forceinline__ uint32_t k3_field(uint32_t v, const K3Scale& k) {
  constexpr uint32_t m = (7u << POS) | (7u << (POS + 16));
  return fma_bf16x2(v & m, k.S, k.C[POS]);
}
// One 32-bit word of each byte plane (4 INT3 groups = 32 channels of one row) -> 16 bf16x2
// registers R[pair][code]: pair p holds groups (2p, 2p+1) in its (low, high) halves.
__device__ __forceinline__ void k3_unpack_row(uint32_t P0, uint32_t P1, uint32_t P2, const K3Scale& scale2,
                                              uint32_t (&R)[2][8]) {
#pragma unroll
  for (int pr = 0; pr < 2; ++pr) {
    const uint32_t sel = pr ? 0x7362u : 0x5140u;
    const uint32_t lo = prmt(P2, P1, sel);  // halves: bits 15..0 of the two 24-bit groups
    const uint32_t hi = prmt(P1, P0, sel);  // halves: bits 23..8
    const uint32_t lo6 = lo >> 6, hi7 = hi >> 7, hi13 = hi >> 13;
    R[pr][7] = k3_field<0>(lo, scale2);
    R[pr][6] = k3_field<3>(lo, scale2);
    R[pr][5] = k3_field<0>(lo6, scale2);
    R[pr][4] = k3_field<1>(hi, scale2);
    R[pr][3] = k3_field<4>(hi, scale2);
    R[pr][2] = k3_field<0>(hi7, scale2);
    R[pr][1] = k3_field<3>(hi7, scale2);
    R[pr][0] = k3_field<0>(hi13, scale2);
  }
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

// A V field as an fp16 operand without arithmetic: the masked 2-bit field, read as fp16, is the
// subnormal code * 2^POS * 2^-24.  The codes' offset of 2 is not removed per element: one extra
// MMA per page and group against a row of ones collects sum(P), and the epilogue forms
// 2^(24 - POS) * acc - 2 * sum(P).
template <int POS>
__device__ __forceinline__ uint32_t v2_field(uint32_t v) {
  constexpr uint32_t m = (3u << POS) | (3u << (POS + 16));
  return v & m;
}
constexpr uint32_t kOnesF16x2 = 0x3C003C00u;

// Per-warp state that lives across pages.
template <int QT>
struct K3State {
  uint32_t qf[QT][8][2];   // query fragments (B operand of the K MMA)
  float oacc[10][4];       // output accumulators, O^T fragments; tiles 8, 9: sum of the P operand per V group
  float m_ref0, m_ref1, l0, l1;
  float pm_a, pm_b;        // largest score of this lane's tokens in the current round, heads 2tig and 2tig+1
  uint32_t smax_bits;      // largest K group scale seen (bf16 bits; positive floats order as integers)
  uint32_t ks_sel;         // PRMT selector: this lane's K group scale into both halves
};

// One 16-token page.  `sb` = shared-memory address of the ring slot; the offsets select the
// page's half of it.  kPartial: the last page of
// a sequence (or a page whose block id was invalid) -- rows at or past `valid` are neutralised;
// the common full-page instance carries none of that logic.
// kParts: 0 = scores and output partials; 1 = scores and softmax sums only (no V);
// 2 = output partials from scores read back from memory (no K).
template <int QT, bool kPartial, int kParts>
__device__ __forceinline__ void k3v2_page(K3State<QT>& st, uint32_t sb, uint32_t k_addr_off, uint32_t v_addr_off,
                                          uint32_t s_addr_off, int t0, int valid, float attn, float* sp0,
                                          float* sp1, bool st0, bool st1) {
  using T = Tile<JF_MODE_K3V2>;
  constexpr bool kDoK = kParts != 2, kDoV = kParts != 1;
  // ---------------- K: unpack + Q.K^T ----------------
  const uint32_t sa = sb + s_addr_off;
  uint32_t ksw0 = 0u, ksw1 = 0u, vsw0 = 0u, vsw1 = 0u;
  if (kDoK) { ksw0 = lds32<0>(sa); ksw1 = lds32<32>(sa); }
  if (kDoV) { vsw0 = lds32<T::kVsRel>(sa); vsw1 = lds32<T::kVsRel + 32>(sa); }
  float vs00 = __uint_as_float(vsw0 << 16), vs01 = __uint_as_float(vsw0 & 0xFFFF0000u);
  float vs10 = __uint_as_float(vsw1 << 16), vs11 = __uint_as_float(vsw1 & 0xFFFF0000u);
  if (kPartial) {
    if (t0 >= valid) { ksw0 = 0u; vs00 = vs01 = 0.f; }
    if (t0 + 8 >= valid) { ksw1 = 0u; vs10 = vs11 = 0.f; }
  }
  // all shared-memory reads of the page are issued up front (the loads keep their source order)
  const uint32_t ka = sb + k_addr_off;
  uint32_t kw0 = 0u, kw1 = 0u, kw2 = 0u, kw3 = 0u, kw4 = 0u, kw5 = 0u;
  if (kDoK) {
    kw0 = lds32<0>(ka); kw1 = lds32<16>(ka); kw2 = lds32<32>(ka);
    kw3 = lds32<8 * T::kKRow>(ka); kw4 = lds32<8 * T::kKRow + 16>(ka); kw5 = lds32<8 * T::kKRow + 32>(ka);
  }
  const uint32_t va_addr = sb + v_addr_off;
  uint32_t vh[2][4] = {{0u, 0u, 0u, 0u}, {0u, 0u, 0u, 0u}};
  if (kDoV) {
    vh[0][0] = lds16<0>(va_addr); vh[0][1] = lds16<4 * T::kVRow>(va_addr);
    vh[0][2] = lds16<8 * T::kVRow>(va_addr); vh[0][3] = lds16<12 * T::kVRow>(va_addr);
    vh[1][0] = lds16<16>(va_addr); vh[1][1] = lds16<4 * T::kVRow + 16>(va_addr);
    vh[1][2] = lds16<8 * T::kVRow + 16>(va_addr); vh[1][3] = lds16<12 * T::kVRow + 16>(va_addr);
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (kDoK) {
    const uint32_t sc0 = prmt(ksw0, ksw0, st.ks_sel), sc1 = prmt(ksw1, ksw1, st.ks_sel);
    st.smax_bits = max(st.smax_bits, max(sc0 & 0x7FFFu, sc1 & 0x7FFFu));
    uint32_t R0[2][8], R1[2][8];
    k3_unpack_row(kw0, kw1, kw2, k3_scale(sc0), R0);
    k3_unpack_row(kw3, kw4, kw5, k3_scale(sc1), R1);
#pragma unroll
    for (int t = 0; t < QT; ++t)
#pragma unroll
      for (int x = 0; x < 8; ++x)
        mma_bf16_16816(acc, R0[0][x], R1[0][x], R0[1][x], R1[1][x], st.qf[t][x][0], st.qf[t][x][1]);
  }

  // ---------------- scores ----------------
  float s0 = acc[0] * attn;  // row g,   head 2tig
  float s1 = acc[1] * attn;  // row g,   head 2tig+1
  float s2 = acc[2] * attn;  // row g+8, head 2tig
  float s3 = acc[3] * attn;  // row g+8, head 2tig+1
  const bool lo = !kPartial || t0 < valid, hi = !kPartial || t0 + 8 < valid;
  if (!kDoK) {
    // the scores an earlier scan stored (heads past the group stay at 0: their columns are dropped)
    if (st0 && lo) s0 = sp0[0];
    if (st0 && hi) s2 = sp0[8];
    if (st1 && lo) s1 = sp1[0];
    if (st1 && hi) s3 = sp1[8];
  }
  if (kPartial) {
    if (!lo) { s0 = s1 = -INFINITY; }
    if (!hi) { s2 = s3 = -INFINITY; }
  }
  if (kDoK) {
    if (kPartial) {
      if (st0 && lo) sp0[0] = s0;
      if (st0 && hi) sp0[8] = s2;
      if (st1 && lo) sp1[0] = s1;
      if (st1 && hi) sp1[8] = s3;
    } else {
      if (st0) { sp0[0] = s0; sp0[8] = s2; }
      if (st1) { sp1[0] = s1; sp1[8] = s3; }
    }
    // running maxima of this lane's tokens, for the page-pair maxima the select kernel reads
    st.pm_a = fmaxf(st.pm_a, fmaxf(s0, s2));
    st.pm_b = fmaxf(st.pm_b, fmaxf(s1, s3));
  }

  // ---------------- online softmax ----------------
  float p0, p1, p2, p3;
  softmax_step(s0, s1, s2, s3, st.m_ref0, st.m_ref1, st.l0, st.l1, st.oacc, p0, p1, p2, p3);
  // ---------------- V: unpack + (P * vscale).V ----------------
#pragma unroll
  for (int qh = 0; kDoV && qh < 2; ++qh) {
    const float va = qh ? vs01 : vs00, vb = qh ? vs11 : vs10;
    const uint32_t B0 = movmatrix_trans(pack_f16x2_sat(p0 * va, p1 * va));  // tokens tig, tig+4
    const uint32_t B1 = movmatrix_trans(pack_f16x2_sat(p2 * vb, p3 * vb));  // tokens tig+8, tig+12
    const uint32_t Ha = vh[qh][0], Hb = vh[qh][1], Hc = vh[qh][2], Hd = vh[qh][3];
    const uint32_t XA = join16(Ha, Hb), XB = join16(Hc, Hd);
    const uint32_t XA2 = XA >> 10, XB2 = XB >> 10;
    // fields 2ml -> output row g, 2ml+1 -> output row g+8
    mma_f16_16816(st.oacc[qh * 4 + 0], v2_field<0>(XA), v2_field<2>(XA), v2_field<0>(XB), v2_field<2>(XB), B0, B1);
    mma_f16_16816(st.oacc[qh * 4 + 1], v2_field<4>(XA), v2_field<6>(XA), v2_field<4>(XB), v2_field<6>(XB), B0, B1);
    mma_f16_16816(st.oacc[qh * 4 + 2], v2_field<8>(XA), v2_field<0>(XA2), v2_field<8>(XB), v2_field<0>(XB2), B0, B1);
    mma_f16_16816(st.oacc[qh * 4 + 3], v2_field<2>(XA2), v2_field<4>(XA2), v2_field<2>(XB2), v2_field<4>(XB2), B0, B1);
    mma_f16_16816(st.oacc[8 + qh], kOnesF16x2, kOnesF16x2, kOnesF16x2, kOnesF16x2, B0, B1);
  }
}

}  // namespace

// ------------------------------------------------------------------------------------
// K3V2
// ------------------------------------------------------------------------------------
template <int DT, int kParts>
__global__ void __launch_bounds__(kScanWarps * 32, (DT == JF_DTYPE_FP16) ? 3 : 4)
scan_k3v2_kernel(const ScanParams p) {
  using T = Tile<JF_MODE_K3V2>;
  constexpr int kQTerms = (DT == JF_DTYPE_FP16) ? 2 : 1;
  constexpr bool kDoK = kParts != 2, kDoV = kParts != 1;
  constexpr uint32_t kTxPage = (kDoK ? T::kKPage + T::kSPage : 0) + (kDoV ? T::kVPage + T::kSPage : 0);
  extern __shared__ __align__(128) uint8_t smem[];
  // the warp index is the same for all lanes; routing it through a shuffle tells the
  // compiler so, and lets stage / barrier addresses live in uniform registers
  const int warp = __shfl_sync(0xFFFFFFFFu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;

  const uint32_t smem_base = smem_u32(smem);
  constexpr int kRingBytes = kScanWarps * T::kSlots * T::kSlotBytes;
  constexpr int kPagesInFlight = 2 * T::kSlots;
  const uint32_t slots0 = smem_base + warp * (T::kSlots * T::kSlotBytes);
  const uint32_t bars0 = smem_base + kRingBytes + warp * (T::kSlots * 8);   // one barrier per slot
  // parked per page: the first cache row of its block and how many of its 16 tokens are live
  int2* bt_s = reinterpret_cast<int2*>(smem + kRingBytes + kScanWarps * T::kSlots * 8) + warp * (2 * kBtChunk);

  if (lane == 0) {
    for (int s = 0; s < T::kSlots; ++s) mbar_init(reinterpret_cast<uint64_t*>(smem + (bars0 - smem_base)) + s, 1);
  }
  fence_barrier_init();
  __syncwarp();
  pdl_wait();  // nothing above reads global memory

  const int len = min(p.seq_lens[b], p.max_S);
  const int n_pages = (len + 15) >> 4;
  // Warp w owns a contiguous quarter of the split's pages, so its block-table entries are
  // contiguous too: sixteen lanes fetch sixteen entries with one load, a whole chunk ahead of
  // its use, and park them in shared memory.  (A load issued while megabytes of page copies are
  // queued in the memory system takes microseconds; fetched one entry at a time, a page or two
  // ahead, those loads stalled the loop.)
  const int pg_first = split * p.pages_per_split + warp * p.pages_per_warp;
  const int my_n = max(0, min(min(pg_first + p.pages_per_warp, (split + 1) * p.pages_per_split), n_pages) - pg_first);
  const int64_t* bt_w = p.block_table + static_cast<int64_t>(b) * p.max_blocks + pg_first;
  const int bt_avail = p.max_blocks - pg_first;   // entries of the row from this warp's first page on
  auto bt_load = [&](int chunk) -> int64_t {   // lanes 0..15: entry 16 * chunk + lane (never read when out of range)
    const int e = chunk * kBtChunk + lane;
    return (lane < kBtChunk && e < bt_avail) ? bt_w[e] : -1;
  };
  int64_t bt_pend = bt_load(0);
  const int64_t n_blocks_phys = p.num_slots >> 4;

  // One elected lane issues the four bulk copies of a page (K data, V data, K scales, V scales).
  // The packed cache is read once per call: fetched as first-to-evict, it leaves the scores
  // this kernel writes (and the next kernel reads) in L2.
  const uint64_t stream_policy = l2_policy_evict_first();
  const int64_t head_rows = static_cast<int64_t>(hkv >> p.kv_shift) * p.num_slots;
  const uint8_t* ks_b = reinterpret_cast<const uint8_t*>(p.k_scales);
  const uint8_t* vs_b = reinterpret_cast<const uint8_t*>(p.v_scales);
  const int last_pg = (len & 15) ? (n_pages - 1) : -1;   // the only page that can be partial
  // entry e of this warp (page pg_first + e) from its block id, worked out by sixteen lanes at
  // once when a chunk arrives: an invalid block id reads block 0 and counts no live token; the
  // sequence's last page may be partial
  auto bt_entry = [&](int64_t blk64, int e) -> int2 {
    const int pg = pg_first + e;
    const bool bad = blk64 < 0 || blk64 >= n_blocks_phys;
    const int valid = bad ? 0 : (pg == last_pg ? len - pg * 16 : 16);
    return make_int2(static_cast<int>(head_rows + (bad ? 0 : blk64) * 16), valid);
  };
  // By one elected lane: the copies of one or two pages into slot `sl`.  Two pages whose blocks
  // are neighbours in the cache take one copy per array; otherwise each page takes its own four.
  // Either way everything lands on the slot's barrier.
  auto refill = [&](int sl, int2 ent_a, int2 ent_b, bool two) {
    if (elect_one()) {
      const uint32_t bar = bars0 + sl * 8;
      const uint32_t dst = slots0 + sl * T::kSlotBytes;
      const int64_t ra = ent_a.x, rb = ent_b.x;
      const bool joined = two && rb == ra + 16;
      const uint32_t n = joined ? 2u : 1u;
      mbar_expect_tx_u32(bar, two ? 2 * kTxPage : kTxPage);
      if (kDoK) {
        bulk_g2s_u32_hint(dst, p.k_data + ra * T::kKRow, n * T::kKPage, bar, stream_policy);
        bulk_g2s_u32(dst + T::kKsOff, ks_b + ra * (2 * T::kNG), n * T::kSPage, bar);
      }
      if (kDoV) {
        bulk_g2s_u32_hint(dst + T::kVOff, p.v_data + ra * T::kVRow, n * T::kVPage, bar, stream_policy);
        bulk_g2s_u32(dst + T::kKsOff + T::kVsRel, vs_b + ra * (2 * T::kNG), n * T::kSPage, bar);
      }
      if (two && !joined) {
        if (kDoK) {
          bulk_g2s_u32_hint(dst + T::kKPage, p.k_data + rb * T::kKRow, T::kKPage, bar, stream_policy);
          bulk_g2s_u32(dst + T::kKsOff + T::kSPage, ks_b + rb * (2 * T::kNG), T::kSPage, bar);
        }
        if (kDoV) {
          bulk_g2s_u32_hint(dst + T::kVOff + T::kVPage, p.v_data + rb * T::kVRow, T::kVPage, bar, stream_policy);
          bulk_g2s_u32(dst + T::kKsOff + T::kVsRel + T::kSPage, vs_b + rb * (2 * T::kNG), T::kSPage, bar);
        }
      }
    }
  };

  // prologue: chunk 0 to shared memory, chunk 1 requested, the ring filled
  if (lane < kBtChunk) bt_s[lane] = bt_entry(bt_pend, lane);
  int bt_stored = 0;   // chunks 0..bt_stored are in shared memory; chunk bt_stored + 1 is in bt_pend
  bt_pend = bt_load(1);
  __syncwarp();
  for (int sl = 0; sl < T::kSlots; ++sl)
    if (2 * sl < my_n) refill(sl, bt_s[2 * sl], bt_s[2 * sl + 1], 2 * sl + 1 < my_n);

  // ---- query fragments: B operand of the K MMA, scaled by 2^(33 - pos) of the code it meets.
  //      Lane (head n = g, tig) covers channels 32 tig + 8 j + x (group j, code x); k-step x
  //      pairs groups (0,1) in b0 and (2,3) in b1.  A bf16 query is used as is; an fp16 query
  //      (11-bit significand) is split exactly into two bf16 terms, hi + lo. ----
  K3State<kQTerms> st;
  if (kDoK) {
    const int h = hkv * p.G + g;
    const bool live = g < p.G;
    const int64_t qbase = (static_cast<int64_t>(b) * p.H_q + h) * JF_HEAD_DIM;
    // this lane's 32 channels are contiguous: four 16-byte loads
    uint32_t qraw[16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (live) v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + qbase + 32 * tig) + i);
      qraw[4 * i] = v.x; qraw[4 * i + 1] = v.y; qraw[4 * i + 2] = v.z; qraw[4 * i + 3] = v.w;
    }
    auto qval = [&](int d) {  // channel 32 tig + d of this lane's head
      const uint32_t w = qraw[d >> 1];
      return Elem<DT>::to_f32(static_cast<uint16_t>((d & 1) ? (w >> 16) : (w & 0xFFFFu)));
    };
#pragma unroll
    for (int x = 0; x < 8; ++x) {
      const float sc = 8589934592.0f / static_cast<float>(1 << k3_pos(x));   // 2^(33 - POS), see k3_field
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int d0 = 16 * half + x;  // group j = 2 * half
        const float a = qval(d0) * sc, c = qval(d0 + 8) * sc;
        const uint32_t hi2 = pack_bf16x2(a, c);
        st.qf[0][x][half] = hi2;
        if (kQTerms == 2) {
          const float ra = a - __uint_as_float(hi2 << 16), rc = c - __uint_as_float(hi2 & 0xFFFF0000u);
          st.qf[kQTerms - 1][x][half] = pack_bf16x2(ra, rc);
        }
      }
    }
  }
  st.ks_sel = (tig >> 1) ? 0x3232u : 0x1010u;
#pragma unroll
  for (int i = 0; i < 10; ++i) { st.oacc[i][0] = st.oacc[i][1] = st.oacc[i][2] = st.oacc[i][3] = 0.f; }
  st.m_ref0 = kMinusBig; st.m_ref1 = kMinusBig; st.l0 = 0.f; st.l1 = 0.f;
  st.smax_bits = 0u;
  st.pm_a = st.pm_b = -INFINITY;
  bool failed = false;

  const int t0 = (g >> 1) | ((g & 1) << 2);  // token of MMA row g (rows g + 8 -> t0 + 8)
  const uint32_t k_addr_off = t0 * T::kKRow + tig * 4;               // in the slot's first half
  const uint32_t v_addr_off = T::kVOff + tig * T::kVRow + 2 * g;
  const uint32_t s_addr_off = T::kKsOff + t0 * 4;
  const int h0 = hkv * p.G + 2 * tig;
  float* sp0 = p.scores + (static_cast<int64_t>(b) * p.H_q + h0) * p.max_S + t0 +
               static_cast<int64_t>(pg_first) * 16;
  float* sp1 = sp0 + p.max_S;
  const bool st0 = (2 * tig) < p.G, st1 = (2 * tig + 1) < p.G;
  // Page-pair maxima (pages 2m, 2m+1; a warp's range starts at an even page): after the round's
  // butterfly the lanes with bits 2 and 3 clear hold them -- lane bit 4 clear: head 2tig, set: 2tig+1.
  const int pm_head = 2 * tig + (lane >> 4);
  const bool want_pm = kDoK && p.pmax != nullptr;   // the same for the whole grid
  float* pmw = (want_pm && (lane & 12) == 0 && pm_head < p.G)
                   ? p.pmax + (static_cast<int64_t>(b) * p.H_q + hkv * p.G + pm_head) * p.np_stride + (pg_first >> 1)
                   : nullptr;
  const float attn = p.attn_scale;

  // A round takes one slot: two pages (one at the end of the range), processed one after the
  // other; the ring bookkeeping and the election of the copying lane are paid once per round.
  int sl = 0;
  uint32_t parity = 0u;
  for (int it = 0; it < my_n; it += 2) {
    const int n_here = (it + 1 < my_n) ? 2 : 1;
    if (!mbar_wait(reinterpret_cast<uint64_t*>(smem + (bars0 - smem_base)) + sl, parity)) {
      // give the copies that were already issued a short, bounded chance to land
      for (int j = 1; j < T::kSlots && it + 2 * j < my_n; ++j) {
        const int o = (sl + j) % T::kSlots;
        mbar_wait(reinterpret_cast<uint64_t*>(smem + (bars0 - smem_base)) + o, o > sl ? parity : parity ^ 1u, 1000000ull);
      }
      failed = true;
      break;
    }
    const uint32_t sb = slots0 + sl * T::kSlotBytes;
#pragma unroll 1
    for (int k = 0; k < n_here; ++k) {
      const int live = bt_s[(it + k) & (2 * kBtChunk - 1)].y;   // the page's parked entry is still resident
      const uint32_t ko = k_addr_off + k * T::kKPage, vo = v_addr_off + k * T::kVPage, so = s_addr_off + k * T::kSPage;
      if (live != 16)
        k3v2_page<kQTerms, true, kParts>(st, sb, ko, vo, so, t0, live, attn, sp0, sp1, st0, st1);
      else
        k3v2_page<kQTerms, false, kParts>(st, sb, ko, vo, so, t0, 16, attn, sp0, sp1, st0, st1);
      sp0 += 16;
      sp1 += 16;
    }
    if (want_pm) {
      // largest score of the round's pages per head: the halves of the warp trade one head for the
      // other (each lane sends one value and keeps one), then reduce over lane bits 3 and 2
      const bool up = (lane & 16) != 0;
      float v = fmaxf(up ? st.pm_b : st.pm_a, __shfl_xor_sync(0xFFFFFFFFu, up ? st.pm_a : st.pm_b, 16));
      v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, 8));
      v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, 4));
      if (pmw) *pmw++ = v;
      st.pm_a = st.pm_b = -INFINITY;
    }
    __syncwarp();
    if (((it + kPagesInFlight + 1) >> 4) > bt_stored) {   // the refill below reads entries up to it + kPagesInFlight + 1
      ++bt_stored;
      if (lane < kBtChunk) bt_s[(bt_stored & 1) * kBtChunk + lane] = bt_entry(bt_pend, bt_stored * kBtChunk + lane);
      bt_pend = bt_load(bt_stored + 1);
      __syncwarp();
    }
    const int e0 = it + kPagesInFlight;   // first page to fetch into the slot just freed
    if (e0 < my_n) refill(sl, bt_s[e0 & (2 * kBtChunk - 1)], bt_s[(e0 + 1) & (2 * kBtChunk - 1)], e0 + 1 < my_n);
    if (++sl == T::kSlots) { sl = 0; parity ^= 1u; }
  }

  pdl_trigger();  // the next kernel may start its prologue; it waits for this grid before reading
  if (failed && lane == 0) report_status(p.status, JF_ERR_TIMEOUT);
  if (kDoK && threadIdx.x == 0 && (blockIdx.x | blockIdx.y | blockIdx.z) == 0) p.status[4] = want_pm ? kPageMaxTag : 0;

  // ---------------- CTA merge: 4 warps -> one partial ----------------
  __syncthreads();  // every warp is done with its stages (or gave up); smem is reused below
  {
    float* wo = reinterpret_cast<float*>(smem) + warp * (kHeadsPad * JF_HEAD_DIM);
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      const int qh = mt >> 2, ml = mt & 3;
      const int fa = 2 * ml, fb = 2 * ml + 1;
      const int da = 64 * qh + 8 * g + v2_dlocal(fa), db = 64 * qh + 8 * g + v2_dlocal(fb);
      // 2^(24 - POS) * sum(P * field) - 2 * sum(P): the codes' offset leaves here (see v2_field)
      const float ua = 16777216.0f / static_cast<float>(1 << v2_pos(fa)), ub = 16777216.0f / static_cast<float>(1 << v2_pos(fb));
      wo[(2 * tig) * JF_HEAD_DIM + da] = fmaf(st.oacc[mt][0], ua, -2.0f * st.oacc[8 + qh][0]);
      wo[(2 * tig + 1) * JF_HEAD_DIM + da] = fmaf(st.oacc[mt][1], ua, -2.0f * st.oacc[8 + qh][1]);
      wo[(2 * tig) * JF_HEAD_DIM + db] = fmaf(st.oacc[mt][2], ub, -2.0f * st.oacc[8 + qh][2]);
      wo[(2 * tig + 1) * JF_HEAD_DIM + db] = fmaf(st.oacc[mt][3], ub, -2.0f * st.oacc[8 + qh][3]);
    }
  }
  const float smax = __uint_as_float(st.smax_bits << 16);
  cta_merge_store(p, smem, st.l0, st.l1, st.m_ref0, st.m_ref1, (tig >> 1) ? 0.f : smax, (tig >> 1) ? smax : 0.f,
                  split, hkv, b);
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
jf_status_t validate_decode_args(const jf_decode_args* a) {
  if (!a) return JF_ERR_ARG;
  if (a->mode != JF_MODE_K3V2 && a->mode != JF_MODE_K4V4) return JF_ERR_UNSUPPORTED;
  if (a->q_dtype != JF_DTYPE_BF16 && a->q_dtype != JF_DTYPE_FP16) return JF_ERR_UNSUPPORTED;
  if (a->B <= 0 || a->H_q <= 0 || a->H_kv <= 0 || a->max_S <= 0) return JF_ERR_ARG;
  if (a->H_q % a->H_kv != 0) return JF_ERR_ARG;
  const int G = a->H_q / a->H_kv;
  if (G > kHeadsPad && G != JF_MAX_GROUP) return JF_ERR_UNSUPPORTED;   // 1..8, or 16 as two halves
  if (a->block_size != JF_BLOCK_SIZE) return JF_ERR_UNSUPPORTED;
  if (a->max_S > 262144) return JF_ERR_UNSUPPORTED;
  if (a->top_k < 1 || a->top_k > JF_MAX_TOP_K) return JF_ERR_UNSUPPORTED;
  if (a->max_blocks < (a->max_S + 15) / 16) return JF_ERR_ARG;
  if (a->num_slots <= 0 || (a->num_slots % 16) != 0) return JF_ERR_ARG;
  // the scan kernels carry a page's first cache row (over all KV heads) as a 32-bit integer
  if (static_cast<uint64_t>(a->H_kv) * static_cast<uint64_t>(a->num_slots) > 0x7FFFFFFFull) return JF_ERR_UNSUPPORTED;
  if (a->scan_parts < JF_SCAN_ALL || a->scan_parts > JF_SCAN_V_ONLY) return JF_ERR_ARG;
  if (a->stage_b != JF_STAGE_B_FP32 && a->stage_b != JF_STAGE_B_INT8P) return JF_ERR_ARG;
  if (a->stage_b == JF_STAGE_B_INT8P && a->mode != JF_MODE_K4V4) return JF_ERR_UNSUPPORTED;
  const bool need_k = a->scan_parts != JF_SCAN_V_ONLY, need_v = a->scan_parts != JF_SCAN_K_ONLY;
  if (!a->block_table || !a->seq_lens) return JF_ERR_ARG;
  if (need_k && (!a->q || !a->k_data || !a->k_scales)) return JF_ERR_ARG;
  if (need_v && (!a->v_data || !a->v_scales)) return JF_ERR_ARG;
  if (!need_k && !a->scores) return JF_ERR_ARG;   // the scores are this call's input
  if (!aligned(a->k_data, 16) || !aligned(a->v_data, 16) || !aligned(a->k_scales, 16) || !aligned(a->v_scales, 16))
    return JF_ERR_ARG;
  if (!a->workspace || !aligned(a->workspace, 256)) return JF_ERR_WORKSPACE;
  if (a->workspace_bytes < jf_decode_workspace_bytes(a->mode, a->B, a->H_q, a->H_kv, a->max_S, a->top_k))
    return JF_ERR_WORKSPACE;
  return JF_OK;
}

template <int DT, int kParts>
jf_status_t launch_k3v2(const ScanParams& sp, dim3 grid, cudaStream_t stream) {
  using T = Tile<JF_MODE_K3V2>;
  const size_t smem = kScanWarps * T::kSlots * (T::kSlotBytes + 8) + kScanWarps * 2 * kBtChunk * 8;  // ring, barriers, block-table chunks
  static_assert(kScanWarps * T::kSlots * T::kSlotBytes >= kMergeBytes, "merge buffer");
  JF_ENSURE_SMEM((scan_k3v2_kernel<DT, kParts>), smem);
  JF_CUDA_TRY(launch_pdl(scan_k3v2_kernel<DT, kParts>, grid, dim3(kScanWarps * 32), smem, stream, sp));
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

__global__ void fill_neg_inf_tail_kernel(float* scores, const int32_t* seq_lens, int H_q, int max_S) {
  const int bh = blockIdx.x, b = bh / H_q;
  const int len = min(seq_lens[b], max_S);
  float* row = scores + static_cast<int64_t>(bh) * max_S;
  for (int i = len + threadIdx.x; i < max_S; i += blockDim.x) row[i] = -INFINITY;
}

}  // namespace jf

extern "C" uint64_t jf_decode_workspace_bytes(int32_t mode, int32_t B, int32_t H_q, int32_t H_kv,
                                              int32_t max_S, int32_t top_k) {
  if (B <= 0 || H_q <= 0 || H_kv <= 0 || max_S <= 0 || top_k <= 0) return 0;
  return jf::carve_workspace(nullptr, mode, B, H_q, H_kv, max_S, top_k, true).bytes;
}

extern "C" jf_status_t jf_decode_scan(const jf_decode_args* a, jf_stream_t stream_) {
  using namespace jf;
  jf_status_t st = validate_decode_args(a);
  if (st != JF_OK) return st;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  Workspace ws = carve_workspace(a->workspace, a->mode, a->B, a->H_q, a->H_kv, a->max_S, a->top_k, true);
  ScanParams sp{};
  sp.q = a->q;
  sp.k_data = a->k_data;  sp.k_scales = static_cast<const uint16_t*>(a->k_scales);
  sp.v_data = a->v_data;  sp.v_scales = static_cast<const uint16_t*>(a->v_scales);
  sp.block_table = a->block_table;  sp.seq_lens = a->seq_lens;
  sp.scores = a->scores ? a->scores : ws.scores;
  // the maxima of groups of pages, if the select kernel of this call will work from them
  const SelectPlan plan = select_plan(a, sp.scores);
  if (!plan.supported) return JF_ERR_UNSUPPORTED;
  sp.pmax = plan.lean ? ws.pmax : nullptr;
  sp.np_stride = page_max_stride(a->mode, a->max_S);
  sp.part_o = ws.part_o; sp.part_m = ws.part_m; sp.part_l = ws.part_l; sp.part_smax = ws.part_smax;
  sp.status = ws.status;
  sp.num_slots = a->num_slots;
  const HeadGeom hg = head_geom(a->H_q, a->H_kv);
  sp.B = a->B; sp.H_q = a->H_q; sp.H_kv = hg.H_kv; sp.G = hg.G; sp.kv_shift = hg.shift;
  sp.max_S = a->max_S; sp.max_blocks = a->max_blocks;
  sp.splits = scan_splits(a->mode, a->q_dtype, a->B, hg.H_kv, a->max_S);
  const int pages = (a->max_S + 15) / 16;
  sp.pages_per_split = (pages + sp.splits - 1) / sp.splits;
  sp.pages_per_warp = (sp.pages_per_split + kScanWarps - 1) / kScanWarps;
  if (a->mode == JF_MODE_K3V2) {
    // every warp's range starts at an even page, so that the pairs of pages a round takes are the
    // pairs (2m, 2m+1) of the row -- the groups of the page maxima
    sp.pages_per_split = (sp.pages_per_split + 1) & ~1;
    sp.pages_per_warp = (((sp.pages_per_split + kScanWarps - 1) / kScanWarps) + 1) & ~1;
  }
  sp.attn_scale = a->attn_scale;
  sp.q_dtype = a->q_dtype;
  dim3 grid(sp.splits, hg.H_kv, a->B);
  if (a->mode == JF_MODE_K3V2) {
    // the query's type only matters where the query is read
    const int dt = a->scan_parts == JF_SCAN_V_ONLY ? JF_DTYPE_BF16 : a->q_dtype;
    if (dt == JF_DTYPE_BF16) {
      if (a->scan_parts == JF_SCAN_ALL) st = launch_k3v2<JF_DTYPE_BF16, 0>(sp, grid, stream);
      else if (a->scan_parts == JF_SCAN_K_ONLY) st = launch_k3v2<JF_DTYPE_BF16, 1>(sp, grid, stream);
      else st = launch_k3v2<JF_DTYPE_BF16, 2>(sp, grid, stream);
    } else {
      if (a->scan_parts == JF_SCAN_ALL) st = launch_k3v2<JF_DTYPE_FP16, 0>(sp, grid, stream);
      else st = launch_k3v2<JF_DTYPE_FP16, 1>(sp, grid, stream);
    }
  } else {
    st = launch_scan_k4v4(sp, a->stage_b == JF_STAGE_B_INT8P, a->scan_parts, grid, stream);
  }
  if (st != JF_OK) return st;
  if (a->scores && a->scan_parts != JF_SCAN_V_ONLY) {
    fill_neg_inf_tail_kernel<<<a->B * a->H_q, 256, 0, stream>>>(a->scores, a->seq_lens, a->H_q, a->max_S);
    JF_CUDA_TRY(cudaGetLastError());
  }
  return JF_OK;
}
