// Exact, deterministic top-k per query head over the scan's approximate scores.
//
// The reference selects with a 4-level radix select on fp32 scores that came out of a
// tensor-core accumulation (jetfire_vllm/csrc/int3_qk_scores.cu:426-554): which position
// wins near the k-th score depends on an unspecified summation order, and the output order
// and the choice among ties depend on atomics.  Here selection is two-tier:
//   1. a 2048-bin histogram (bin width 1/64 below an upper bound of the row maximum) of the
//      maxima of small groups of positions -- taken from the staged row, or, for long K3V2 rows,
//      the page-pair maxima the scan left -- finds a bin T at or below the k-th largest
//      approximate score (the k-th largest group maximum is a lower bound of it); rows the bins
//      do not fit get the k-th largest approximate score exactly from a radix select;
//   2. every position whose approximate score can still beat it -- bins <= T + ceil(2*delta*64)
//      + 1, with delta a bound on |approximate - canonical| (fp32 summation-order error only,
//      the scan dequantises with the reference's rounding) -- is re-scored in the canonical
//      arithmetic, and the k best by (canonical score desc, position asc) are emitted in
//      that order.
// The result is reproducible by a CPU and independent of tensor-core internals.  If the
// band does not fit the sort buffer (massive ties, degenerate scales) a slow exact path
// radix-selects on the 64-bit key (canonical score, ~position) computed on the fly.
// Slot translation and -1 padding follow csrc/int3_qk_scores.cu:399-417.
#include "finish_tail.cuh"

namespace jf {

namespace {

constexpr int kBins = 2048;
constexpr float kBinsPerUnit = 64.0f;

struct TopkParams {
  const float* scores;
  const float* pmax;      // K3V2: the scan's page maxima, [B][H_q][np_stride]
  const float* part_m;
  const float* part_smax;
  const void* q;
  const uint8_t* k_data;
  const uint16_t* k_scales;
  const int64_t* block_table;
  const int32_t* seq_lens;
  int64_t* topk_idx;
  int64_t* topk_slots;       // either may be null, not both
  int32_t* topk_slots_i32;
  int32_t* status;
  int64_t num_slots;
  int B, H_q, H_kv, G, max_S, max_blocks, splits, top_k, sort_n, q_dtype;
  int kv_shift;   // cache head = KV head >> kv_shift (see head_geom)
  int hm_chunks;  // score chunks whose per-float4 maxima fit the shared-memory side table (0: none)
  int np_stride;  // entries per row of pmax
  float attn_scale;
};

struct RowCtx {
  const float* q;         // smem, 128 floats (exact values of the query row)
  const int8_t* qi;       // smem, K4: quantised query
  const float* qs;        // smem, K4: per-32-channel query scales
  const uint8_t* k_rows;  // k_data of this KV head
  const uint16_t* k_sc;   // k_scales of this KV head
  const int64_t* bt;      // block-table row
  int64_t num_slots;
  float attn;
};

__device__ __forceinline__ int64_t slot_of(const RowCtx& c, int pos) {
  const int64_t blk = c.bt[pos >> 4];
  if (blk < 0 || blk >= (c.num_slots >> 4)) return -1;
  return blk * 16 + (pos & 15);
}

// Canonical K3 score, one warp per position.  k_hat = bf16(float(code - 4) * float(scale_bf16))
// as in jetfire_vllm/csrc/int3_qk_scores.cu:90-100.  Products of two 16-bit floats are exact
// in fp32; the canonical summation order is: lane l accumulates channels l, l+32, l+64, l+96
// with fma (ascending, from 0), then the 32 partials are added by a butterfly over lane
// distances 16, 8, 4, 2, 1.  Every lane returns the same value.  (The reference's own order is
// whatever its tensor-core instruction does; any fixed order stays inside its 2e-5 gate.)
// `row` = the 48 packed bytes (global or shared memory), `sw` = the two bf16 group scales.
__device__ __forceinline__ float canon_score_k3(const float* q, const uint8_t* row, uint32_t sw, float attn, int lane) {
  const int x = lane & 7;
  float part = 0.f;
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = 4 * r + (lane >> 3);  // INT3 group of channel 32 r + lane
    const uint32_t w24 = (static_cast<uint32_t>(row[i]) << 16) | (static_cast<uint32_t>(row[16 + i]) << 8) | row[32 + i];
    const float sc = (r < 2) ? __uint_as_float(sw << 16) : __uint_as_float(sw & 0xFFFF0000u);
    const int code = static_cast<int>((w24 >> (21 - 3 * x)) & 7u) - 4;
    const float kh = __bfloat162float(__float2bfloat16_rn(__fmul_rn(static_cast<float>(code), sc)));
    part = __fmaf_rn(q[32 * r + lane], kh, part);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xFFFFFFFFu, part, o));
  return __fmul_rn(part, attn);
}

// The same value as canon_score_k3, computed by EIGHT lanes per candidate (four candidates
// per warp): lane `sub` = lane & 7 owns the code at position sub of all 16 INT3 groups, i.e.
// channels 32 r + 8 m + sub, whose partial sums are the canonical order's lanes sub + 8 m.
// Code sub of a group is a 3-bit field of the 24-bit word (byte planes b0 b1 b2); for
// sub <= 4 it lies in the 16-bit window b0:b1, otherwise in b1:b2, so two PRMTs build the
// windows of four groups and one shift + mask leaves two codes at bit 0 of the two halves of a
// register.  Read as bf16 such a half is the subnormal code * 2^-133, and one packed fma with
// S = scale * 2^100 and C = -4 * 2^-133 * S yields 2^-33 * bf16_rn((code - 4) * scale) for both:
// a single rounding, and a power of two commutes with it (K scales between 2^-93 and 2^27, or
// zero -- the scan's dequantisation rests on the same identity).  `qv[4 r + m]` =
// 2^33 * q[32 r + 8 m + sub], so every product is the exact q * k_hat of the canonical order.
// Every lane of the warp must call this; lanes of a candidate get the same value.
__device__ __forceinline__ float canon_score_k3_x8(const float (&qv)[16], const uint32_t* row, float attn, int lane) {
  const int sub = lane & 7;
  const uint32_t sw = row[12];
  const uint32_t sc0 = prmt(sw, sw, 0x1010u), sc1 = prmt(sw, sw, 0x3232u);   // each group scale in both halves
  const uint32_t S0 = mul_bf16x2(sc0, 0x71807180u), C0 = mul_bf16x2(sc0, 0xB000B000u);   // * 2^100, * -2^-31
  const uint32_t S1 = mul_bf16x2(sc1, 0x71807180u), C1 = mul_bf16x2(sc1, 0xB000B000u);
  const bool early = sub <= 4;
  const int sh = early ? 13 - 3 * sub : 21 - 3 * sub;
  float part[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const uint32_t p0 = row[r], p1 = row[4 + r], p2 = row[8 + r];
    const uint32_t hi = early ? p0 : p1, lo = early ? p1 : p2;
    const uint32_t c01 = (prmt(lo, hi, 0x5140u) >> sh) & 0x00070007u;   // groups 4r, 4r+1
    const uint32_t c23 = (prmt(lo, hi, 0x7362u) >> sh) & 0x00070007u;   // groups 4r+2, 4r+3
    const uint32_t k01 = fma_bf16x2(c01, (r < 2) ? S0 : S1, (r < 2) ? C0 : C1);
    const uint32_t k23 = fma_bf16x2(c23, (r < 2) ? S0 : S1, (r < 2) ? C0 : C1);
    part[0] = __fmaf_rn(qv[4 * r], __uint_as_float(k01 << 16), part[0]);
    part[1] = __fmaf_rn(qv[4 * r + 1], __uint_as_float(k01 & 0xFFFF0000u), part[1]);
    part[2] = __fmaf_rn(qv[4 * r + 2], __uint_as_float(k23 << 16), part[2]);
    part[3] = __fmaf_rn(qv[4 * r + 3], __uint_as_float(k23 & 0xFFFF0000u), part[3]);
  }
  // butterfly distances 16 and 8 pair partials held by this lane, 4, 2, 1 pair lanes
  float t = __fadd_rn(__fadd_rn(part[0], part[2]), __fadd_rn(part[1], part[3]));
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) t = __fadd_rn(t, __shfl_xor_sync(0xFFFFFFFFu, t, o));
  return __fmul_rn(t, attn);
}

// Canonical K4/G128 score (jetfire_vllm/csrc/int8tc_qk_scores.cu:445-487): exact int32 dot per
// 32-channel block against the INT8 query, s = fma(float(acc_c), qs_c, s) for c = 0..3,
// * k_scale, * attn.  Lane l handles channels 4l..4l+3 (block l / 8).
__device__ __forceinline__ float canon_score_k4(const int8_t* qi, const float* qs, const uint8_t* row, float ks,
                                                float attn, int lane) {
  const uint32_t two = reinterpret_cast<const uint16_t*>(row)[lane];
  const int d = 4 * lane;
  int acc = (static_cast<int>((two >> 4) & 15u) - 8) * qi[d] + (static_cast<int>(two & 15u) - 8) * qi[d + 1] +
            (static_cast<int>((two >> 12) & 15u) - 8) * qi[d + 2] + (static_cast<int>((two >> 8) & 15u) - 8) * qi[d + 3];
  acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 1);
  acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 2);
  acc += __shfl_xor_sync(0xFFFFFFFFu, acc, 4);
  float s = 0.f;
#pragma unroll
  for (int blk = 0; blk < 4; ++blk)
    s = __fmaf_rn(static_cast<float>(__shfl_sync(0xFFFFFFFFu, acc, 8 * blk)), qs[blk], s);
  return __fmul_rn(__fmul_rn(s, ks), attn);
}

// Key: canonical score in the high word (order-preserving), ~position in the low word, so
// that a larger key is a better rank and equal scores prefer the lower position.
__device__ __forceinline__ uint64_t make_key(float s, int pos) {
  return (static_cast<uint64_t>(float_order_key(s)) << 32) | (0xFFFFFFFFu - static_cast<uint32_t>(pos));
}

// Key of a position straight from global memory (slow exact path only), whole warp.
template <int MODE>
__device__ __forceinline__ uint64_t canon_key_global(const RowCtx& c, int pos, int lane) {
  const int64_t slot = slot_of(c, pos);
  float s = -INFINITY;
  if (slot >= 0) {
    if (MODE == JF_MODE_K3V2)
      s = canon_score_k3(c.q, c.k_rows + slot * 48, *reinterpret_cast<const uint32_t*>(c.k_sc + slot * 2), c.attn, lane);
    else
      s = canon_score_k4(c.qi, c.qs, c.k_rows + slot * 64, bf16_bits_to_f32(c.k_sc[slot]), c.attn, lane);
  }
  return make_key(s, pos);
}

// Bin of a score: floor((top - s) * 64) clamped to [0, kBins - 1]; `top64` = top * 64.
// float -> int without a conversion instruction: adding 2^23 with round-toward-zero leaves
// floor(x) in the low mantissa bits (0 <= x < 2^11 here).
__device__ __forceinline__ float score_binf(float top64, float s) { return fmaf(s, -kBinsPerUnit, top64); }
__device__ __forceinline__ int score_bin(float top64, float s) {
  const float x = fminf(fmaxf(score_binf(top64, s), 0.0f), static_cast<float>(kBins - 1));
  return __float_as_int(__fadd_rz(x, 8388608.0f)) & (kBins - 1);
}

// candidates staged in shared memory per round: a top-k of 512 and its band in one (K4V4 has no band to speak of)
template <int MODE> struct RowChunk { static constexpr int v = (MODE == JF_MODE_K3V2) ? 768 : 576; };
constexpr int kChunkVec = 8;                   // float4 reads per thread and pass over a chunk
// 32-bit words per staged K row: K3V2 holds 12 of data and one of scales in a 64-byte slot (16-byte copies land aligned)
template <int MODE> struct RowWords { static constexpr int v = 16; };

struct SelSmemFixed {
  uint64_t bar;               // mbarrier of the score-chunk copy
  unsigned long long prefix;
  int hist[kBins];
  float q[JF_HEAD_DIM];
  float qs[4];
  int8_t qi[JF_HEAD_DIM];
  float w3[kSelWarps][3];
  float red[4];
  int wsum[kSelWarps];
  int ncand, tbin, remaining, pad_;
};

// What lives in the score chunk's shared memory once the candidates are collected.
template <int MODE>
struct SelSmemLate {
  union {   // the K rows are done with (canonical scores) before the finish stage starts
    TailSmem<MODE> tail;
    uint32_t rows[(MODE == JF_MODE_K3V2) ? RowChunk<MODE>::v * RowWords<MODE>::v : 4];   // K3V2: packed K rows + scales (K4V4 re-scores nothing)
  };
  uint32_t vrows[RowChunk<MODE>::v * TailSmem<MODE>::VW];  // packed V rows of the candidates (fused kernel)
  int64_t cand_slot[RowChunk<MODE>::v];
  uint32_t vsc[RowChunk<MODE>::v];                         // V scales
};

__host__ __device__ constexpr size_t hm_chunk_bytes(int nt) { return static_cast<size_t>(kChunkVec) * nt * 2; }   // side table of one chunk
constexpr size_t kSelSmemLimit = 227 * 1024;
// Bytes of the first shared-memory region: the resident score chunk (whose memory the late
// structures reuse), or -- lean kernel, which never stages the scores -- the late structures alone.
template <int MODE, bool LEAN, int NT>
__host__ __device__ constexpr size_t sel_region0_bytes() {
  constexpr size_t late = ((sizeof(SelSmemLate<MODE>) + 127) / 128) * 128;
  constexpr size_t chunk = static_cast<size_t>(4 * kChunkVec * NT) * 4;   // the resident chunk of an NT-wide block
  return LEAN ? late : (chunk > late ? chunk : late);
}
__host__ __device__ constexpr size_t sel_smem_bytes(size_t region0, int sort_n, int hm_chunks = 0, int nt = kSelThreads) {
  // region 0 | fixed | keys[sort_n] | cand_score[sort_n] | perm[sort_n] | bucket[sort_n] | hm16[hm_chunks]
  return region0 + sizeof(SelSmemFixed) + static_cast<size_t>(sort_n) * 8 +
         static_cast<size_t>(sort_n) * 4 + static_cast<size_t>(sort_n) * 4 + static_cast<size_t>(hm_chunks) * hm_chunk_bytes(nt);
}

// One CTA per (query head, batch element).  The row's approximate scores are pulled into
// shared memory by one bulk copy per 32768 positions, issued before anything else so that
// the prologue runs under it; every later pass over the scores reads shared memory.
// FUSED: the finish stage follows in the same kernel.
// LEAN (K3V2, long rows): the scores are never staged.  The scan left the largest score of every
// pair of 16-token pages next to them; the threshold comes from a histogram of those maxima (the
// K-th largest of them is a lower bound of the K-th largest score), and only the pairs whose
// maximum passes it are fetched -- a few hundred 128-byte reads instead of two passes over
// the row.  Rows the bins do not fit take the radix tier over global memory.
// NT: threads per block -- 1024, or (lean only) 512 with two blocks per multiprocessor, so that
// one row's chains of dependent memory round trips run under the other's arithmetic.
template <int MODE, int DT, bool FUSED, bool LEAN, int NT>
__global__ void __launch_bounds__(NT, kSelThreads / NT)
topk_select_kernel(const TopkParams p, const TailParams tp) {
  constexpr int kW = NT / 32;                   // warps of this block
  constexpr int kChunkPos = 4 * kChunkVec * NT; // positions per pass over a chunk
  constexpr int W = RowWords<MODE>::v;         // 32-bit words staged per candidate: data + scales
  constexpr size_t kRegion0 = sel_region0_bytes<MODE, LEAN, NT>();
  constexpr int kRowChunk = RowChunk<MODE>::v;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  float* chunk = reinterpret_cast<float*>(smem_raw);
  SelSmemLate<MODE>& late = *reinterpret_cast<SelSmemLate<MODE>*>(smem_raw);
  SelSmemFixed& sm = *reinterpret_cast<SelSmemFixed*>(smem_raw + kRegion0);
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw + kRegion0 + sizeof(SelSmemFixed));  // [sort_n]
  float* cand_score = reinterpret_cast<float*>(keys + p.sort_n);  // [sort_n] scan score per candidate
  uint16_t* perm = reinterpret_cast<uint16_t*>(cand_score + p.sort_n);             // [sort_n] rank -> candidate
  uint16_t* bucket = perm + p.sort_n;                                              // [sort_n] candidates grouped by bin
  // Rows of several chunks: an upper bound (16 bits of the order-preserving key, rounded up) of the
  // largest score of every float4 the histogram pass saw, [chunk][j][thread].  The collection then
  // fetches only the float4s that can hold a candidate instead of streaming the row a second time.
  uint16_t* hm16 = bucket + p.sort_n;
  int* hist = sm.hist;

  const int h = blockIdx.x, b = blockIdx.y;
  const int hkv = h / p.G, hi = h - hkv * p.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.top_k;
  const int64_t bh = static_cast<int64_t>(b) * p.H_q + h;
  const float* srow = p.scores + bh * p.max_S;
  const int64_t pbase = (static_cast<int64_t>(b) * p.H_kv + hkv) * p.splits;

  // ---- score chunks: bulk copy (16-byte aligned rows) or plain loads ----
  const bool vec = ((p.max_S & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.scores) & 15) == 0);
  uint32_t phase = 0;
  auto issue_chunk = [&](int ci) {  // the row's allocation covers max_S positions
    const int cnt = min(kChunkPos, p.max_S - ci * kChunkPos);
    if (vec) {
      if (tid == 0) {
        fence_proxy_async();
        mbar_expect_tx(&sm.bar, static_cast<uint32_t>(cnt) * 4u);
        bulk_g2s(chunk, srow + static_cast<int64_t>(ci) * kChunkPos, static_cast<uint32_t>(cnt) * 4u, &sm.bar);
      }
    } else {
      for (int i = tid; i < cnt; i += NT) chunk[i] = srow[static_cast<int64_t>(ci) * kChunkPos + i];
    }
  };
  // Block-wide; positions past the sequence read as -inf afterwards.  False (for every
  // thread) if the copy did not arrive within the wait's budget.
  auto wait_chunk = [&](int ci, int n) {
    bool ok = true;
    if (vec) {
      ok = mbar_wait(&sm.bar, phase);
      if (!ok) ok = mbar_wait(&sm.bar, phase);  // once more for the copy still in flight
      phase ^= 1u;
    }
    const int valid = max(0, min(n - ci * kChunkPos, kChunkPos));
    if (!vec) __syncthreads();
    for (int i = valid + tid; i < kChunkPos; i += NT) chunk[i] = -INFINITY;
    return __syncthreads_and(ok ? 1 : 0) != 0;
  };
  if (tid == 0) {
    mbar_init(&sm.bar, 1);
    fence_barrier_init();
  }
  // In the fused call this kernel directly follows the scan, and what the scan itself read (the
  // query, the sequence lengths) was complete before the scan started: the query model and the
  // zeroing below need nothing of the scan's output and run while the scan's last CTAs finish.
  // The stand-alone select may follow any kernel, so there the wait comes first.
  if (!FUSED) pdl_wait();
  uint16_t q_bits = 0;
  if (tid < JF_HEAD_DIM) q_bits = reinterpret_cast<const uint16_t*>(p.q)[bh * JF_HEAD_DIM + tid];
  const int n_seq_raw = p.seq_lens[b];
  const int n_seq = min(n_seq_raw, p.max_S);
  int64_t* out_idx = p.topk_idx + bh * K;
  int64_t* out_slot = p.topk_slots ? p.topk_slots + bh * K : nullptr;
  int32_t* out_slot32 = p.topk_slots_i32 ? p.topk_slots_i32 + bh * K : nullptr;

  // ---- query row (exact values), per-group L1 norms, INT8 model for K4 ----
  if (tid < JF_HEAD_DIM) sm.q[tid] = Elem<DT>::to_f32(q_bits);
  __syncthreads();
  if (warp < 4) {  // warp w handles channels 32w..32w+31
    const float v = sm.q[32 * warp + lane];
    float a = fabsf(v), s1 = fabsf(v) + 0.001953125f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
      s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, o);
    }
    if (MODE == JF_MODE_K4V4) {
      const float qs = fmaxf(__fdiv_rn(a, 127.0f), 1e-12f);
      const float inv = __fdiv_rn(1.0f, qs);
      const int qv = max(-128, min(127, __float2int_rn(__fmul_rn(v, inv))));
      sm.qi[32 * warp + lane] = static_cast<int8_t>(qv);
      if (lane == 0) sm.qs[warp] = qs;
    }
    if (lane == 0) sm.red[warp] = s1;
  }
  if (tid == 0) { sm.ncand = 0; sm.tbin = -1; }
  for (int i = tid; i < kBins; i += NT) hist[i] = 0;
  for (int i = tid; i < p.sort_n; i += NT) keys[i] = 0ull;

  // what this block reads first once the scan is done: warm the address translations now
  if (FUSED && warp == 0) {
    const void* first = p.part_m + pbase * kHeadsPad;
    if (lane == 1) first = p.part_smax + pbase * 2;
    if (lane == 2) first = tp.part_l + pbase * kHeadsPad;
    if (lane == 3) first = tp.part_o + pbase * (kHeadsPad * JF_HEAD_DIM);
    if (lane == 4) first = srow;
    if (lane == 5) first = LEAN ? static_cast<const void*>(p.pmax + bh * p.np_stride) : static_cast<const void*>(srow + p.max_S - 1);
    if (lane == 6) first = p.block_table + static_cast<int64_t>(b) * p.max_blocks;
    if (lane == 7) first = out_idx;
    if (lane < 8) prefetch_l2(first);
  }

  // ---- the scan's results: split statistics first (small), then the 128 KB score chunk ----
  if (FUSED) pdl_wait();
  float top = kMinusBig, sm0 = 0.f, sm1 = 0.f;
  if (tid < p.splits) {  // the first split of this thread; the loop below takes the rest
    top = p.part_m[(pbase + tid) * kHeadsPad + hi];
    sm0 = p.part_smax[(pbase + tid) * 2];
    sm1 = p.part_smax[(pbase + tid) * 2 + 1];
  }
  SplitPre<NT> pre;
  if (FUSED) split_preload<NT>(tp, pbase, hi, tid, pre);
  // lean: the scan's maxima of groups of pages -- K3V2: pairs of pages, K4V4: single pages
  constexpr int kGroupPages = (MODE == JF_MODE_K3V2) ? 2 : 1;
  const int n_pages = (n_seq + 15) >> 4, n_groups = (n_pages + kGroupPages - 1) / kGroupPages;
  const float4* pm4 = reinterpret_cast<const float4*>(p.pmax + bh * p.np_stride);
  if (!LEAN) issue_chunk(0);
  {
    for (int s = tid + NT; s < p.splits; s += NT) {
      top = fmaxf(top, p.part_m[(pbase + s) * kHeadsPad + hi]);
      sm0 = fmaxf(sm0, p.part_smax[(pbase + s) * 2]);
      sm1 = fmaxf(sm1, p.part_smax[(pbase + s) * 2 + 1]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      top = fmaxf(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
      sm0 = fmaxf(sm0, __shfl_xor_sync(0xFFFFFFFFu, sm0, o));
      sm1 = fmaxf(sm1, __shfl_xor_sync(0xFFFFFFFFu, sm1, o));
    }
    if (lane == 0) { sm.w3[warp][0] = top; sm.w3[warp][1] = sm0; sm.w3[warp][2] = sm1; }
  }
  __syncthreads();

  RowCtx ctx;
  ctx.q = sm.q; ctx.qi = sm.qi; ctx.qs = sm.qs;
  const ModeInfo mi = mode_info(MODE);
  ctx.k_rows = p.k_data + static_cast<int64_t>(hkv >> p.kv_shift) * p.num_slots * mi.k_row;
  ctx.k_sc = p.k_scales + static_cast<int64_t>(hkv >> p.kv_shift) * p.num_slots * mi.ng;
  ctx.bt = p.block_table + static_cast<int64_t>(b) * p.max_blocks;
  ctx.num_slots = p.num_slots;
  ctx.attn = p.attn_scale;

  float row_max = kMinusBig;  // max over the splits of the scan's reference points
#pragma unroll
  for (int w = 0; w < kW; ++w) row_max = fmaxf(row_max, sm.w3[w][0]);

  // the copy issued at the top must have landed before its shared memory is reused
  bool copied = LEAN ? true : wait_chunk(0, n_seq);
  if (!copied && tid == 0) report_status(p.status, JF_ERR_TIMEOUT);
  if (LEAN && p.status[4] != kPageMaxTag) {   // the scan before this call left no page maxima: arguments do not match
    if (tid == 0) report_status(p.status, JF_ERR_STATE);
    copied = false;
  }
  const int n = copied ? n_seq : 0;   // a row whose scores did not arrive selects nothing

  int m_sel = 0;  // entries of keys[] that hold the ranked result
  bool prefetch = false;
  if (n > 0) {
    int ncand = 0;
    int cand_last = kBins;  // bound on the candidates' canonical-score bin, when one is known
    bool slow = false;

    if (n <= p.sort_n) {
      // short row: every position is a candidate
      for (int i = tid; i < n; i += NT) { keys[i] = static_cast<uint64_t>(i); cand_score[i] = LEAN ? srow[i] : chunk[i]; }
      ncand = n;
    } else {
      float sm0 = 0.f, sm1 = 0.f;
#pragma unroll
      for (int w = 0; w < kW; ++w) { sm0 = fmaxf(sm0, sm.w3[w][1]); sm1 = fmaxf(sm1, sm.w3[w][2]); }
      const float top = row_max + 4.0f;  // the scan lets its reference point lag the true maximum by at most 4
      const float top64 = top * kBinsPerUnit;
      float delta = 0.f;
      if (MODE == JF_MODE_K3V2) {
        // The scan and the canonical order add the same exact products q_d * k_hat_d in fp32,
        // in different orders: each stays within (roundings) * 2^-24 * sum|q_d k_hat_d| of the
        // exact sum (canonical: 9 roundings; tensor core: one per k-step, 8, possibly
        // truncating).  sum|q_d k_hat_d| <= sum_g 3 * scale_g * sum_{d in g} |q_d|.  A factor 32
        // covers both paths with slack; the last term covers the final multiply by attn_scale.
        const float q1a = sm.red[0] + sm.red[1], q1b = sm.red[2] + sm.red[3];
        const float mag = fabsf(p.attn_scale) * (sm0 * q1a + sm1 * q1b) * 3.0f;
        delta = mag * (32.0f / 16777216.0f) + mag * (4.0f / 16777216.0f) + 1e-7f;
      }
      float nbf = ceilf(2.0f * delta * kBinsPerUnit) + 1.0f;
      if (!(nbf < 4096.0f)) nbf = 4096.0f;
      const int nb = (MODE == JF_MODE_K3V2) ? static_cast<int>(nbf) : 0;  // K4: scan scores are canonical
      const int n_chunks = (n + kChunkPos - 1) / kChunkPos;
      const float4* chunk4 = reinterpret_cast<const float4*>(chunk);
      // element (j, c) of thread tid is chunk position 4 * (j * 1024 + tid) + c
      auto next_chunk = [&](int ci) {  // block-wide: replace the resident chunk by chunk ci
        __syncthreads();
        issue_chunk(ci);
        if (!wait_chunk(ci, n)) { copied = false; }
      };

      // Block-wide: turns hist[] into inclusive prefix counts (from the top bin down) and
      // leaves in sm.tbin the bin where the count reaches `want` (-1: never).
      auto scan_hist = [&](int want) {
        constexpr int kPer = kBins / NT;   // consecutive bins per thread
        int hv[kPer];
        int v = 0;
#pragma unroll
        for (int i = 0; i < kPer; ++i) { hv[i] = hist[kPer * tid + i]; v += hv[i]; }
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
          if (lane >= o) incl += t;
        }
        if (lane == 31) sm.wsum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
          int t = (lane < kW) ? sm.wsum[lane] : 0, inc2 = t;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xFFFFFFFFu, inc2, o);
            if (lane >= o) inc2 += u;
          }
          if (lane < kW) sm.wsum[lane] = inc2 - t;  // exclusive prefix of the warp totals
        }
        __syncthreads();
        int run = sm.wsum[warp] + incl - v;   // count in the bins above this thread's
#pragma unroll
        for (int i = 0; i < kPer; ++i) {
          if (run < want && run + hv[i] >= want) sm.tbin = kPer * tid + i;
          run += hv[i];
          hist[kPer * tid + i] = run;
        }
        __syncthreads();
      };
      // Block-wide: positions whose score passes the test against `thr` (kind 0: greater, 1: greater
      // or equal, 2: equal) go to keys[off0 ...], in position order (offsets from a warp scan and a
      // block scan, no atomics); entries at or past `cap` are dropped.  Returns how many passed.
      float hm[kChunkVec];  // per float4 of the resident chunk: its largest score (tier 1a's pass)
      bool have_hm = false;
      auto collect = [&](float thr, int kind, int off0, int cap, bool use16 = false) {
        int running = 0;  // candidates found in earlier chunks
        const uint32_t thr16 = float_order_key(thr) >> 16;
        const bool glob = LEAN || use16;   // the scores come straight from memory
        for (int ci = 0; ci < n_chunks; ++ci) {
          if (n_chunks > 1 && !glob) next_chunk(ci);
          uint32_t mask = 0u;
          // which of the thread's float4s can hold a candidate at all (branch-free; most threads
          // find none and skip the loads altogether)
          uint32_t hits = (1u << kChunkVec) - 1u;
          if (LEAN) {
#pragma unroll
            for (int j = 0; j < kChunkVec; ++j)
              if (ci * kChunkPos + 4 * (j * NT + tid) >= n) hits &= ~(1u << j);
          } else if (have_hm && kind == 0) {
            hits = 0u;
#pragma unroll
            for (int j = 0; j < kChunkVec; ++j) hits |= static_cast<uint32_t>(hm[j] > thr) << j;
          } else if (use16) {
            hits = 0u;
#pragma unroll
            for (int j = 0; j < kChunkVec; ++j)
              hits |= static_cast<uint32_t>(hm16[(ci * kChunkVec + j) * NT + tid] >= thr16) << j;
          }
          while (hits) {
            const int j = __ffs(hits) - 1;
            hits &= hits - 1u;
            float4 v;
            if (glob) {    // straight from memory; positions at or past the length read as -inf
              const int pos = ci * kChunkPos + 4 * (j * NT + tid);
              v = *reinterpret_cast<const float4*>(srow + pos);
              if (pos >= n) v.x = -INFINITY;
              if (pos + 1 >= n) v.y = -INFINITY;
              if (pos + 2 >= n) v.z = -INFINITY;
              if (pos + 3 >= n) v.w = -INFINITY;
            } else {
              v = chunk4[j * NT + tid];
            }
            uint32_t m4;
            if (kind == 0)
              m4 = static_cast<uint32_t>(v.x > thr) | (static_cast<uint32_t>(v.y > thr) << 1) |
                   (static_cast<uint32_t>(v.z > thr) << 2) | (static_cast<uint32_t>(v.w > thr) << 3);
            else if (kind == 1)
              m4 = static_cast<uint32_t>(v.x >= thr) | (static_cast<uint32_t>(v.y >= thr) << 1) |
                   (static_cast<uint32_t>(v.z >= thr) << 2) | (static_cast<uint32_t>(v.w >= thr) << 3);
            else
              m4 = static_cast<uint32_t>(v.x == thr) | (static_cast<uint32_t>(v.y == thr) << 1) |
                   (static_cast<uint32_t>(v.z == thr) << 2) | (static_cast<uint32_t>(v.w == thr) << 3);
            mask |= m4 << (4 * j);
          }
          const int cnt = __popc(mask);
          int incl = cnt;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
          }
          // warp totals -> every warp's offset (no atomics: 32 same-address atomics with a
          // return value cost more than the whole pass)
          __syncthreads();   // the previous round's (or caller's) reads of wsum are done
          if (lane == 31) sm.wsum[warp] = incl;
          __syncthreads();
          int wt = (lane < kW) ? sm.wsum[lane] : 0, winc = wt;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, winc, o);
            if (lane >= o) winc += t;
          }
          const int base = running + __shfl_sync(0xFFFFFFFFu, winc - wt, warp);
          running += __shfl_sync(0xFFFFFFFFu, winc, 31);
          int o = off0 + base + incl - cnt;
          while (mask) {
            const int e = __ffs(mask) - 1;
            mask &= mask - 1u;
            const int at = 4 * ((e >> 2) * NT + tid) + (e & 3);
            if (o < cap) {
              keys[o] = static_cast<uint64_t>(ci * kChunkPos + at);
              cand_score[o] = glob ? srow[ci * kChunkPos + at] : chunk[at];
            }
            ++o;
          }
        }
        __syncthreads();
        return running;
      };

      const bool use_hm16 = vec && n_chunks > 1 && n_chunks <= p.hm_chunks;
      // ---- tier 1a: a bound from group maxima.  Each thread holds four groups of positions
      //      per chunk (stride 4096 inside a group); the K-th largest group maximum is a lower
      //      bound of the K-th largest score, and far fewer values enter the histogram. ----
      for (int ci = 0; !LEAN && ci < n_chunks; ++ci) {
        if (ci > 0) next_chunk(ci);
        float gm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < kChunkVec; ++j) {
          const float4 v = chunk4[j * NT + tid];
          gm[0] = fmaxf(gm[0], v.x); gm[1] = fmaxf(gm[1], v.y); gm[2] = fmaxf(gm[2], v.z); gm[3] = fmaxf(gm[3], v.w);
          hm[j] = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
          if (use_hm16) {
            const uint32_t k32 = float_order_key(hm[j]);
            hm16[(ci * kChunkVec + j) * NT + tid] =
                static_cast<uint16_t>(min(0xFFFFu, (k32 >> 16) + ((k32 & 0xFFFFu) ? 1u : 0u)));
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (gm[c] > -INFINITY) atomicAdd(&hist[score_bin(top64, gm[c])], 1);
      }
      have_hm = !LEAN && n_chunks == 1;  // hm[] describes the chunk that stays resident
      if (LEAN) {
        // the groups are the scan's; their maxima came with it.  +inf marks a K4V4 page whose
        // maximum is not known (it is always fetched below) and does not count here; groups past
        // the sequence were never written.
        for (int i4 = tid; 4 * i4 < n_groups; i4 += NT) {
          const float4 v = pm4[i4];
          const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (4 * i4 + c < n_groups && e[c] > -INFINITY && e[c] < INFINITY) atomicAdd(&hist[score_bin(top64, e[c])], 1);
        }
      }
      __syncthreads();
      scan_hist(K);
      bool ok = false;
      {
        const int tbin = sm.tbin;
        const int last = tbin + nb;
        if (tbin >= 0 && last < kBins - 1) {
          // bin <= last  <=>  fma(s, -64, top64) < last + 1; one comparison per score against a
          // threshold a little below the exact boundary (a few extra candidates are harmless)
          const float xlim = static_cast<float>(last + 1);
          const float thr = (top64 - xlim) * (1.0f / kBinsPerUnit) - (fabsf(top64) + xlim) * (1.0f / (kBinsPerUnit * 2097152.0f)) - 1e-30f;
          int total;
          if (LEAN) {
            // The pages of the pairs whose maximum passes the threshold go to a list (every such
            // pair holds a candidate, so more pairs than the sort buffer has entries means the row
            // does not fit); then one thread per listed page fetches its sixteen scores (64 bytes, four
            // independent loads) and appends the ones that pass.  Offsets come from one
            // shared-memory atomic per warp: the order of the candidates in the buffer is not
            // fixed, the ranking below does not depend on it.
            uint16_t* page_list = perm;   // perm and bucket, contiguous: 2 * sort_n entries
            const int list_cap = 2 * p.sort_n;
            for (int b4 = 0; 4 * b4 < n_groups; b4 += NT) {   // the same trip count for every thread
              const int i4 = b4 + tid;
              uint32_t flags = 0u;   // kGroupPages bits per group: its pages that exist
              if (4 * i4 < n_groups) {
                const float4 v = pm4[i4];
                const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  const int pg = kGroupPages * (4 * i4 + c);
                  if (4 * i4 + c < n_groups && e[c] > thr)
                    flags |= ((kGroupPages == 2 && pg + 1 < n_pages) ? 3u : 1u) << (kGroupPages * c);
                }
              }
              const int cnt = __popc(flags);
              int incl = cnt;
#pragma unroll
              for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                if (lane >= o) incl += t;
              }
              int base = 0;
              if (lane == 31 && incl > 0) base = atomicAdd(&sm.ncand, incl);
              int o = __shfl_sync(0xFFFFFFFFu, base, 31) + incl - cnt;
              while (flags) {
                const int i = __ffs(flags) - 1;   // bit i: page kGroupPages * 4 * i4 + i
                flags &= flags - 1u;
                if (o < list_cap) page_list[o] = static_cast<uint16_t>(kGroupPages * 4 * i4 + i);
                ++o;
              }
            }
            __syncthreads();
            const int n_list = sm.ncand;
            __syncthreads();
            if (tid == 0) sm.ncand = 0;
            __syncthreads();
            if (n_list <= list_cap) {
              // the listed pages come into the (still unused) late region with asynchronous copies,
              // all in flight at once: one trip to the scores instead of one per round of threads
              float* stage = reinterpret_cast<float*>(smem_raw);
              constexpr int kStageCap = static_cast<int>(sizeof(SelSmemLate<MODE>) / 64);
              for (int b0 = 0; b0 < n_list; b0 += kStageCap) {
                const int nb = min(kStageCap, n_list - b0);
                for (int u = tid; u < 4 * nb; u += NT) {
                  const int l = u >> 2, q4 = u & 3;
                  cp_async_16(stage + 16 * l + 4 * q4, srow + 16 * static_cast<int>(page_list[b0 + l]) + 4 * q4);
                }
                cp_async_commit();
                cp_async_wait_all();
                __syncthreads();
                for (int lb = 0; lb < nb; lb += NT) {
                  const int l = lb + tid;
                  uint32_t m16 = 0u;
                  int pos0 = 0;
                  if (l < nb) {
                    pos0 = 16 * static_cast<int>(page_list[b0 + l]);
                    // the four float4s of the page, starting at a different one in neighbouring
                    // threads: the pages lie 64 bytes apart, and read in step they would collide
                    // on two groups of banks
                    const float4* s4 = reinterpret_cast<const float4*>(stage + 16 * l);
                    const int rot = (l >> 1) & 3;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      const int q4 = (j + rot) & 3;
                      const float4 v = s4[q4];
                      const uint32_t m4 = static_cast<uint32_t>(v.x > thr) | (static_cast<uint32_t>(v.y > thr) << 1) |
                                          (static_cast<uint32_t>(v.z > thr) << 2) | (static_cast<uint32_t>(v.w > thr) << 3);
                      m16 |= m4 << (4 * q4);
                    }
                    const int live = n - pos0;   // tokens of the page inside the sequence
                    if (live < 16) m16 &= (1u << max(live, 0)) - 1u;
                  }
                  const int cnt = __popc(m16);
                  int incl = cnt;
#pragma unroll
                  for (int o = 1; o < 32; o <<= 1) {
                    const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
                    if (lane >= o) incl += t;
                  }
                  int base = 0;
                  if (lane == 31 && incl > 0) base = atomicAdd(&sm.ncand, incl);
                  int o = __shfl_sync(0xFFFFFFFFu, base, 31) + incl - cnt;
                  while (m16) {   // one candidate per listed page, as a rule
                    const int t = __ffs(m16) - 1;
                    m16 &= m16 - 1u;
                    if (o < p.sort_n) { keys[o] = static_cast<uint64_t>(pos0 + t); cand_score[o] = stage[16 * l + t]; }
                    ++o;
                  }
                }
                __syncthreads();
              }
              total = sm.ncand;
            } else {
              total = n_list;   // too many: the row does not fit this tier
            }
            __syncthreads();
          } else {
            total = collect(thr, 0, 0, p.sort_n, use_hm16);
          }
          ok = total <= p.sort_n;
          ncand = total;
          cand_last = last + nb;
        }
      }
      if (!ok) {
        // ---- tier 1b (rows the fixed bins do not fit: a score far above the rest, scores packed
        //      closer than a bin, or too many in the band): the K-th largest approximate score
        //      EXACTLY, by a radix select over the order-preserving keys of the resident scores --
        //      three levels of 11, 11 and 10 bits, each one pass over shared memory -- and then
        //      the positions at or above it (minus the band for K3V2).  Independent of the range and
        //      the spacing of the scores, and a few passes over the row at most. ----
        have_hm = false;
        uint32_t prefix = 0u;
        int want = K;
        for (int level = 0; level < 3; ++level) {
          const int bits = (level == 2) ? 10 : 11, shift = (level == 0) ? 21 : (level == 1) ? 10 : 0;
          const uint32_t dmask = (1u << bits) - 1u;
          __syncthreads();
          if (tid == 0) sm.tbin = -1;
          for (int i = tid; i < kBins; i += NT) hist[i] = 0;
          __syncthreads();
          for (int ci = 0; ci < n_chunks; ++ci) {
            if (n_chunks > 1 && !LEAN) next_chunk(ci);
#pragma unroll
            for (int j = 0; j < kChunkVec; ++j) {
              float4 v;
              if (LEAN) {
                const int pos = ci * kChunkPos + 4 * (j * NT + tid);
                v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
                if (pos < n) {
                  v = *reinterpret_cast<const float4*>(srow + pos);
                  if (pos + 1 >= n) v.y = -INFINITY;
                  if (pos + 2 >= n) v.z = -INFINITY;
                  if (pos + 3 >= n) v.w = -INFINITY;
                }
              } else {
                v = chunk4[j * NT + tid];
              }
              const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                if (e[c] > -INFINITY) {
                  const uint32_t key = float_order_key(e[c]);
                  // larger keys first: digit d goes to bin kBins - 1 - d
                  if (level == 0 || (key >> (shift + bits)) == prefix)
                    atomicAdd(&hist[kBins - 1 - static_cast<int>((key >> shift) & dmask)], 1);
                }
              }
            }
          }
          __syncthreads();
          scan_hist(want);
          const int tb = max(sm.tbin, 0);
          want -= (tb > 0) ? hist[tb - 1] : 0;   // hist[] now holds inclusive counts from the top bin down
          prefix = (prefix << bits) | static_cast<uint32_t>(kBins - 1 - tb);
        }
        const float kth = float_from_order_key(prefix);   // the K-th largest approximate score
        __syncthreads();
        for (int i = tid; i < p.sort_n; i += NT) keys[i] = 0ull;
        __syncthreads();
        if (MODE == JF_MODE_K4V4) {
          // the scores are canonical: everything above the K-th, then the lowest positions among
          // those equal to it (the collection runs in position order) -- exactly K candidates
          const int n_gt = collect(kth, 0, 0, p.sort_n);
          collect(kth, 2, n_gt, K);
          ncand = K;
        } else {
          const int total = collect(kth - 2.0f * delta - 1e-30f, 1, 0, p.sort_n);
          if (total > p.sort_n) slow = true;   // more scores inside the band than the sort buffer holds: massive ties
          ncand = min(total, p.sort_n);
        }
        cand_last = kBins;
      }
      if (!copied) {  // a later chunk did not arrive: select nothing
        if (tid == 0) report_status(p.status, JF_ERR_TIMEOUT);
        ncand = 0;
        slow = false;
      }
    }
    __syncthreads();   // every read of the score chunk is done: its memory is reused from here on

    // the fused finish stage takes slots, scores and V rows of the candidates from shared memory
    prefetch = FUSED && !slow && ncand <= kRowChunk && p.sort_n <= kSelThreads;
    if (!slow) {
      // ---- re-score the candidates canonically: slots, then their packed rows into shared
      //      memory with independent 16-byte loads, then the canonical arithmetic ----
      for (int base = 0; base < ncand; base += kRowChunk) {
        const int cn = min(kRowChunk, ncand - base);
        for (int c = tid; c < cn; c += NT) late.cand_slot[c] = slot_of(ctx, static_cast<int>(keys[base + c]));
        __syncthreads();
        {
          // Every candidate's packed K row and scales (K3V2) and, when the finish stage will use
          // them, its V row and scales, as asynchronous 16- and 4-byte copies: the K side in
          // kGroups groups of candidates, the V side as a last group.  The canonical scores of a
          // group are computed while the later groups are still on their way.
          constexpr int kGroups = 3;
          constexpr int VW = TailSmem<MODE>::VW;
          constexpr int kVParts = VW / 4;
          const uint8_t* v_rows = tp.v_data + static_cast<int64_t>(hkv >> p.kv_shift) * p.num_slots * mi.v_row;
          const uint16_t* v_sc = tp.v_scales + static_cast<int64_t>(hkv >> p.kv_shift) * p.num_slots * mi.ng;
          const int per = (cn + kGroups - 1) / kGroups;
          if (MODE == JF_MODE_K3V2) {
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
              const int c_lo = g * per, c_n = max(0, min(cn, c_lo + per) - c_lo);
              for (int u = tid; u < 4 * c_n; u += NT) {
                const int c = c_lo + (u >> 2), part = u & 3;
                const int64_t slot = late.cand_slot[c];
                uint32_t* r = late.rows + c * W;
                if (part < 3) {
                  if (slot >= 0) cp_async_16(r + 4 * part, ctx.k_rows + slot * 48 + 16 * part);
                  else *reinterpret_cast<uint4*>(r + 4 * part) = make_uint4(0u, 0u, 0u, 0u);
                } else {
                  if (slot >= 0) cp_async_4(r + 12, ctx.k_sc + slot * 2);
                  else r[12] = 0u;
                }
              }
              cp_async_commit();
            }
          }
          if (prefetch) {
            for (int u = tid; u < 4 * cn; u += NT) {
              const int c = u >> 2, part = u & 3;
              const int64_t slot = late.cand_slot[c];
              if (part < kVParts) {
                uint4* dst = reinterpret_cast<uint4*>(late.vrows + c * VW) + part;
                if (slot >= 0) cp_async_16(dst, reinterpret_cast<const uint4*>(v_rows + slot * (16 * kVParts)) + part);
                else *dst = make_uint4(0u, 0u, 0u, 0u);
              }
              // the scales: K3V2 both groups' (4 bytes); K4V4 the aligned 4-byte pair that holds the 2-byte scale
              if (part == ((MODE == JF_MODE_K3V2) ? 2 : 0)) {
                if (slot < 0) late.vsc[c] = 0u;
                else if (MODE == JF_MODE_K3V2) cp_async_4(&late.vsc[c], v_sc + slot * 2);
                else cp_async_4(&late.vsc[c], v_sc + (slot & ~static_cast<int64_t>(1)));
              }
            }
          }
          cp_async_commit();
          if (MODE == JF_MODE_K4V4) {
            // K4: the scan's score is the canonical one bit for bit (exact integer dot products,
            // the same fp32 rescale order), so nothing is recomputed
            for (int c = tid; c < cn; c += NT) {
              const int pos = static_cast<int>(keys[base + c]);
              keys[base + c] = make_key(late.cand_slot[c] >= 0 ? cand_score[base + c] : -INFINITY, pos);
            }
          } else {
            // eight lanes per candidate, four candidates per warp and round
            float qv[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) qv[i] = sm.q[32 * (i >> 2) + 8 * (i & 3) + (lane & 7)] * 8589934592.0f;   // 2^33, see canon_score_k3_x8
#pragma unroll
            for (int g = 0; g < kGroups; ++g) {
              // groups 0..g have landed once at most (kGroups - 1 - g) K groups and the V group are in flight
              if (g == 0) cp_async_wait_group<kGroups>();
              else if (g == 1) cp_async_wait_group<kGroups - 1>();
              else cp_async_wait_group<kGroups - 2>();
              __syncthreads();
              const int c_lo = g * per, c_hi = min(cn, c_lo + per);
              for (int c0 = c_lo + 4 * warp; c0 < c_hi; c0 += 4 * kW) {
                const int c = c0 + (lane >> 3);
                const int cc = min(c, c_hi - 1);        // lanes past the end keep the shuffles company
                const float s = canon_score_k3_x8(qv, late.rows + cc * W, ctx.attn, lane);
                if (c < c_hi && (lane & 7) == 0)
                  keys[base + c] = make_key(late.cand_slot[c] >= 0 ? s : -INFINITY, static_cast<int>(keys[base + c]));
              }
            }
          }
        }
        __syncthreads();
      }
    } else {
      // ---- slow exact path: 8-level radix select on the 64-bit canonical key ----
      if (tid == 0) { sm.prefix = 0ull; sm.remaining = K; sm.ncand = 0; }
      __syncthreads();
      for (int level = 7; level >= 0; --level) {
        for (int i = tid; i < 256; i += NT) hist[i] = 0;
        __syncthreads();
        const unsigned long long prefix = sm.prefix;
        for (int i = warp; i < n; i += kW) {
          const uint64_t key = canon_key_global<MODE>(ctx, i, lane);
          const bool match = (level == 7) || ((key >> (8 * (level + 1))) == prefix);
          if (match && lane == 0) atomicAdd(&hist[(key >> (8 * level)) & 255u], 1);
        }
        __syncthreads();
        if (tid == 0) {
          int cum = 0, rem = sm.remaining, cb = 0;
          for (int bin = 255; bin >= 0; --bin) {
            if (cum + hist[bin] >= rem) { cb = bin; break; }
            cum += hist[bin];
          }
          sm.remaining = rem - cum;
          sm.prefix = (prefix << 8) | static_cast<unsigned long long>(cb);
        }
        __syncthreads();
      }
      const unsigned long long tkey = sm.prefix;  // key of the k-th best; keys are unique
      for (int i = tid; i < p.sort_n; i += NT) keys[i] = 0ull;
      __syncthreads();
      for (int i = warp; i < n; i += kW) {
        const uint64_t key = canon_key_global<MODE>(ctx, i, lane);
        if (key >= tkey && lane == 0) {
          const int pos = atomicAdd(&sm.ncand, 1);
          if (pos < p.sort_n) keys[pos] = key;
        }
      }
      __syncthreads();
      ncand = min(sm.ncand, p.sort_n);
    }
    __syncthreads();

    // ---- order the candidates: best first ----
    if (p.sort_n <= kSelThreads) {
      // Rank by buckets: a candidate's rank is the number of candidates in finer score bins
      // above its own plus the number of larger keys inside its bin.  Bins are `f` times finer
      // than the selection histogram's (the candidates span few of those); a larger canonical
      // score never lands in a later bin, so the result is the exact order of the keys, and
      // crowded bins (massive ties) only cost time.  A thread owns candidates tid, tid + NT, ...
      constexpr int kCand = kSelThreads / NT;
      int f = 1;
      while (f < 16 && (cand_last + 2) * f * 2 <= kBins) f *= 2;
      const float fscale = kBinsPerUnit * static_cast<float>(f);
      const float ftop = (row_max + 4.0f) * fscale;
      for (int i = tid; i < kBins; i += NT) hist[i] = 0;
      __syncthreads();
      unsigned long long mine[kCand];
      int fb[kCand], arrival[kCand];
#pragma unroll
      for (int k = 0; k < kCand; ++k) {
        const int c = tid + k * NT;
        mine[k] = 0ull; fb[k] = 0; arrival[k] = 0;
        if (c < ncand) {
          mine[k] = keys[c];
          const float sc = float_from_order_key(static_cast<uint32_t>(mine[k] >> 32));
          const float x = fminf(fmaxf(fmaf(sc, -fscale, ftop), 0.0f), static_cast<float>(kBins - 1));
          fb[k] = __float_as_int(__fadd_rz(x, 8388608.0f)) & (kBins - 1);
          arrival[k] = atomicAdd(&hist[fb[k]], 1);
        }
      }
      __syncthreads();
      {
        // exclusive prefix over the bins, kPer per thread, written back in place
        constexpr int kPer = kBins / NT;
        int hv[kPer];
        int v = 0;
#pragma unroll
        for (int i = 0; i < kPer; ++i) { hv[i] = hist[kPer * tid + i]; v += hv[i]; }
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
          if (lane >= o) incl += t;
        }
        if (lane == 31) sm.wsum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
          int t = (lane < kW) ? sm.wsum[lane] : 0, inc2 = t;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xFFFFFFFFu, inc2, o);
            if (lane >= o) inc2 += u;
          }
          if (lane < kW) sm.wsum[lane] = inc2 - t;
        }
        __syncthreads();
        int run = sm.wsum[warp] + incl - v;
#pragma unroll
        for (int i = 0; i < kPer; ++i) { hist[kPer * tid + i] = run; run += hv[i]; }
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < kCand; ++k) {
        const int c = tid + k * NT;
        if (c < ncand) bucket[hist[fb[k]] + arrival[k]] = static_cast<uint16_t>(c);
      }
      __syncthreads();
      int r[kCand];
#pragma unroll
      for (int k = 0; k < kCand; ++k) {
        r[k] = 0;
        if (tid + k * NT < ncand) {
          const int lo = hist[fb[k]], hi2 = (fb[k] == kBins - 1) ? ncand : hist[fb[k] + 1];
          int above = 0;
          for (int m = lo; m < hi2; ++m) above += (keys[bucket[m]] > mine[k]) ? 1 : 0;
          r[k] = min(lo + above, ncand - 1);
        }
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < kCand; ++k) {
        const int c = tid + k * NT;
        if (c < ncand) { keys[r[k]] = mine[k]; perm[r[k]] = static_cast<uint16_t>(c); }
      }
      __syncthreads();
    } else {
      // bitonic sort, descending, sort_n a power of two
      for (int i = ncand + tid; i < p.sort_n; i += NT) keys[i] = 0ull;
      __syncthreads();
      for (int size = 2; size <= p.sort_n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
          for (int i = tid; i < (p.sort_n >> 1); i += NT) {
            const int lo = 2 * i - (i & (stride - 1));
            const int hi2 = lo + stride;
            const bool desc = ((lo & size) == 0);
            const uint64_t a = keys[lo], c = keys[hi2];
            if ((a < c) == desc) { keys[lo] = c; keys[hi2] = a; }
          }
          __syncthreads();
        }
      }
    }
    m_sel = min(ncand, K);
  }

  pdl_trigger();  // the next kernel may start its prologue; it waits for this grid before reading
  for (int r = tid; r < K; r += NT) {
    int64_t idx = -1, slot = -1;
    if (r < m_sel) {
      idx = static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(keys[r] & 0xFFFFFFFFull));
      slot = prefetch ? late.cand_slot[perm[r]] : slot_of(ctx, static_cast<int>(idx));
    }
    out_idx[r] = idx;
    if (out_slot) out_slot[r] = slot;
    if (out_slot32) out_slot32[r] = static_cast<int32_t>(slot);
  }

  if (FUSED) {
    cp_async_wait_all();
    __syncthreads();
    TailPrefetch pf{};
    if (prefetch) { pf.slot = late.cand_slot; pf.score = cand_score; pf.vsc = late.vsc; pf.vrows = late.vrows; }
    finish_tail<MODE, NT>(tp, late.tail, pf, pre, row_max, n_seq, b, h, ctx.bt, [&](int kk, int& pos, int& cidx) {
      if (kk >= m_sel) return false;
      pos = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(keys[kk] & 0xFFFFFFFFull));
      cidx = prefetch ? static_cast<int>(perm[kk]) : -1;
      return true;
    });
  }
}

int pow2_ceil(int x) { int p = 1; while (p < x) p <<= 1; return p; }

// What one of two co-resident blocks may use: half of the multiprocessor's 228 KB, less the 1 KB the system keeps per block.
constexpr size_t kTwoBlockBytes = 228 * 1024 / 2 - 1024;

template <int MODE, int DT, bool LEAN, int NT>
jf_status_t launch_select_variant(const TopkParams& sp, const TailParams& tp, dim3 grid, cudaStream_t stream, bool fused) {
  constexpr size_t kRegion0 = sel_region0_bytes<MODE, LEAN, NT>();
  const size_t smem = sel_smem_bytes(kRegion0, sp.sort_n, LEAN ? 0 : sp.hm_chunks, NT);
  static_assert(sel_smem_bytes(kRegion0, 2 * (LEAN ? JF_MAX_TOP_K : kStagedTopK)) <= kSelSmemLimit || NT != kSelThreads,
                "select kernel shared memory");
  static_assert(NT == kSelThreads || sel_smem_bytes(kRegion0, 1024) <= kTwoBlockBytes, "two narrow blocks per multiprocessor");
  if (smem > kSelSmemLimit) return JF_ERR_UNSUPPORTED;
  if (fused) {
    JF_ENSURE_SMEM((topk_select_kernel<MODE, DT, true, LEAN, NT>), kSelSmemLimit);
    JF_CUDA_TRY(launch_pdl(topk_select_kernel<MODE, DT, true, LEAN, NT>, grid, dim3(NT), smem, stream, sp, tp));
  } else {
    JF_ENSURE_SMEM((topk_select_kernel<MODE, DT, false, LEAN, NT>), kSelSmemLimit);
    JF_CUDA_TRY(launch_pdl(topk_select_kernel<MODE, DT, false, LEAN, NT>, grid, dim3(NT), smem, stream, sp, tp));
  }
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

template <int MODE, bool LEAN, int NT>
jf_status_t launch_select_dtype(const jf_decode_args* a, const TopkParams& sp, const TailParams& tp, dim3 grid,
                                cudaStream_t stream, bool fused) {
  return a->q_dtype == JF_DTYPE_BF16 ? launch_select_variant<MODE, JF_DTYPE_BF16, LEAN, NT>(sp, tp, grid, stream, fused)
                                     : launch_select_variant<MODE, JF_DTYPE_FP16, LEAN, NT>(sp, tp, grid, stream, fused);
}

}  // namespace

TailParams make_tail_params(const jf_decode_args* a, const Workspace& ws) {
  TailParams tp{};
  tp.scores = a->scores ? a->scores : ws.scores;
  tp.part_o = ws.part_o; tp.part_m = ws.part_m; tp.part_l = ws.part_l;
  tp.v_data = a->v_data; tp.v_scales = static_cast<const uint16_t*>(a->v_scales);
  tp.o_hat = a->o_hat; tp.o_old = a->o_old_unnorm; tp.W = a->W;
  tp.softmax_m = a->softmax_m; tp.softmax_inv_z = a->softmax_inv_z;
  tp.num_slots = a->num_slots;
  const HeadGeom hg = head_geom(a->H_q, a->H_kv);
  tp.H_q = a->H_q; tp.H_kv = hg.H_kv; tp.G = hg.G; tp.kv_shift = hg.shift;
  tp.max_S = a->max_S;
  tp.splits = scan_splits(a->mode, a->q_dtype, a->B, hg.H_kv, a->max_S);
  tp.top_k = a->top_k;
  return tp;
}

// select (fused = false) or select + finish in one kernel (fused = true)
jf_status_t launch_select(const jf_decode_args* a, cudaStream_t stream, bool fused) {
  jf_status_t st = validate_decode_args(a);
  if (st != JF_OK) return st;
  if (!a->topk_idx || (!a->topk_slots && !a->topk_slots_i32)) return JF_ERR_ARG;
  if (a->topk_slots_i32 && a->num_slots > 0x7FFFFFFFll) return JF_ERR_ARG;
  if (fused && (!a->o_hat || !a->o_old_unnorm || !a->W)) return JF_ERR_ARG;
  Workspace ws = carve_workspace(a->workspace, a->mode, a->B, a->H_q, a->H_kv, a->max_S, a->top_k, true);
  TopkParams sp{};
  sp.scores = a->scores ? a->scores : ws.scores;
  sp.pmax = ws.pmax; sp.np_stride = page_max_stride(a->mode, a->max_S);
  sp.part_m = ws.part_m; sp.part_smax = ws.part_smax;
  sp.q = a->q; sp.k_data = a->k_data; sp.k_scales = static_cast<const uint16_t*>(a->k_scales);
  sp.block_table = a->block_table; sp.seq_lens = a->seq_lens;
  sp.topk_idx = a->topk_idx; sp.topk_slots = a->topk_slots; sp.topk_slots_i32 = a->topk_slots_i32; sp.status = ws.status;
  sp.num_slots = a->num_slots;
  const HeadGeom hg = head_geom(a->H_q, a->H_kv);
  sp.B = a->B; sp.H_q = a->H_q; sp.H_kv = hg.H_kv; sp.G = hg.G; sp.kv_shift = hg.shift;
  sp.max_S = a->max_S; sp.max_blocks = a->max_blocks;
  sp.splits = scan_splits(a->mode, a->q_dtype, a->B, hg.H_kv, a->max_S);
  sp.top_k = a->top_k;
  sp.sort_n = pow2_ceil(2 * a->top_k);
  if (sp.sort_n < 512) sp.sort_n = 512;
  sp.q_dtype = a->q_dtype;
  sp.attn_scale = a->attn_scale;
  const TailParams tp = make_tail_params(a, ws);
  const dim3 grid(a->H_q, a->B);
  // With more rows than multiprocessors the 512-thread block runs two rows per multiprocessor (one
  // row's chains of dependent memory round trips under the other's arithmetic); otherwise a row's
  // latency is what counts and the 1024-thread block takes it.
  const SelectPlan plan = select_plan(a, sp.scores);
  if (!plan.supported) return JF_ERR_UNSUPPORTED;
  const bool many = plan.narrow, lean = plan.lean;
  // resident-row kernel: rows of 2..4 score chunks get the side table of float4 maxima if it fits
  auto side_table = [&](int nt, size_t region0, size_t budget) {
    const int chunks = (a->max_S + 32 * nt - 1) / (32 * nt);
    return (chunks >= 2 && chunks <= 4 && sel_smem_bytes(region0, sp.sort_n, chunks, nt) <= budget) ? chunks : 0;
  };
  if (a->mode == JF_MODE_K3V2) {
    if (lean && many) return launch_select_dtype<JF_MODE_K3V2, true, 512>(a, sp, tp, grid, stream, fused);
    if (lean) return launch_select_dtype<JF_MODE_K3V2, true, kSelThreads>(a, sp, tp, grid, stream, fused);
    constexpr size_t r512 = sel_region0_bytes<JF_MODE_K3V2, false, 512>();
    if (many && sel_smem_bytes(r512, sp.sort_n, 0, 512) <= kTwoBlockBytes) {
      sp.hm_chunks = side_table(512, r512, kTwoBlockBytes);
      return launch_select_dtype<JF_MODE_K3V2, false, 512>(a, sp, tp, grid, stream, fused);
    }
    sp.hm_chunks = side_table(kSelThreads, sel_region0_bytes<JF_MODE_K3V2, false, kSelThreads>(), kSelSmemLimit);
    return launch_select_dtype<JF_MODE_K3V2, false, kSelThreads>(a, sp, tp, grid, stream, fused);
  }
  if (lean && many) return launch_select_dtype<JF_MODE_K4V4, true, 512>(a, sp, tp, grid, stream, fused);
  if (lean) return launch_select_dtype<JF_MODE_K4V4, true, kSelThreads>(a, sp, tp, grid, stream, fused);
  constexpr size_t r512 = sel_region0_bytes<JF_MODE_K4V4, false, 512>();
  if (many && sel_smem_bytes(r512, sp.sort_n, 0, 512) <= kTwoBlockBytes) {
    sp.hm_chunks = side_table(512, r512, kTwoBlockBytes);
    return launch_select_dtype<JF_MODE_K4V4, false, 512>(a, sp, tp, grid, stream, fused);
  }
  sp.hm_chunks = side_table(kSelThreads, sel_region0_bytes<JF_MODE_K4V4, false, kSelThreads>(), kSelSmemLimit);
  return launch_select_dtype<JF_MODE_K4V4, false, kSelThreads>(a, sp, tp, grid, stream, fused);
}

}  // namespace jf

extern "C" jf_status_t jf_topk_select(const jf_decode_args* a, jf_stream_t stream) {
  return jf::launch_select(a, static_cast<cudaStream_t>(stream), false);
}
