// Exact, deterministic top-k per query head over the scan's approximate scores.
//
// The reference selects with a 4-level radix select on fp32 scores that came out of a
// tensor-core accumulation (jetfire_vllm/csrc/int3_qk_scores.cu:426-554): which position
// wins near the k-th score depends on an unspecified summation order, and the output order
// and the choice among ties depend on atomics.  Here selection is two-tier:
//   1. a 2048-bin histogram of the approximate scores (bin width 1/64 below an upper bound
//      of the row maximum) finds the bin T that holds the k-th largest approximate score;
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
  const float* part_m;
  const float* part_smax;
  const void* q;
  const uint8_t* k_data;
  const uint16_t* k_scales;
  const int64_t* block_table;
  const int32_t* seq_lens;
  int64_t* topk_idx;
  int64_t* topk_slots;
  float* sel_canon;
  int64_t num_slots;
  int B, H_q, H_kv, G, max_S, max_blocks, splits, top_k, sort_n, q_dtype;
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

// Canonical K4/G128 score by ONE thread.  The integer dot products are exact, so any order
// gives the value of canon_score_k4: byte B of the packed row holds channel 2B in its high
// nibble and channel 2B + 1 in its low nibble; `qe` / `qo` are the INT8 query's even / odd
// channels packed four to a word, `qsum8[c]` = 8 * (sum of the query over block c) removes
// the code offset.
__device__ __forceinline__ float canon_score_k4_thread(const uint32_t* qe, const uint32_t* qo, const int* qsum8,
                                                       const float* qs, const uint32_t* row, float ks, float attn) {
  float s = 0.f;
#pragma unroll
  for (int blk = 0; blk < 4; ++blk) {
    int acc = -qsum8[blk];
#pragma unroll
    for (int w = 4 * blk; w < 4 * blk + 4; ++w) {
      const uint32_t word = row[w];
      acc = __dp4a(static_cast<int>((word >> 4) & 0x0F0F0F0Fu), static_cast<int>(qe[w]), acc);
      acc = __dp4a(static_cast<int>(word & 0x0F0F0F0Fu), static_cast<int>(qo[w]), acc);
    }
    s = __fmaf_rn(static_cast<float>(acc), qs[blk], s);
  }
  return __fmul_rn(__fmul_rn(s, ks), attn);
}

constexpr int kRowChunk = 512;                 // candidates staged in shared memory per round
constexpr int kScoreRegs = 32;                 // scores cached per thread (32768 positions per CTA)
constexpr int kScoreChunk = kScoreRegs * kSelThreads;
template <int MODE> struct RowWords { static constexpr int v = (MODE == JF_MODE_K3V2) ? 13 : 17; };

struct SelSmemFixed {
  int hist[kBins];
  float q[JF_HEAD_DIM];
  float qs[4];
  int qsum8[4];
  uint32_t qe[16], qo[16];
  int8_t qi[JF_HEAD_DIM];
  int64_t cand_slot[kRowChunk];
  uint32_t rows[kRowChunk * 17];
  float w3[kSelWarps][3];
  float red[4];
  int wsum[kSelWarps];
  int ncand, last, fallback, tbin, remaining;
  unsigned long long prefix;
};

// One CTA per (query head, batch element).  FUSED: the finish stage follows in the same
// kernel (the selected list never leaves the SM).
template <int MODE, int DT, bool FUSED>
__global__ void __launch_bounds__(kSelThreads)
topk_select_kernel(const TopkParams p, const TailParams tp) {
  constexpr int W = RowWords<MODE>::v;         // 32-bit words staged per candidate: data + scales
  extern __shared__ __align__(16) uint8_t smem_raw[];
  TailSmem<MODE>& tsm = *reinterpret_cast<TailSmem<MODE>*>(smem_raw);
  SelSmemFixed& sm = *reinterpret_cast<SelSmemFixed*>(smem_raw + sizeof(TailSmem<MODE>));
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw + sizeof(TailSmem<MODE>) + sizeof(SelSmemFixed));  // [sort_n]
  int* hist = sm.hist;

  JF_PHASE(0);
  const int h = blockIdx.x, b = blockIdx.y;
  const int hkv = h / p.G, hi = h - hkv * p.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = p.top_k;
  const int64_t bh = static_cast<int64_t>(b) * p.H_q + h;
  const float* srow = p.scores + bh * p.max_S;
  const int64_t pbase = (static_cast<int64_t>(b) * p.H_kv + hkv) * p.splits;

  // ---- the row's scores go to registers first: nothing else depends on them yet, so their
  //      latency hides behind the prologue.  Positions past the sequence are masked later;
  //      the row's allocation covers max_S. ----
  const bool vec = (p.max_S & 3) == 0;     // rows start on 16-byte boundaries
  float sc[kScoreRegs];
  auto pos_of = [&](int ci, int e) {
    return vec ? ci * kScoreChunk + 4 * ((e >> 2) * kSelThreads + tid) + (e & 3)
               : ci * kScoreChunk + e * kSelThreads + tid;
  };
  auto load_chunk = [&](int ci) {
    if (vec) {
#pragma unroll
      for (int j = 0; j < kScoreRegs / 4; ++j) {
        const int p0 = ci * kScoreChunk + 4 * (j * kSelThreads + tid);
        float4 v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        if (p0 < p.max_S) v = *reinterpret_cast<const float4*>(srow + p0);  // max_S % 4 == 0: stays inside the row
        sc[4 * j] = v.x; sc[4 * j + 1] = v.y; sc[4 * j + 2] = v.z; sc[4 * j + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int e = 0; e < kScoreRegs; ++e) {
        const int pp = ci * kScoreChunk + e * kSelThreads + tid;
        sc[e] = (pp < p.max_S) ? srow[pp] : -INFINITY;
      }
    }
  };
  load_chunk(0);
  SplitPre pre;
  if (FUSED) split_preload(tp, pbase, hi, tid, pre);

  const int n = min(p.seq_lens[b], p.max_S);
  int64_t* out_idx = p.topk_idx + bh * K;
  int64_t* out_slot = p.topk_slots + bh * K;
  float* out_canon = p.sel_canon + bh * K;

  // ---- query row (exact values), per-group L1 norms, INT8 model for K4; split statistics ----
  if (tid < JF_HEAD_DIM) {
    sm.q[tid] = Elem<DT>::to_f32(reinterpret_cast<const uint16_t*>(p.q)[bh * JF_HEAD_DIM + tid]);
  }
  {
    float top = kMinusBig, sm0 = 0.f, sm1 = 0.f;
    for (int s = tid; s < p.splits; s += kSelThreads) {
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
      int qsum = qv;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) qsum += __shfl_xor_sync(0xFFFFFFFFu, qsum, o);
      // words of four even / four odd channels: lanes 8k..8k+7 make word 4 * warp + k
      const uint32_t byte = static_cast<uint32_t>(qv) & 0xFFu;
      const uint32_t b2 = __shfl_down_sync(0xFFFFFFFFu, byte, 2), b4 = __shfl_down_sync(0xFFFFFFFFu, byte, 4),
                     b6 = __shfl_down_sync(0xFFFFFFFFu, byte, 6);
      const uint32_t word = byte | (b2 << 8) | (b4 << 16) | (b6 << 24);
      if ((lane & 7) == 0) sm.qe[4 * warp + (lane >> 3)] = word;
      if ((lane & 7) == 1) sm.qo[4 * warp + (lane >> 3)] = word;
      if (lane == 0) { sm.qs[warp] = qs; sm.qsum8[warp] = 8 * qsum; }
    }
    if (lane == 0) sm.red[warp] = s1;
  }
  if (tid == 0) { sm.ncand = 0; sm.fallback = 0; sm.tbin = -1; }
  for (int i = tid; i < kBins; i += kSelThreads) hist[i] = 0;
  for (int i = tid; i < p.sort_n; i += kSelThreads) keys[i] = 0ull;
  __syncthreads();
  JF_PHASE(1);

  RowCtx ctx;
  ctx.q = sm.q; ctx.qi = sm.qi; ctx.qs = sm.qs;
  const ModeInfo mi = mode_info(MODE);
  ctx.k_rows = p.k_data + static_cast<int64_t>(hkv) * p.num_slots * mi.k_row;
  ctx.k_sc = p.k_scales + static_cast<int64_t>(hkv) * p.num_slots * mi.ng;
  ctx.bt = p.block_table + static_cast<int64_t>(b) * p.max_blocks;
  ctx.num_slots = p.num_slots;
  ctx.attn = p.attn_scale;

  float row_max = kMinusBig;  // max over the splits of the scan's reference points
#pragma unroll
  for (int w = 0; w < kSelWarps; ++w) row_max = fmaxf(row_max, sm.w3[w][0]);

  int m_sel = 0;  // entries of keys[] that hold the ranked result
  if (n > 0) {
    int ncand = 0;
    bool slow = false;

    if (n <= p.sort_n) {
      // short row: every position is a candidate
      for (int i = tid; i < n; i += kSelThreads) keys[i] = static_cast<uint64_t>(i);
      ncand = n;
    } else {
      float sm0 = 0.f, sm1 = 0.f;
#pragma unroll
      for (int w = 0; w < kSelWarps; ++w) { sm0 = fmaxf(sm0, sm.w3[w][1]); sm1 = fmaxf(sm1, sm.w3[w][2]); }
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
      const int n_chunks = (n + kScoreChunk - 1) / kScoreChunk;

      // Block-wide: turns hist[] into inclusive prefix counts (from the top bin down) and
      // leaves in sm.tbin the bin where the count reaches K (-1: never).
      auto scan_hist = [&]() {
        const int h0 = hist[2 * tid], h1 = hist[2 * tid + 1];
        const int v = h0 + h1;
        int incl = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
          if (lane >= o) incl += t;
        }
        if (lane == 31) sm.wsum[warp] = incl;
        __syncthreads();
        if (warp == 0) {
          int t = sm.wsum[lane], inc2 = t;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xFFFFFFFFu, inc2, o);
            if (lane >= o) inc2 += u;
          }
          sm.wsum[lane] = inc2 - t;  // exclusive prefix of the warp totals
        }
        __syncthreads();
        const int ex = sm.wsum[warp] + incl - v;
        hist[2 * tid] = ex + h0;
        hist[2 * tid + 1] = ex + v;
        if (ex < K && ex + h0 >= K) sm.tbin = 2 * tid;
        else if (ex + h0 < K && ex + v >= K) sm.tbin = 2 * tid + 1;
        __syncthreads();
      };
      // Block-wide: positions whose bin is <= last go to keys[] (one shared-memory atomic per
      // warp and chunk); returns how many there are (may exceed sort_n: then keys[] is partial).
      auto collect = [&](int last) {
        const float xlim = static_cast<float>(last + 1);  // bin <= last  <=>  (top - s) * 64 < last + 1
        for (int ci = 0; ci < n_chunks; ++ci) {
          if (n_chunks > 1) load_chunk(ci);
          int cnt = 0;
#pragma unroll
          for (int e = 0; e < kScoreRegs; ++e) cnt += (pos_of(ci, e) < n && score_binf(top64, sc[e]) < xlim) ? 1 : 0;
          int incl = cnt;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
            if (lane >= o) incl += t;
          }
          int base = 0;
          if (lane == 31 && incl > 0) base = atomicAdd(&sm.ncand, incl);
          base = __shfl_sync(0xFFFFFFFFu, base, 31);
          if (cnt > 0) {
            int o = base + incl - cnt;
#pragma unroll
            for (int e = 0; e < kScoreRegs; ++e) {
              const int pp = pos_of(ci, e);
              if (pp < n && score_binf(top64, sc[e]) < xlim) {
                if (o < p.sort_n) keys[o] = static_cast<uint64_t>(pp);
                ++o;
              }
            }
          }
        }
        __syncthreads();
        return sm.ncand;
      };

      // ---- tier 1a: a bound from group maxima.  Each thread holds four groups of positions
      //      per chunk (stride 4096 inside a group); the K-th largest group maximum is a lower
      //      bound of the K-th largest score, and far fewer values enter the histogram. ----
      for (int ci = 0; ci < n_chunks; ++ci) {
        if (ci > 0) load_chunk(ci);
        float gm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < kScoreRegs; ++e)
          if (pos_of(ci, e) < n) gm[e & 3] = fmaxf(gm[e & 3], sc[e]);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          if (gm[c] > -INFINITY) atomicAdd(&hist[score_bin(top64, gm[c])], 1);
      }
      __syncthreads();
      JF_PHASE(2);
      scan_hist();
      JF_PHASE(3);
      bool ok = false;
      {
        const int tbin = sm.tbin;
        const int last = tbin + nb;
        if (tbin >= 0 && last < kBins - 1) {
          const int total = collect(last);
          ok = total <= p.sort_n;
          ncand = total;
        }
      }
      if (!ok) {
        // ---- tier 1b: histogram of every score; the band around the bin of the K-th largest ----
        __syncthreads();
        if (tid == 0) { sm.ncand = 0; sm.tbin = -1; }
        for (int i = tid; i < kBins; i += kSelThreads) hist[i] = 0;
        __syncthreads();
        for (int ci = 0; ci < n_chunks; ++ci) {
          if (n_chunks > 1) load_chunk(ci);
#pragma unroll
          for (int e = 0; e < kScoreRegs; ++e)
            if (pos_of(ci, e) < n) atomicAdd(&hist[score_bin(top64, sc[e])], 1);
        }
        __syncthreads();
        scan_hist();
        const int tbin = sm.tbin;
        const int last = min(max(tbin, 0) + nb, kBins - 1);
        if (tbin < 0 || last >= kBins - 1 || hist[last] > p.sort_n) {
          slow = true;
        } else {
          for (int i = tid; i < p.sort_n; i += kSelThreads) keys[i] = 0ull;
          __syncthreads();
          ncand = collect(last);
        }
      }
    }
    __syncthreads();
    JF_PHASE(4);

    if (!slow) {
      // ---- re-score the candidates canonically: slots, then their packed rows into shared
      //      memory with independent 16-byte loads, then the canonical arithmetic ----
      for (int base = 0; base < ncand; base += kRowChunk) {
        const int cn = min(kRowChunk, ncand - base);
        if (tid < cn) sm.cand_slot[tid] = slot_of(ctx, static_cast<int>(keys[base + tid]));
        __syncthreads();
        JF_PHASE(5);
        {
          // unit u = (candidate, quarter): K4 rows are 4 x 16 bytes (+ the scale with quarter 0),
          // K3 rows 3 x 16 bytes and quarter 3 fetches the two scales
          uint4 v[2];
          uint32_t sc16[2];
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int u = tid + i * kSelThreads;
            const int c = u >> 2, part = u & 3;
            v[i] = make_uint4(0u, 0u, 0u, 0u);
            sc16[i] = 0u;
            if (c < cn) {
              const int64_t slot = sm.cand_slot[c];
              if (slot >= 0) {
                if (MODE == JF_MODE_K3V2) {
                  if (part < 3) v[i] = __ldg(reinterpret_cast<const uint4*>(ctx.k_rows + slot * 48) + part);
                  else sc16[i] = __ldg(reinterpret_cast<const uint32_t*>(ctx.k_sc + slot * 2));
                } else {
                  v[i] = __ldg(reinterpret_cast<const uint4*>(ctx.k_rows + slot * 64) + part);
                  if (part == 0) sc16[i] = static_cast<uint32_t>(__ldg(ctx.k_sc + slot));
                }
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int u = tid + i * kSelThreads;
            const int c = u >> 2, part = u & 3;
            if (c < cn) {
              uint32_t* r = sm.rows + c * W;
              if (MODE == JF_MODE_K3V2) {
                if (part < 3) { r[4 * part] = v[i].x; r[4 * part + 1] = v[i].y; r[4 * part + 2] = v[i].z; r[4 * part + 3] = v[i].w; }
                else r[12] = sc16[i];
              } else {
                r[4 * part] = v[i].x; r[4 * part + 1] = v[i].y; r[4 * part + 2] = v[i].z; r[4 * part + 3] = v[i].w;
                if (part == 0) r[16] = sc16[i];
              }
            }
          }
        }
        __syncthreads();
        JF_PHASE(6);
        if (MODE == JF_MODE_K4V4) {
          // one thread per candidate (integer arithmetic: order-free)
          if (tid < cn) {
            const int pos = static_cast<int>(keys[base + tid]);
            const uint32_t* r = sm.rows + tid * W;
            float s = -INFINITY;
            if (sm.cand_slot[tid] >= 0)
              s = canon_score_k4_thread(sm.qe, sm.qo, sm.qsum8, sm.qs, r, bf16_bits_to_f32(r[16] & 0xFFFFu), ctx.attn);
            keys[base + tid] = make_key(s, pos);
          }
        } else {
          // one warp per candidate, four candidates in flight per warp
          for (int c0 = warp; c0 < cn; c0 += 4 * kSelWarps) {
            float s[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int c = c0 + i * kSelWarps;
              s[i] = -INFINITY;
              if (c < cn && sm.cand_slot[c] >= 0) {
                const uint32_t* r = sm.rows + c * W;
                s[i] = canon_score_k3(sm.q, reinterpret_cast<const uint8_t*>(r), r[12], ctx.attn, lane);
              }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int c = c0 + i * kSelWarps;
              if (c < cn && lane == i) keys[base + c] = make_key(s[i], static_cast<int>(keys[base + c]));
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
        for (int i = tid; i < 256; i += kSelThreads) hist[i] = 0;
        __syncthreads();
        const unsigned long long prefix = sm.prefix;
        for (int i = warp; i < n; i += kSelWarps) {
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
      for (int i = tid; i < p.sort_n; i += kSelThreads) keys[i] = 0ull;
      __syncthreads();
      for (int i = warp; i < n; i += kSelWarps) {
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

    JF_PHASE(7);
    // ---- order the candidates: best first ----
    if (p.sort_n <= kSelThreads) {
      // rank by counting (keys are unique): the ncand^2 comparisons are spread evenly, thread
      // (c, part) counts the keys above candidate c among j = part, part + P, ...
      int* rank = hist;
      for (int i = tid; i < ncand; i += kSelThreads) rank[i] = 0;
      __syncthreads();
      const int P = kSelThreads / max(ncand, 1);
      const int part = tid / max(ncand, 1), c = tid - part * max(ncand, 1);
      if (part < P && ncand > 0) {
        const uint64_t mine = keys[c];
        int above = 0;
#pragma unroll 4
        for (int j = part; j < ncand; j += P) above += (keys[j] > mine) ? 1 : 0;
        atomicAdd(&rank[c], above);
      }
      __syncthreads();
      uint64_t mine = 0ull;
      int r = 0;
      if (tid < ncand) { mine = keys[tid]; r = rank[tid]; }
      __syncthreads();
      if (tid < ncand) keys[r] = mine;
      __syncthreads();
    } else {
      // bitonic sort, descending, sort_n a power of two
      for (int i = ncand + tid; i < p.sort_n; i += kSelThreads) keys[i] = 0ull;
      __syncthreads();
      for (int size = 2; size <= p.sort_n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
          for (int i = tid; i < (p.sort_n >> 1); i += kSelThreads) {
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
    JF_PHASE(8);
  }

  for (int r = tid; r < K; r += kSelThreads) {
    int64_t idx = -1, slot = -1;
    float canon = -INFINITY;
    if (r < m_sel) {
      idx = static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(keys[r] & 0xFFFFFFFFull));
      slot = slot_of(ctx, static_cast<int>(idx));
      canon = float_from_order_key(static_cast<uint32_t>(keys[r] >> 32));
    }
    out_idx[r] = idx;
    out_slot[r] = slot;
    out_canon[r] = canon;
  }
  JF_PHASE(9);

  if (FUSED) {
    finish_tail<MODE>(tp, tsm, pre, row_max, n, b, h, ctx.bt, [&](int kk, int& pos, float& canon) {
      if (kk >= m_sel) return false;
      pos = static_cast<int>(0xFFFFFFFFu - static_cast<uint32_t>(keys[kk] & 0xFFFFFFFFull));
      canon = float_from_order_key(static_cast<uint32_t>(keys[kk] >> 32));
      return true;
    });
  }
}

int pow2_ceil(int x) { int p = 1; while (p < x) p <<= 1; return p; }

template <int MODE, int DT>
jf_status_t launch_select_variant(const TopkParams& sp, const TailParams& tp, dim3 grid, cudaStream_t stream, bool fused) {
  const size_t smem = sizeof(TailSmem<MODE>) + sizeof(SelSmemFixed) + static_cast<size_t>(sp.sort_n) * 8;
  constexpr size_t kMaxSmem = sizeof(TailSmem<MODE>) + sizeof(SelSmemFixed) + static_cast<size_t>(2 * JF_MAX_TOP_K) * 8;
  static_assert(kMaxSmem <= 227 * 1024, "select kernel shared memory");
  if (fused) {
    JF_ENSURE_SMEM((topk_select_kernel<MODE, DT, true>), kMaxSmem);
    topk_select_kernel<MODE, DT, true><<<grid, kSelThreads, smem, stream>>>(sp, tp);
  } else {
    JF_ENSURE_SMEM((topk_select_kernel<MODE, DT, false>), kMaxSmem);
    topk_select_kernel<MODE, DT, false><<<grid, kSelThreads, smem, stream>>>(sp, tp);
  }
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
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
  tp.H_q = a->H_q; tp.H_kv = a->H_kv; tp.G = a->H_q / a->H_kv;
  tp.max_S = a->max_S;
  tp.splits = scan_splits(a->mode, a->q_dtype, a->B, a->H_kv, a->max_S);
  tp.top_k = a->top_k;
  return tp;
}

// select (fused = false) or select + finish in one kernel (fused = true)
jf_status_t launch_select(const jf_decode_args* a, cudaStream_t stream, bool fused) {
  jf_status_t st = validate_decode_args(a);
  if (st != JF_OK) return st;
  if (!a->topk_idx || !a->topk_slots) return JF_ERR_ARG;
  if (fused && (!a->o_hat || !a->o_old_unnorm || !a->W)) return JF_ERR_ARG;
  Workspace ws = carve_workspace(a->workspace, a->mode, a->B, a->H_q, a->H_kv, a->max_S, a->top_k, true);
  TopkParams sp{};
  sp.scores = a->scores ? a->scores : ws.scores;
  sp.part_m = ws.part_m; sp.part_smax = ws.part_smax;
  sp.q = a->q; sp.k_data = a->k_data; sp.k_scales = static_cast<const uint16_t*>(a->k_scales);
  sp.block_table = a->block_table; sp.seq_lens = a->seq_lens;
  sp.topk_idx = a->topk_idx; sp.topk_slots = a->topk_slots; sp.sel_canon = ws.sel_canon;
  sp.num_slots = a->num_slots;
  sp.B = a->B; sp.H_q = a->H_q; sp.H_kv = a->H_kv; sp.G = a->H_q / a->H_kv;
  sp.max_S = a->max_S; sp.max_blocks = a->max_blocks;
  sp.splits = scan_splits(a->mode, a->q_dtype, a->B, a->H_kv, a->max_S);
  sp.top_k = a->top_k;
  sp.sort_n = pow2_ceil(2 * a->top_k);
  if (sp.sort_n < 512) sp.sort_n = 512;
  sp.q_dtype = a->q_dtype;
  sp.attn_scale = a->attn_scale;
  const TailParams tp = make_tail_params(a, ws);
  const dim3 grid(a->H_q, a->B);
  if (a->mode == JF_MODE_K3V2) {
    return a->q_dtype == JF_DTYPE_BF16 ? launch_select_variant<JF_MODE_K3V2, JF_DTYPE_BF16>(sp, tp, grid, stream, fused)
                                       : launch_select_variant<JF_MODE_K3V2, JF_DTYPE_FP16>(sp, tp, grid, stream, fused);
  }
  return a->q_dtype == JF_DTYPE_BF16 ? launch_select_variant<JF_MODE_K4V4, JF_DTYPE_BF16>(sp, tp, grid, stream, fused)
                                     : launch_select_variant<JF_MODE_K4V4, JF_DTYPE_FP16>(sp, tp, grid, stream, fused);
}

}  // namespace jf

#ifdef JF_PHASE_TIMING
extern "C" int jf_debug_phase_times(unsigned long long* out) {
  return static_cast<int>(cudaMemcpyFromSymbol(out, g_phase_t, sizeof(g_phase_t)));
}
#endif

extern "C" jf_status_t jf_topk_select(const jf_decode_args* a, jf_stream_t stream) {
  return jf::launch_select(a, static_cast<cudaStream_t>(stream), false);
}
