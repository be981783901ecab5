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
#include "decode_common.cuh"

namespace jf {

namespace {

constexpr int kTopkThreads = 1024;
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

constexpr int kRowChunk = 512;                 // candidates staged in shared memory per round
constexpr int kScoreRegs = 32;                 // scores cached per thread (32768 positions per CTA)
constexpr int kScoreChunk = kScoreRegs * kTopkThreads;
template <int MODE> struct RowWords { static constexpr int v = (MODE == JF_MODE_K3V2) ? 13 : 17; };

template <int MODE, int DT>
__global__ void __launch_bounds__(kTopkThreads)
topk_select_kernel(const TopkParams p) {
  constexpr int W = RowWords<MODE>::v;         // 32-bit words staged per candidate: data + scales
  extern __shared__ __align__(16) uint8_t smem_raw[];
  uint64_t* keys = reinterpret_cast<uint64_t*>(smem_raw);                   // [sort_n]
  int* hist = reinterpret_cast<int*>(keys + p.sort_n);                      // [kBins]
  float* q_sm = reinterpret_cast<float*>(hist + kBins);                     // [128]
  float* qs_sm = q_sm + JF_HEAD_DIM;                                        // [4]
  int8_t* qi_sm = reinterpret_cast<int8_t*>(qs_sm + 4);                     // [128]
  int64_t* cand_slot = reinterpret_cast<int64_t*>(qi_sm + JF_HEAD_DIM);     // [kRowChunk]
  uint32_t* rows = reinterpret_cast<uint32_t*>(cand_slot + kRowChunk);      // [kRowChunk][W]
  __shared__ int sh_ncand, sh_last, sh_fallback, sh_tbin;
  __shared__ float sh_red[4];
  __shared__ float sh_w3[32][3];
  __shared__ int sh_wsum[32];
  __shared__ unsigned long long sh_prefix;
  __shared__ int sh_remaining;

  const int h = blockIdx.x, b = blockIdx.y;
  const int hkv = h / p.G, hi = h - hkv * p.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = min(p.seq_lens[b], p.max_S);
  const int K = p.top_k;
  const int64_t bh = static_cast<int64_t>(b) * p.H_q + h;
  int64_t* out_idx = p.topk_idx + bh * K;
  int64_t* out_slot = p.topk_slots + bh * K;
  float* out_canon = p.sel_canon + bh * K;
  if (n <= 0) {
    for (int r = tid; r < K; r += kTopkThreads) { out_idx[r] = -1; out_slot[r] = -1; out_canon[r] = -INFINITY; }
    return;
  }

  // ---- query row (exact values), per-group L1 norms, INT8 model for K4; split statistics ----
  if (tid < JF_HEAD_DIM) {
    q_sm[tid] = Elem<DT>::to_f32(reinterpret_cast<const uint16_t*>(p.q)[bh * JF_HEAD_DIM + tid]);
  }
  {
    float top = kMinusBig, sm0 = 0.f, sm1 = 0.f;
    const int64_t pbase = (static_cast<int64_t>(b) * p.H_kv + hkv) * p.splits;
    for (int s = tid; s < p.splits; s += kTopkThreads) {
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
    if (lane == 0) { sh_w3[warp][0] = top; sh_w3[warp][1] = sm0; sh_w3[warp][2] = sm1; }
  }
  __syncthreads();
  if (warp < 4) {  // warp w handles channels 32w..32w+31
    const float v = q_sm[32 * warp + lane];
    float a = fabsf(v), s1 = fabsf(v) + 0.001953125f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a = fmaxf(a, __shfl_xor_sync(0xFFFFFFFFu, a, o));
      s1 += __shfl_xor_sync(0xFFFFFFFFu, s1, o);
    }
    if (MODE == JF_MODE_K4V4) {
      const float qs = fmaxf(__fdiv_rn(a, 127.0f), 1e-12f);
      const float inv = __fdiv_rn(1.0f, qs);
      qi_sm[32 * warp + lane] = static_cast<int8_t>(max(-128, min(127, __float2int_rn(__fmul_rn(v, inv)))));
      if (lane == 0) qs_sm[warp] = qs;
    }
    if (lane == 0) sh_red[warp] = s1;
  }
  if (tid == 0) { sh_ncand = 0; sh_fallback = 0; sh_tbin = -1; }
  for (int i = tid; i < kBins; i += kTopkThreads) hist[i] = 0;
  for (int i = tid; i < p.sort_n; i += kTopkThreads) keys[i] = 0ull;
  __syncthreads();

  RowCtx ctx;
  ctx.q = q_sm; ctx.qi = qi_sm; ctx.qs = qs_sm;
  const ModeInfo mi = mode_info(MODE);
  ctx.k_rows = p.k_data + static_cast<int64_t>(hkv) * p.num_slots * mi.k_row;
  ctx.k_sc = p.k_scales + static_cast<int64_t>(hkv) * p.num_slots * mi.ng;
  ctx.bt = p.block_table + static_cast<int64_t>(b) * p.max_blocks;
  ctx.num_slots = p.num_slots;
  ctx.attn = p.attn_scale;

  const float* srow = p.scores + bh * p.max_S;
  int ncand = 0;
  bool slow = false;

  if (n <= p.sort_n) {
    // short row: every position is a candidate
    for (int i = tid; i < n; i += kTopkThreads) keys[i] = static_cast<uint64_t>(i);
    ncand = n;
  } else {
    // ---- tier 1: histogram of approximate scores (kept in registers for the second sweep) ----
    float top = kMinusBig, sm0 = 0.f, sm1 = 0.f;
#pragma unroll
    for (int w = 0; w < 32; ++w) {
      top = fmaxf(top, sh_w3[w][0]); sm0 = fmaxf(sm0, sh_w3[w][1]); sm1 = fmaxf(sm1, sh_w3[w][2]);
    }
    top += 4.0f;  // the scan lets its reference point lag the true maximum by at most 4
    const float top64 = top * kBinsPerUnit;
    float delta = 0.f;
    if (MODE == JF_MODE_K3V2) {
      // The scan and the canonical order add the same exact products q_d * k_hat_d in fp32,
      // in different orders: each stays within (roundings) * 2^-24 * sum|q_d k_hat_d| of the
      // exact sum (canonical: 9 roundings; tensor core: one per k-step, 8, possibly
      // truncating).  sum|q_d k_hat_d| <= sum_g 3 * scale_g * sum_{d in g} |q_d|.  A factor 32
      // covers both paths with slack; the last term covers the final multiply by attn_scale.
      const float q1a = sh_red[0] + sh_red[1], q1b = sh_red[2] + sh_red[3];
      const float mag = fabsf(p.attn_scale) * (sm0 * q1a + sm1 * q1b) * 3.0f;
      delta = mag * (32.0f / 16777216.0f) + mag * (4.0f / 16777216.0f) + 1e-7f;
    }
    const bool vec = (p.max_S & 3) == 0;     // rows start on 16-byte boundaries
    const int n_chunks = (n + kScoreChunk - 1) / kScoreChunk;
    float sc[kScoreRegs];
    auto pos_of = [&](int ci, int e) {
      return vec ? ci * kScoreChunk + 4 * ((e >> 2) * kTopkThreads + tid) + (e & 3)
                 : ci * kScoreChunk + e * kTopkThreads + tid;
    };
    auto load_chunk = [&](int ci) {
      if (vec) {
#pragma unroll
        for (int j = 0; j < kScoreRegs / 4; ++j) {
          const int p0 = ci * kScoreChunk + 4 * (j * kTopkThreads + tid);
          float4 v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
          if (p0 < n) v = *reinterpret_cast<const float4*>(srow + p0);  // max_S % 4 == 0: stays inside the row
          sc[4 * j] = v.x; sc[4 * j + 1] = v.y; sc[4 * j + 2] = v.z; sc[4 * j + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < kScoreRegs; ++e) {
          const int pp = ci * kScoreChunk + e * kTopkThreads + tid;
          sc[e] = (pp < n) ? srow[pp] : -INFINITY;
        }
      }
    };
    for (int ci = 0; ci < n_chunks; ++ci) {
      load_chunk(ci);
#pragma unroll
      for (int e = 0; e < kScoreRegs; ++e)
        if (pos_of(ci, e) < n) atomicAdd(&hist[score_bin(top64, sc[e])], 1);
    }
    __syncthreads();
    {
      // block-wide inclusive scan of the histogram, two bins per thread, written back in place
      const int h0 = hist[2 * tid], h1 = hist[2 * tid + 1];
      const int v = h0 + h1;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xFFFFFFFFu, incl, o);
        if (lane >= o) incl += t;
      }
      if (lane == 31) sh_wsum[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        int t = sh_wsum[lane], inc2 = t;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int u = __shfl_up_sync(0xFFFFFFFFu, inc2, o);
          if (lane >= o) inc2 += u;
        }
        sh_wsum[lane] = inc2 - t;  // exclusive prefix of the warp totals
      }
      __syncthreads();
      const int ex = sh_wsum[warp] + incl - v;
      hist[2 * tid] = ex + h0;
      hist[2 * tid + 1] = ex + v;
      if (ex < K && ex + h0 >= K) sh_tbin = 2 * tid;
      else if (ex + h0 < K && ex + v >= K) sh_tbin = 2 * tid + 1;
    }
    __syncthreads();
    if (tid == 0) {
      const int tbin = sh_tbin;
      float nbf = ceilf(2.0f * delta * kBinsPerUnit) + 1.0f;
      if (!(nbf < 4096.0f)) nbf = 4096.0f;
      const int nb = (MODE == JF_MODE_K3V2) ? static_cast<int>(nbf) : 0;
      const int last = min(max(tbin, 0) + nb, kBins - 1);
      sh_last = last;
      sh_fallback = (tbin < 0 || last >= kBins - 1 || hist[last] > p.sort_n) ? 1 : 0;
    }
    __syncthreads();
    if (!sh_fallback) {
      // ---- tier 2: collect the band (positions into keys[]) ----
      const float xlim = static_cast<float>(sh_last + 1);  // bin <= last  <=>  (top - s) * 64 < last + 1
      for (int ci = 0; ci < n_chunks; ++ci) {
        if (n_chunks > 1) load_chunk(ci);
#pragma unroll
        for (int e = 0; e < kScoreRegs; ++e) {
          const int pp = pos_of(ci, e);
          if (pp < n && score_binf(top64, sc[e]) < xlim) {
            const int slot = atomicAdd(&sh_ncand, 1);
            if (slot < p.sort_n) keys[slot] = static_cast<uint64_t>(pp);
          }
        }
      }
      __syncthreads();
      ncand = min(sh_ncand, p.sort_n);
    } else {
      slow = true;
    }
  }
  __syncthreads();

  if (!slow) {
    // ---- re-score the candidates canonically: slots, then their packed rows into shared
    //      memory with independent loads, then one warp per candidate ----
    for (int base = 0; base < ncand; base += kRowChunk) {
      const int cn = min(kRowChunk, ncand - base);
      if (tid < cn) cand_slot[tid] = slot_of(ctx, static_cast<int>(keys[base + tid]));
      __syncthreads();
      for (int idx = tid; idx < cn * W; idx += kTopkThreads) {
        const int c = idx / W, w = idx - c * W;
        const int64_t slot = cand_slot[c];
        uint32_t v = 0u;
        if (slot >= 0) {
          if (MODE == JF_MODE_K3V2) {
            v = (w < 12) ? __ldg(reinterpret_cast<const uint32_t*>(ctx.k_rows + slot * 48) + w)
                         : __ldg(reinterpret_cast<const uint32_t*>(ctx.k_sc + slot * 2));
          } else {
            v = (w < 16) ? __ldg(reinterpret_cast<const uint32_t*>(ctx.k_rows + slot * 64) + w)
                         : static_cast<uint32_t>(__ldg(ctx.k_sc + slot));
          }
        }
        rows[idx] = v;
      }
      __syncthreads();
      for (int c = warp; c < cn; c += kTopkThreads / 32) {
        const int pos = static_cast<int>(keys[base + c]);
        const uint32_t* r = rows + c * W;
        float s = -INFINITY;
        if (cand_slot[c] >= 0) {
          if (MODE == JF_MODE_K3V2)
            s = canon_score_k3(q_sm, reinterpret_cast<const uint8_t*>(r), r[12], ctx.attn, lane);
          else
            s = canon_score_k4(qi_sm, qs_sm, reinterpret_cast<const uint8_t*>(r), bf16_bits_to_f32(r[16] & 0xFFFFu),
                               ctx.attn, lane);
        }
        __syncwarp();
        if (lane == 0) keys[base + c] = make_key(s, pos);
      }
      __syncthreads();
    }
  } else {
    // ---- slow exact path: 8-level radix select on the 64-bit canonical key ----
    if (tid == 0) { sh_prefix = 0ull; sh_remaining = K; sh_ncand = 0; }
    __syncthreads();
    for (int level = 7; level >= 0; --level) {
      for (int i = tid; i < 256; i += kTopkThreads) hist[i] = 0;
      __syncthreads();
      const unsigned long long prefix = sh_prefix;
      for (int i = warp; i < n; i += kTopkThreads / 32) {
        const uint64_t key = canon_key_global<MODE>(ctx, i, lane);
        const bool match = (level == 7) || ((key >> (8 * (level + 1))) == prefix);
        if (match && lane == 0) atomicAdd(&hist[(key >> (8 * level)) & 255u], 1);
      }
      __syncthreads();
      if (tid == 0) {
        int cum = 0, rem = sh_remaining, cb = 0;
        for (int bin = 255; bin >= 0; --bin) {
          if (cum + hist[bin] >= rem) { cb = bin; break; }
          cum += hist[bin];
        }
        sh_remaining = rem - cum;
        sh_prefix = (prefix << 8) | static_cast<unsigned long long>(cb);
      }
      __syncthreads();
    }
    const unsigned long long tkey = sh_prefix;  // key of the k-th best; keys are unique
    for (int i = tid; i < p.sort_n; i += kTopkThreads) keys[i] = 0ull;
    __syncthreads();
    for (int i = warp; i < n; i += kTopkThreads / 32) {
      const uint64_t key = canon_key_global<MODE>(ctx, i, lane);
      if (key >= tkey && lane == 0) {
        const int pos = atomicAdd(&sh_ncand, 1);
        if (pos < p.sort_n) keys[pos] = key;
      }
    }
    __syncthreads();
    ncand = min(sh_ncand, p.sort_n);
  }
  __syncthreads();

  // ---- order the candidates: best first ----
  uint64_t* ranked = keys;
  if (p.sort_n <= 1024) {
    // rank by counting (keys are unique): thread (c, part) counts the keys above candidate c in
    // its share of the list; the partial counts of a candidate are added by a shuffle
    const int parts = (ncand <= kTopkThreads / 4) ? 4 : ((ncand <= kTopkThreads / 2) ? 2 : 1);
    const int c = tid / parts, part = tid - c * parts;
    uint64_t mine = 0ull;
    int rank = 0;
    if (c < ncand) {
      mine = keys[c];
      for (int j = part; j < ncand; j += parts) rank += (keys[j] > mine) ? 1 : 0;
    }
    if (parts >= 2) rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 1);
    if (parts == 4) rank += __shfl_xor_sync(0xFFFFFFFFu, rank, 2);
    __syncthreads();
    if (c < ncand && part == 0) keys[rank] = mine;
    __syncthreads();
  } else {
    // bitonic sort, descending, sort_n a power of two
    for (int i = ncand + tid; i < p.sort_n; i += kTopkThreads) keys[i] = 0ull;
    __syncthreads();
    for (int size = 2; size <= p.sort_n; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int i = tid; i < (p.sort_n >> 1); i += kTopkThreads) {
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

  const int m = min(ncand, K);
  for (int r = tid; r < K; r += kTopkThreads) {
    int64_t idx = -1, slot = -1;
    float canon = -INFINITY;
    if (r < m) {
      idx = static_cast<int64_t>(0xFFFFFFFFu - static_cast<uint32_t>(ranked[r] & 0xFFFFFFFFull));
      slot = slot_of(ctx, static_cast<int>(idx));
      canon = float_from_order_key(static_cast<uint32_t>(ranked[r] >> 32));
    }
    out_idx[r] = idx;
    out_slot[r] = slot;
    out_canon[r] = canon;
  }
}

int pow2_ceil(int x) { int p = 1; while (p < x) p <<= 1; return p; }

}  // namespace

}  // namespace jf

extern "C" jf_status_t jf_topk_select(const jf_decode_args* a, jf_stream_t stream_) {
  using namespace jf;
  jf_status_t st = validate_decode_args(a);
  if (st != JF_OK) return st;
  if (!a->topk_idx || !a->topk_slots) return JF_ERR_ARG;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  Workspace ws = carve_workspace(a->workspace, a->mode, a->B, a->H_q, a->H_kv, a->max_S, a->top_k, true);
  TopkParams tp{};
  tp.scores = a->scores ? a->scores : ws.scores;
  tp.part_m = ws.part_m; tp.part_smax = ws.part_smax;
  tp.q = a->q; tp.k_data = a->k_data; tp.k_scales = static_cast<const uint16_t*>(a->k_scales);
  tp.block_table = a->block_table; tp.seq_lens = a->seq_lens;
  tp.topk_idx = a->topk_idx; tp.topk_slots = a->topk_slots; tp.sel_canon = ws.sel_canon;
  tp.num_slots = a->num_slots;
  tp.B = a->B; tp.H_q = a->H_q; tp.H_kv = a->H_kv; tp.G = a->H_q / a->H_kv;
  tp.max_S = a->max_S; tp.max_blocks = a->max_blocks;
  tp.splits = scan_splits(a->mode, a->q_dtype, a->B, a->H_kv, a->max_S);
  tp.top_k = a->top_k;
  tp.sort_n = pow2_ceil(2 * a->top_k);
  if (tp.sort_n < 512) tp.sort_n = 512;
  tp.q_dtype = a->q_dtype;
  tp.attn_scale = a->attn_scale;
  constexpr size_t kFixedSmem = kBins * 4 + JF_HEAD_DIM * 4 + 16 + JF_HEAD_DIM + kRowChunk * 8 + kRowChunk * 17 * 4;
  const size_t smem = static_cast<size_t>(tp.sort_n) * 8 + kFixedSmem;
  constexpr size_t kTopkMaxSmem = static_cast<size_t>(2 * JF_MAX_TOP_K) * 8 + kFixedSmem;
  dim3 grid(a->H_q, a->B);
#define JF_TOPK(MODE, DT)                                                                              \
  do {                                                                                                 \
    JF_ENSURE_SMEM((topk_select_kernel<MODE, DT>), kTopkMaxSmem);                                      \
    topk_select_kernel<MODE, DT><<<grid, kTopkThreads, smem, stream>>>(tp);                            \
  } while (0)
  if (a->mode == JF_MODE_K3V2) {
    if (a->q_dtype == JF_DTYPE_BF16) JF_TOPK(JF_MODE_K3V2, JF_DTYPE_BF16); else JF_TOPK(JF_MODE_K3V2, JF_DTYPE_FP16);
  } else {
    if (a->q_dtype == JF_DTYPE_BF16) JF_TOPK(JF_MODE_K4V4, JF_DTYPE_BF16); else JF_TOPK(JF_MODE_K4V4, JF_DTYPE_FP16);
  }
#undef JF_TOPK
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}
