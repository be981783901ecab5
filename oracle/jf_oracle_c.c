/*
 * C restatement of the decode scan for CPU-baseline timing and for checking the numpy
 * oracle at sizes numpy handles slowly.  TEST INFRASTRUCTURE ONLY (see oracle/__init__.py):
 * only tests and the CPU-baseline / reference arms of bench.py load this; the product
 * never does.
 *
 * The JetFire project has no native CPU implementation of the scan; this follows the
 * arithmetic of its GPU kernels and validation scripts (paths inside that project):
 *   dequantisation   scripts/validate_runtime.py:22-43, csrc/int3_qk_scores.cu:90-100
 *   K3 scores        csrc/int3_qk_scores.cu:284-311 (canonical order: 32 strided partials + butterfly)
 *   K4/G128 scores   csrc/int8tc_qk_scores.cu:272-290, 445-487 (INT8 query)
 *   top-k            csrc/int3_qk_scores.cu:426-554, order (score desc, position asc)
 *   Stage B (fp32)   csrc/int2_softmax_v.cu:120-143, 681-705, 738-788
 *   Stage B (INT8-P) csrc/int8tc_softmax_v_fused.cu:62, 1049-1053, 1203-1311 (K4V4, batch > 1 plan)
 * One (batch, query head) row per OpenMP task.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16f(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline float round_bf16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  u += 0x7FFFu + ((u >> 16) & 1u);
  u &= 0xFFFF0000u;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

typedef struct {
  float s;
  int32_t idx;
} cand_t;

static int cmp_cand(const void* a, const void* b) {
  const cand_t* x = (const cand_t*)a;
  const cand_t* y = (const cand_t*)b;
  if (x->s > y->s) return -1;
  if (x->s < y->s) return 1;
  return (x->idx > y->idx) - (x->idx < y->idx);
}

int jf_oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/*
 * mode 0 = K3V2 (group 64), 1 = K4V4 (group 128).  q: (B,H_q,128) f32 values.
 * scores may be NULL; if given it is (B,H_q,max_S) and filled up to each row's length.
 * Returns 0.
 */
static int jf_oracle_decode_impl(int mode, int stage_b, const float* q, const uint8_t* k_data, const uint16_t* k_scales,
                     const uint8_t* v_data, const uint16_t* v_scales, const int64_t* block_table,
                     const int32_t* seq_lens, int B, int H_q, int H_kv, int max_S, int max_blocks,
                     int64_t num_slots, float attn_scale, int top_k, int n_threads, float* scores,
                     int64_t* topk_idx, int64_t* topk_slots, float* o_hat, float* o_old, float* W,
                     float* soft_m, float* soft_inv_z) {
  const int G = H_q / H_kv;
  if (stage_b && !mode) return -1; /* the INT8-P arithmetic exists for K4V4 only */
  const int k_row = mode ? 64 : 48, v_row = mode ? 64 : 32, ng = mode ? 1 : 2;
#ifdef _OPENMP
  if (n_threads > 0) omp_set_num_threads(n_threads);
#endif
#pragma omp parallel for schedule(dynamic, 1)
  for (int bh = 0; bh < B * H_q; ++bh) {
    const int b = bh / H_q, h = bh % H_q, hk = h / G;
    int n = seq_lens[b] < max_S ? seq_lens[b] : max_S;
    if (n < 0) n = 0;
    const float* qr = q + (int64_t)bh * 128;
    float* s = (float*)malloc(sizeof(float) * (n > 0 ? n : 1));
    cand_t* cand = (cand_t*)malloc(sizeof(cand_t) * (n > 0 ? n : 1));
    /* INT8 query model for K4 */
    int qi[128];
    float qs[4];
    if (mode) {
      for (int c = 0; c < 4; ++c) {
        float amax = 0.f;
        for (int d = 0; d < 32; ++d) amax = fmaxf(amax, fabsf(qr[32 * c + d]));
        qs[c] = fmaxf(amax / 127.0f, 1e-12f);
        const float inv = 1.0f / qs[c];
        for (int d = 0; d < 32; ++d) {
          float r = nearbyintf(qr[32 * c + d] * inv);
          if (r > 127.f) r = 127.f;
          if (r < -128.f) r = -128.f;
          qi[32 * c + d] = (int)r;
        }
      }
    }
    float mx = -INFINITY;
    for (int p = 0; p < n; ++p) {
      const int64_t slot = block_table[(int64_t)b * max_blocks + (p >> 4)] * 16 + (p & 15);
      const uint8_t* kr = k_data + ((int64_t)hk * num_slots + slot) * k_row;
      const uint16_t* ksc = k_scales + ((int64_t)hk * num_slots + slot) * ng;
      float sc;
      if (!mode) {
        /* canonical order: 32 partials (channels l, l+32, l+64, l+96), then a butterfly */
        float part[32];
        for (int l = 0; l < 32; ++l) part[l] = 0.f;
        for (int r = 0; r < 4; ++r) {
          for (int l = 0; l < 32; ++l) {
            const int d = 32 * r + l, i = d >> 3, x = d & 7;
            const uint32_t w = ((uint32_t)kr[i] << 16) | ((uint32_t)kr[16 + i] << 8) | kr[32 + i];
            const int code = (int)((w >> (21 - 3 * x)) & 7u) - 4;
            const float kh = round_bf16((float)code * bf16f(ksc[i >> 3]));
            part[l] = fmaf(qr[d], kh, part[l]);
          }
        }
        for (int o = 16; o > 0; o >>= 1) {
          float nxt[32];
          for (int l = 0; l < 32; ++l) nxt[l] = part[l] + part[l ^ o];
          for (int l = 0; l < 32; ++l) part[l] = nxt[l];
        }
        const float acc = part[0];
        sc = acc * attn_scale;
      } else {
        float t = 0.f;
        for (int c = 0; c < 4; ++c) {
          int acc = 0;
          for (int j = 0; j < 16; ++j) {
            const uint8_t byte = kr[16 * c + j];
            acc += ((int)(byte >> 4) - 8) * qi[32 * c + 2 * j] + ((int)(byte & 15) - 8) * qi[32 * c + 2 * j + 1];
          }
          t = fmaf((float)acc, qs[c], t);
        }
        sc = (t * bf16f(ksc[0])) * attn_scale;
      }
      sc += 0.0f;
      s[p] = sc;
      cand[p].s = sc;
      cand[p].idx = p;
      if (sc > mx) mx = sc;
      if (scores) scores[(int64_t)bh * max_S + p] = sc;
    }
    /* top-k */
    if (n > 0) qsort(cand, n, sizeof(cand_t), cmp_cand);
    for (int r = 0; r < top_k; ++r) {
      int64_t idx = -1, slot = -1;
      if (r < n) {
        idx = cand[r].idx;
        slot = block_table[(int64_t)b * max_blocks + (idx >> 4)] * 16 + (idx & 15);
      }
      topk_idx[(int64_t)bh * top_k + r] = idx;
      topk_slots[(int64_t)bh * top_k + r] = slot;
    }
    /* Stage B, fp32 weights, double accumulators */
    double oh[128], oo[128], z = 0.0, wsum = 0.0;
    for (int d = 0; d < 128; ++d) oh[d] = oo[d] = 0.0;
    if (!isfinite(mx)) mx = 0.f;
    for (int p = 0; p < n; ++p) z += exp((double)(s[p] - mx));
    const double inv_z = z > 0 ? 1.0 / z : 0.0;
    if (stage_b) {
      /* INT8-P o_hat: positions cut into 8 splits of ceil(max_S / 8); inside a split 32-token
       * tiles start at the split's first 16-token block; per tile pv = p * vs (p normalised, fp32),
       * scale = max|pv| / 127, pq = clamp(rint(pv * (1 / scale)), -127, 127),
       * o_hat += float(sum pq * code) * scale in fp32. */
      float ohf[128];
      for (int d = 0; d < 128; ++d) ohf[d] = 0.f;
      const float mxf = mx, inv_zf = (float)inv_z;
      const int chunk = (max_S + 7) / 8;
      for (int sp = 0; sp < 8; ++sp) {
        const int lo = sp * chunk, hi = (sp + 1) * chunk < n ? (sp + 1) * chunk : n;
        if (lo >= hi) continue;
        for (int t0 = (lo / 16) * 16; t0 < hi; t0 += 32) {
          const int a = t0 > lo ? t0 : lo, e = t0 + 32 < hi ? t0 + 32 : hi;
          float pv[32], amax = 0.f;
          for (int p = a; p < e; ++p) {
            const int64_t slot = block_table[(int64_t)b * max_blocks + (p >> 4)] * 16 + (p & 15);
            const float pr = expf(s[p] - mxf) * inv_zf;
            pv[p - a] = pr * bf16f(v_scales[(int64_t)hk * num_slots + slot]);
            if (fabsf(pv[p - a]) > amax) amax = fabsf(pv[p - a]);
          }
          const float scale = amax / 127.0f;
          if (!(scale > 0.f)) continue;
          const float inv_scale = 1.0f / scale;
          int acc[128];
          for (int d = 0; d < 128; ++d) acc[d] = 0;
          for (int p = a; p < e; ++p) {
            int pq = (int)nearbyintf(pv[p - a] * inv_scale);
            if (pq > 127) pq = 127;
            if (pq < -127) pq = -127;
            const int64_t slot = block_table[(int64_t)b * max_blocks + (p >> 4)] * 16 + (p & 15);
            const uint8_t* vr = v_data + ((int64_t)hk * num_slots + slot) * v_row;
            for (int d = 0; d < 128; ++d)
              acc[d] += pq * ((int)((d & 1) ? (vr[d >> 1] & 15) : (vr[d >> 1] >> 4)) - 8);
          }
          for (int d = 0; d < 128; ++d) ohf[d] += (float)acc[d] * scale;
        }
      }
      for (int d = 0; d < 128; ++d) oh[d] = ohf[d];
    }
    for (int pass = stage_b ? 1 : 0; pass < 2; ++pass) {
      const int cnt = pass ? (top_k < n ? top_k : n) : n;
      double* dst = pass ? oo : oh;
      for (int r = 0; r < cnt; ++r) {
        const int p = pass ? cand[r].idx : r;
        const double pr = exp((double)(s[p] - mx)) * inv_z;
        if (pass) wsum += pr;
        const int64_t slot = block_table[(int64_t)b * max_blocks + (p >> 4)] * 16 + (p & 15);
        const uint8_t* vr = v_data + ((int64_t)hk * num_slots + slot) * v_row;
        const uint16_t* vsc = v_scales + ((int64_t)hk * num_slots + slot) * ng;
        if (!mode) {
          const double w0 = pr * bf16f(vsc[0]), w1 = pr * bf16f(vsc[1]);
          for (int d = 0; d < 128; ++d) {
            const int code = (int)((vr[d >> 2] >> ((3 - (d & 3)) * 2)) & 3) - 2;
            dst[d] += (d < 64 ? w0 : w1) * code;
          }
        } else {
          const double w0 = pr * bf16f(vsc[0]);
          for (int d = 0; d < 128; ++d) {
            const int code = (int)((d & 1) ? (vr[d >> 1] & 15) : (vr[d >> 1] >> 4)) - 8;
            dst[d] += w0 * code;
          }
        }
      }
    }
    for (int d = 0; d < 128; ++d) {
      o_hat[(int64_t)bh * 128 + d] = (float)oh[d];
      o_old[(int64_t)bh * 128 + d] = (float)oo[d];
    }
    W[bh] = (float)wsum;
    if (soft_m) soft_m[bh] = mx;
    if (soft_inv_z) soft_inv_z[bh] = (float)inv_z;
    free(s);
    free(cand);
  }
  return 0;
}

int jf_oracle_decode(int mode, const float* q, const uint8_t* k_data, const uint16_t* k_scales,
                     const uint8_t* v_data, const uint16_t* v_scales, const int64_t* block_table,
                     const int32_t* seq_lens, int B, int H_q, int H_kv, int max_S, int max_blocks,
                     int64_t num_slots, float attn_scale, int top_k, int n_threads, float* scores,
                     int64_t* topk_idx, int64_t* topk_slots, float* o_hat, float* o_old, float* W,
                     float* soft_m, float* soft_inv_z) {
  return jf_oracle_decode_impl(mode, 0, q, k_data, k_scales, v_data, v_scales, block_table, seq_lens, B, H_q, H_kv,
                               max_S, max_blocks, num_slots, attn_scale, top_k, n_threads, scores, topk_idx,
                               topk_slots, o_hat, o_old, W, soft_m, soft_inv_z);
}

/* stage_b: 0 = fp32 weights, 1 = the INT8-P arithmetic (mode 1 only). */
int jf_oracle_decode_stage_b(int mode, int stage_b, const float* q, const uint8_t* k_data, const uint16_t* k_scales,
                             const uint8_t* v_data, const uint16_t* v_scales, const int64_t* block_table,
                             const int32_t* seq_lens, int B, int H_q, int H_kv, int max_S, int max_blocks,
                             int64_t num_slots, float attn_scale, int top_k, int n_threads, float* scores,
                             int64_t* topk_idx, int64_t* topk_slots, float* o_hat, float* o_old, float* W,
                             float* soft_m, float* soft_inv_z) {
  return jf_oracle_decode_impl(mode, stage_b, q, k_data, k_scales, v_data, v_scales, block_table, seq_lens, B, H_q,
                               H_kv, max_S, max_blocks, num_slots, attn_scale, top_k, n_threads, scores, topk_idx,
                               topk_slots, o_hat, o_old, W, soft_m, soft_inv_z);
}
