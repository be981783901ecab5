// Quantise-on-append: fp16/bf16 K/V rows -> INT2/3/4 packed rows + bf16 group scales,
// scattered into the paged cache by slot.
//
// Arithmetic is the torch reference's (jetfire_vllm/kernels/intN_pack.py:81-98):
//   amax over the group -> fp32 amax / qmax (IEEE) clamped to 1e-8 -> bf16 (RNE)
//   q = clamp(rint(x / float(scale_bf16)), -qmax, qmax)   (IEEE divide, half-even)
// and the wire format is :172-222 (INT4 nibbles, INT2 MSB-first quads, INT3 24-bit
// groups split over three byte planes).  Negative slots are skipped
// (jetfire_vllm/kernels/fused_quant_write.py:150-152).
//
// Half a warp owns a (token, kv-head) row: lane l (0..15) holds elements 8l..8l+7 (one
// 16-byte load), which are one INT3 group, one INT4 word or one INT2 half-word of the packed
// row, so packing needs no shuffles; the group maximum takes 3 or 4.  Each warp loads eight
// rows (2 KB) before it processes any, so that enough bytes are in flight per SM, and the
// slot lookup runs beside the row loads, not before them.  HBM-bound: 256 B read +
// 36..66 B written per row.
//
// Mirror rows: the reference keeps every appended row in full precision in host memory
// (jetfire_vllm/adapter/cache_store.py:311-323) and fills it with a device-to-host copy, a
// host synchronisation and an index_copy_ per append (:746-756), or through pinned staging
// and a host callback under CUDA graphs (:616-640).  Here the kernel that packs a row also
// stores its 256 raw bytes -- already in the half-warp's registers as sixteen 16-byte pieces
// -- straight into the mirror through a device-visible pointer (mapped pinned host memory),
// one coalesced 256-byte write per row, so an append is one launch with no host step.
#include "jf_common.cuh"

namespace jf {

constexpr int kPairsPerWarp = 2;   // row pairs (one per half-warp) per warp
constexpr int kWarpsPerCta = 8;

struct PackSide {
  const void* x;
  int64_t stride_t, stride_h;
  uint8_t* data;
  uint16_t* scales;
  int nbits;
  uint16_t* mirror;   // (H_kv, num_slots, 128) 16-bit rows, device-visible; may be null
};

template <int DT, int NBITS, int GS>
__device__ __forceinline__ void pack_row(uint4 raw, uint8_t* __restrict__ out_row,
                                         uint16_t* __restrict__ scale_row, int sub, bool live) {
  constexpr int QMAX = (1 << (NBITS - 1)) - 1;
  constexpr int OFF = 1 << (NBITS - 1);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
  float f[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = Elem<DT>::to_f32(w[i] & 0xFFFF);
    f[2 * i + 1] = Elem<DT>::to_f32(w[i] >> 16);
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
  for (int o = 1; o < GS / 8; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  const float scale = fmaxf(__fdiv_rn(amax, static_cast<float>(QMAX)), 1e-8f);
  const uint16_t sb = __bfloat16_as_ushort(__float2bfloat16_rn(scale));
  const float sf = bf16_bits_to_f32(sb);
  // q = rint(fl(x / sf)) without an IEEE division per element: t = x * rcp(sf) is within
  // 2^-19 of the exact quotient (|quotient| < 8, both steps within 2^-23 relative), and so is
  // the correctly rounded quotient; unless t sits within 2^-17 of a rounding boundary k + 1/2
  // all three round to the same integer.  Only those rare elements take the true division.
  float rs;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rs) : "f"(sf));
  // Rounding and float -> int without conversion instructions: t + 1.5 * 2^23 is rounded
  // (half-even) to an integer that sits in the low mantissa bits.  The clamp to +-QMAX comes
  // first (it commutes with rounding); an element whose t is not within 1/2 - 2^-17 of the
  // rounded value -- near a boundary, or NaN / far out of range -- takes the true division.
  constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23
  uint32_t c[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float t = f[i] * rs;
    float tm = fminf(fmaxf(t, -static_cast<float>(QMAX)), static_cast<float>(QMAX)) + kMagic;
    if (fabsf(t - (tm - kMagic)) > 0.5f - 0.00000762939453125f) {
      const float q = rintf(__fdiv_rn(f[i], sf));
      tm = fminf(fmaxf(q, -static_cast<float>(QMAX)), static_cast<float>(QMAX)) + kMagic;
    }
    c[i] = static_cast<uint32_t>(__float_as_int(tm) - 0x4B400000 + OFF);
  }
  if (!live) return;  // after the shuffles: the other half of the warp may still need them
  // scales: one per group, written by the group's first lane
  if (GS == 64) { if ((sub & 7) == 0) scale_row[sub >> 3] = sb; }
  else { if (sub == 0) scale_row[0] = sb; }
  if (NBITS == 4) {        // byte B = (code 2B << 4) | code 2B+1
    reinterpret_cast<uint32_t*>(out_row)[sub] = ((c[0] << 4) | c[1]) | (((c[2] << 4) | c[3]) << 8) |
                                                (((c[4] << 4) | c[5]) << 16) | (((c[6] << 4) | c[7]) << 24);
  } else if (NBITS == 2) { // byte B = four codes, first in the top bits
    reinterpret_cast<uint16_t*>(out_row)[sub] = static_cast<uint16_t>(
        ((c[0] << 6) | (c[1] << 4) | (c[2] << 2) | c[3]) | (((c[4] << 6) | (c[5] << 4) | (c[6] << 2) | c[7]) << 8));
  } else {                 // eight codes -> 24 bits MSB-first, byte p of group i at out_row[16 p + i]
    const uint32_t w24 = (c[0] << 21) | (c[1] << 18) | (c[2] << 15) | (c[3] << 12) | (c[4] << 9) | (c[5] << 6) |
                         (c[6] << 3) | c[7];
    out_row[sub] = static_cast<uint8_t>(w24 >> 16);
    out_row[16 + sub] = static_cast<uint8_t>(w24 >> 8);
    out_row[32 + sub] = static_cast<uint8_t>(w24);
  }
}

// One batch of rows per warp; residency (not a loop) overlaps the loads of some warps with
// the arithmetic of others -- a persistent loop with a register double buffer measured slower.
template <int DT, int GS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
pack_append_kernel(PackSide s0, PackSide s1, int64_t T, int H, const int64_t* __restrict__ slots,
                   int64_t num_slots) {
  const PackSide s = (blockIdx.y == 0) ? s0 : s1;
  const int lane = threadIdx.x & 31, half = lane >> 4, sub = lane & 15;
  const int64_t rows = T * H;
  const int64_t n_batches = (rows + 2 * kPairsPerWarp - 1) / (2 * kPairsPerWarp);
  constexpr int NG = 128 / GS;
  const int dp = 16 * s.nbits;
  const bool small = rows <= 0x7FFFFFFF;   // 32-bit index arithmetic (a 64-bit division costs more than a row)

  struct Batch {
    uint4 raw[kPairsPerWarp];
    int64_t slot[kPairsPerWarp];
    int hh[kPairsPerWarp];
  };
  auto load = [&](int64_t batch, Batch& bt) {
    const int64_t r0 = batch * (2 * kPairsPerWarp) + half;   // this half-warp's rows: r0, r0 + 2, ...
#pragma unroll
    for (int i = 0; i < kPairsPerWarp; ++i) {
      const int64_t r = r0 + 2 * i;
      bt.slot[i] = -1;
      bt.hh[i] = 0;
      bt.raw[i] = make_uint4(0u, 0u, 0u, 0u);
      if (batch < n_batches && r < rows) {
        int64_t t;
        if (small) {
          const uint32_t tq = static_cast<uint32_t>(r) / static_cast<uint32_t>(H);
          bt.hh[i] = static_cast<int>(static_cast<uint32_t>(r) - tq * static_cast<uint32_t>(H));
          t = tq;
        } else {
          t = r / H;
          bt.hh[i] = static_cast<int>(r - t * H);
        }
        bt.slot[i] = slots[t];   // rows of skipped tokens are read too: the load does not wait for the slot
        const uint16_t* row = reinterpret_cast<const uint16_t*>(s.x) + t * s.stride_t + bt.hh[i] * s.stride_h;
        bt.raw[i] = __ldg(reinterpret_cast<const uint4*>(row) + sub);
      }
    }
  };

  const int64_t batch = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  if (batch >= n_batches) return;
  Batch cur;
  load(batch, cur);
#pragma unroll
  for (int i = 0; i < kPairsPerWarp; ++i) {
    // the two halves of a warp may disagree here; the shuffles inside stay within a half
    const bool live = cur.slot[i] >= 0 && cur.slot[i] < num_slots;   // never write outside the cache
    const int64_t o = static_cast<int64_t>(cur.hh[i]) * num_slots + (live ? cur.slot[i] : 0);
    uint8_t* out_row = s.data + o * dp;
    uint16_t* scale_row = s.scales + o * NG;
    if (s.mirror != nullptr && live) reinterpret_cast<uint4*>(s.mirror + o * JF_HEAD_DIM)[sub] = cur.raw[i];
    // every lane runs the arithmetic (full-mask shuffles); only live rows are stored
    if (s.nbits == 3) pack_row<DT, 3, GS>(cur.raw[i], out_row, scale_row, sub, live);
    else if (s.nbits == 2) pack_row<DT, 2, GS>(cur.raw[i], out_row, scale_row, sub, live);
    else pack_row<DT, 4, GS>(cur.raw[i], out_row, scale_row, sub, live);
  }
}

static jf_status_t check_side(const void* x, int64_t st, int64_t sh, const void* data, const void* scales, int nbits) {
  if (!x || !data || !scales) return JF_ERR_ARG;
  if (nbits < 2 || nbits > 4) return JF_ERR_UNSUPPORTED;
  if (!aligned(x, 16) || (st % 8) != 0 || (sh % 8) != 0) return JF_ERR_ARG;
  if (!aligned(data, 16) || !aligned(scales, 4)) return JF_ERR_ARG;
  return JF_OK;
}

static jf_status_t launch_pack(const PackSide& k, const PackSide* v, int dtype, int64_t T, int H,
                               const int64_t* slots, int64_t num_slots, int gs, cudaStream_t stream) {
  if (T < 0 || H <= 0 || num_slots <= 0 || !slots) return JF_ERR_ARG;
  if (gs != 64 && gs != 128) return JF_ERR_UNSUPPORTED;
  if (dtype != JF_DTYPE_BF16 && dtype != JF_DTYPE_FP16) return JF_ERR_UNSUPPORTED;
  if (T == 0) return JF_OK;
  const int64_t rows = T * H;
  const int64_t warps = (rows + 2 * kPairsPerWarp - 1) / (2 * kPairsPerWarp);
  const int64_t ctas = (warps + kWarpsPerCta - 1) / kWarpsPerCta;
  if (ctas > 0x7FFFFFFF) return JF_ERR_UNSUPPORTED;
  dim3 grid(static_cast<unsigned>(ctas), v ? 2 : 1);
  dim3 block(kWarpsPerCta * 32);
  const PackSide s1 = v ? *v : k;
#define JF_LAUNCH(DT, GS) pack_append_kernel<DT, GS><<<grid, block, 0, stream>>>(k, s1, T, H, slots, num_slots)
  if (dtype == JF_DTYPE_BF16) {
    if (gs == 64) JF_LAUNCH(JF_DTYPE_BF16, 64); else JF_LAUNCH(JF_DTYPE_BF16, 128);
  } else {
    if (gs == 64) JF_LAUNCH(JF_DTYPE_FP16, 64); else JF_LAUNCH(JF_DTYPE_FP16, 128);
  }
#undef JF_LAUNCH
  JF_CUDA_TRY(cudaGetLastError());
  return JF_OK;
}

}  // namespace jf

extern "C" jf_status_t jf_pack_append(const void* x_tok, int32_t dtype, int64_t T, int32_t H_kv,
                                      int64_t stride_t, int64_t stride_h, const int64_t* slots,
                                      uint8_t* out_data, void* out_scales, int64_t num_slots,
                                      int32_t nbits, int32_t group_size, jf_stream_t stream) {
  jf_status_t st = jf::check_side(x_tok, stride_t, stride_h, out_data, out_scales, nbits);
  if (st != JF_OK) return st;
  jf::PackSide k{x_tok, stride_t, stride_h, out_data, static_cast<uint16_t*>(out_scales), nbits, nullptr};
  return jf::launch_pack(k, nullptr, dtype, T, H_kv, slots, num_slots, group_size,
                         static_cast<cudaStream_t>(stream));
}

extern "C" jf_status_t jf_pack_append_kv(const void* key_tok, const void* value_tok, int32_t dtype,
                                         int64_t T, int32_t H_kv, int64_t k_stride_t, int64_t k_stride_h,
                                         int64_t v_stride_t, int64_t v_stride_h, const int64_t* slots,
                                         uint8_t* k_data, void* k_scales, uint8_t* v_data, void* v_scales,
                                         int64_t num_slots, int32_t k_bits, int32_t v_bits,
                                         int32_t group_size, jf_stream_t stream) {
  jf_status_t st = jf::check_side(key_tok, k_stride_t, k_stride_h, k_data, k_scales, k_bits);
  if (st != JF_OK) return st;
  st = jf::check_side(value_tok, v_stride_t, v_stride_h, v_data, v_scales, v_bits);
  if (st != JF_OK) return st;
  jf::PackSide k{key_tok, k_stride_t, k_stride_h, k_data, static_cast<uint16_t*>(k_scales), k_bits, nullptr};
  jf::PackSide v{value_tok, v_stride_t, v_stride_h, v_data, static_cast<uint16_t*>(v_scales), v_bits, nullptr};
  return jf::launch_pack(k, &v, dtype, T, H_kv, slots, num_slots, group_size,
                         static_cast<cudaStream_t>(stream));
}

extern "C" jf_status_t jf_pack_append_kv_mirror(const void* key_tok, const void* value_tok, int32_t dtype,
                                                int64_t T, int32_t H_kv, int64_t k_stride_t, int64_t k_stride_h,
                                                int64_t v_stride_t, int64_t v_stride_h, const int64_t* slots,
                                                uint8_t* k_data, void* k_scales, uint8_t* v_data, void* v_scales,
                                                int64_t num_slots, int32_t k_bits, int32_t v_bits,
                                                int32_t group_size, void* k_mirror, void* v_mirror,
                                                jf_stream_t stream) {
  jf_status_t st = jf::check_side(key_tok, k_stride_t, k_stride_h, k_data, k_scales, k_bits);
  if (st != JF_OK) return st;
  st = jf::check_side(value_tok, v_stride_t, v_stride_h, v_data, v_scales, v_bits);
  if (st != JF_OK) return st;
  if (!k_mirror || !v_mirror || !jf::aligned(k_mirror, 16) || !jf::aligned(v_mirror, 16)) return JF_ERR_ARG;
  jf::PackSide k{key_tok, k_stride_t, k_stride_h, k_data, static_cast<uint16_t*>(k_scales), k_bits,
                 static_cast<uint16_t*>(k_mirror)};
  jf::PackSide v{value_tok, v_stride_t, v_stride_h, v_data, static_cast<uint16_t*>(v_scales), v_bits,
                 static_cast<uint16_t*>(v_mirror)};
  return jf::launch_pack(k, &v, dtype, T, H_kv, slots, num_slots, group_size,
                         static_cast<cudaStream_t>(stream));
}
