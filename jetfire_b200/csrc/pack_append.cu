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
// One warp owns a (token, kv-head) row: lane l holds elements 4l..4l+3 (one 8-byte
// load); four rows per warp are loaded before any is processed so that enough bytes
// are in flight per SM.  HBM-bound: 256 B read + 36..66 B written per row.
#include "jf_common.cuh"

namespace jf {

constexpr int kRowsPerWarp = 4;
constexpr int kWarpsPerCta = 8;

struct PackSide {
  const void* x;
  int64_t stride_t, stride_h;
  uint8_t* data;
  uint16_t* scales;
  int nbits;
};

template <int DT, int NBITS, int GS>
__device__ __forceinline__ void pack_row(uint2 raw, uint8_t* __restrict__ out_row,
                                         uint16_t* __restrict__ scale_row, int lane) {
  constexpr int QMAX = (1 << (NBITS - 1)) - 1;
  constexpr int OFF = 1 << (NBITS - 1);
  float f[4];
  f[0] = Elem<DT>::to_f32(raw.x & 0xFFFF);
  f[1] = Elem<DT>::to_f32(raw.x >> 16);
  f[2] = Elem<DT>::to_f32(raw.y & 0xFFFF);
  f[3] = Elem<DT>::to_f32(raw.y >> 16);
  float amax = fmaxf(fmaxf(fabsf(f[0]), fabsf(f[1])), fmaxf(fabsf(f[2]), fabsf(f[3])));
#pragma unroll
  for (int o = 1; o < GS / 4; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, o));
  const float scale = fmaxf(__fdiv_rn(amax, static_cast<float>(QMAX)), 1e-8f);
  const uint16_t sb = __bfloat16_as_ushort(__float2bfloat16_rn(scale));
  const float sf = bf16_bits_to_f32(sb);
  uint32_t c[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float q = rintf(__fdiv_rn(f[i], sf));
    q = fminf(fmaxf(q, -static_cast<float>(QMAX)), static_cast<float>(QMAX));
    c[i] = static_cast<uint32_t>(static_cast<int>(q) + OFF);
  }
  // scales: one per group, written by the group's first lane
  if (GS == 64) {
    const uint32_t hi = __shfl_sync(0xFFFFFFFFu, static_cast<uint32_t>(sb), 16);
    if (lane == 0) *reinterpret_cast<uint32_t*>(scale_row) = static_cast<uint32_t>(sb) | (hi << 16);
  } else {
    if (lane == 0) scale_row[0] = sb;
  }
  if (NBITS == 4) {
    const uint32_t two = ((c[0] << 4) | c[1]) | (((c[2] << 4) | c[3]) << 8);
    const uint32_t nxt = __shfl_down_sync(0xFFFFFFFFu, two, 1);
    if ((lane & 1) == 0) reinterpret_cast<uint32_t*>(out_row)[lane >> 1] = two | (nxt << 16);
  } else if (NBITS == 2) {
    const uint32_t b = (c[0] << 6) | (c[1] << 4) | (c[2] << 2) | c[3];
    const uint32_t b1 = __shfl_down_sync(0xFFFFFFFFu, b, 1);
    const uint32_t b2 = __shfl_down_sync(0xFFFFFFFFu, b, 2);
    const uint32_t b3 = __shfl_down_sync(0xFFFFFFFFu, b, 3);
    if ((lane & 3) == 0) reinterpret_cast<uint32_t*>(out_row)[lane >> 2] = b | (b1 << 8) | (b2 << 16) | (b3 << 24);
  } else {  // NBITS == 3: eight codes -> 24 bits MSB-first, byte p of group i at out_row[16 p + i]
    const uint32_t c12 = (c[0] << 9) | (c[1] << 6) | (c[2] << 3) | c[3];
    const uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, c12, 1);
    const uint32_t w24 = (c12 << 12) | other;  // valid on even lanes (group lane/2)
    const uint32_t wb = __shfl_down_sync(0xFFFFFFFFu, w24, 2);
    const uint32_t wc = __shfl_down_sync(0xFFFFFFFFu, w24, 4);
    const uint32_t wd = __shfl_down_sync(0xFFFFFFFFu, w24, 6);
    if ((lane & 7) == 0) {
      const int j = lane >> 3;  // word index inside a plane: groups 4j..4j+3
      uint32_t* o32 = reinterpret_cast<uint32_t*>(out_row);
#pragma unroll
      for (int p = 0; p < 3; ++p) {
        const int sh = 16 - 8 * p;
        o32[4 * p + j] = ((w24 >> sh) & 255u) | (((wb >> sh) & 255u) << 8) | (((wc >> sh) & 255u) << 16) |
                         (((wd >> sh) & 255u) << 24);
      }
    }
  }
}

template <int DT, int GS>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
pack_append_kernel(PackSide s0, PackSide s1, int64_t T, int H, const int64_t* __restrict__ slots,
                   int64_t num_slots) {
  const PackSide s = (blockIdx.y == 0) ? s0 : s1;
  const int lane = threadIdx.x & 31;
  const int64_t warp = static_cast<int64_t>(blockIdx.x) * kWarpsPerCta + (threadIdx.x >> 5);
  const int64_t rows = T * H;
  const int64_t r0 = warp * kRowsPerWarp;
  if (r0 >= rows) return;
  constexpr int NG = 128 / GS;
  const int dp = 16 * s.nbits;

  uint2 raw[kRowsPerWarp];
  int64_t slot[kRowsPerWarp];
  int hh[kRowsPerWarp];
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    const int64_t r = r0 + i;
    slot[i] = -1;
    hh[i] = 0;
    raw[i] = make_uint2(0u, 0u);
    if (r < rows) {
      const int64_t t = r / H;
      hh[i] = static_cast<int>(r - t * H);
      slot[i] = slots[t];
      if (slot[i] >= num_slots) slot[i] = -1;  // never write outside the cache
      if (slot[i] >= 0) {
        const uint16_t* row = reinterpret_cast<const uint16_t*>(s.x) + t * s.stride_t + hh[i] * s.stride_h;
        raw[i] = __ldg(reinterpret_cast<const uint2*>(row) + lane);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kRowsPerWarp; ++i) {
    if (slot[i] < 0) continue;  // warp-uniform
    const int64_t o = static_cast<int64_t>(hh[i]) * num_slots + slot[i];
    uint8_t* out_row = s.data + o * dp;
    uint16_t* scale_row = s.scales + o * NG;
    if (s.nbits == 3) pack_row<DT, 3, GS>(raw[i], out_row, scale_row, lane);
    else if (s.nbits == 2) pack_row<DT, 2, GS>(raw[i], out_row, scale_row, lane);
    else pack_row<DT, 4, GS>(raw[i], out_row, scale_row, lane);
  }
}

static jf_status_t check_side(const void* x, int64_t st, int64_t sh, const void* data, const void* scales, int nbits) {
  if (!x || !data || !scales) return JF_ERR_ARG;
  if (nbits < 2 || nbits > 4) return JF_ERR_UNSUPPORTED;
  if (!aligned(x, 8) || (st % 4) != 0 || (sh % 4) != 0) return JF_ERR_ARG;
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
  const int64_t warps = (rows + kRowsPerWarp - 1) / kRowsPerWarp;
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
  jf::PackSide k{x_tok, stride_t, stride_h, out_data, static_cast<uint16_t*>(out_scales), nbits};
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
  jf::PackSide k{key_tok, k_stride_t, k_stride_h, k_data, static_cast<uint16_t*>(k_scales), k_bits};
  jf::PackSide v{value_tok, v_stride_t, v_stride_h, v_data, static_cast<uint16_t*>(v_scales), v_bits};
  return jf::launch_pack(k, &v, dtype, T, H_kv, slots, num_slots, group_size,
                         static_cast<cudaStream_t>(stream));
}
