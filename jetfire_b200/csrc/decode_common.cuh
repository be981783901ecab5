// Workspace layout and launch geometry shared by the scan, select and finish kernels.
#pragma once

#include "jf_common.cuh"

namespace jf {

constexpr int kScanWarps = 4;         // consumer warps per scan CTA; each owns whole pages
constexpr int kHeadsPad = 8;          // query heads of one KV head, padded to the MMA N
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kMinusBig = -1.0e30f; // finite stand-in for "no score seen yet"

struct ModeInfo {
  int k_bits, v_bits, group_size, ng, k_row, v_row;
};
__host__ __device__ inline ModeInfo mode_info(int mode) {
  if (mode == JF_MODE_K4V4) return ModeInfo{4, 4, 128, 1, 64, 64};
  return ModeInfo{3, 2, 64, 2, 48, 32};
}

// The scan puts the query heads of one KV head on the eight columns of an MMA.  A GQA group of
// 16 (the reference's limit, jetfire_vllm/adapter/release_policy.py:31-34) is handled as two
// "virtual" KV heads of eight query heads each that read the same cache rows: every kernel sees
// H_kv << shift heads of G >> shift query heads and indexes the cache with (head >> shift).
struct HeadGeom { int H_kv, G, shift; };
__host__ __device__ inline HeadGeom head_geom(int H_q, int H_kv) {
  const int G = H_q / H_kv;
  const int shift = (G > kHeadsPad) ? 1 : 0;
  return HeadGeom{H_kv << shift, G >> shift, shift};
}

// Resident scan CTAs per SM (set by registers / shared memory of the kernel variant).
__host__ __device__ inline int scan_ctas_per_sm(int mode, int q_dtype) {
  return (mode == JF_MODE_K3V2 && q_dtype == JF_DTYPE_FP16) ? 3 : 4;
}

// How many splits of the page range one (b, h_kv) pair is cut into: as many as fit in ONE
// wave of resident CTAs (a second, partial wave would idle most of the GPU), but at least
// two pages per warp.  Depends only on its arguments, so every launch agrees.
inline int scan_splits(int mode, int q_dtype, int B, int H_kv, int max_S) {
  const int pages = (max_S + JF_BLOCK_SIZE - 1) / JF_BLOCK_SIZE;
  const int pairs = B * H_kv;
  int target = (num_sms() * scan_ctas_per_sm(mode, q_dtype)) / pairs;
  int cap = pages / 8;
  if (cap < 1) cap = 1;
  if (target > cap) target = cap;
  if (target > 512) target = 512;
  if (target < 1) target = 1;
  return target;
}

// Which select kernel a call takes -- decided from the arguments alone, so that the scan (which
// then leaves the maxima of groups of pages: K3V2 pairs of pages, K4V4 pages) and the select
// kernel (which then takes its threshold from them and never stages the row) agree.
//   narrow: more rows than multiprocessors -> 512-thread blocks, two per multiprocessor;
//   lean:   the row does not fit one resident chunk of that block (32 positions per thread), there
//           are enough groups for the K-th largest group maximum to be a tight bound, and the
//           score rows are whole pages that 16-byte loads can read.
// Rows of one chunk stay with the kernel that stages them: it is as fast there, and the scan
// saves the few per cent the maxima cost it.
constexpr int kStagedTopK = 2048;   // widest top-k of the kernel that stages the row
struct SelectPlan { bool narrow, lean, supported; };
inline SelectPlan select_plan(const jf_decode_args* a, const float* scores) {
  int sort_n = 512;
  while (sort_n < 2 * a->top_k) sort_n <<= 1;
  SelectPlan pl;
  pl.narrow = a->B * a->H_q > num_sms() && sort_n <= 1024;
  const int groups = (a->max_S + 15) / 16 / (a->mode == JF_MODE_K3V2 ? 2 : 1);
  const bool readable = (a->max_S & 15) == 0 && (reinterpret_cast<uintptr_t>(scores) & 15) == 0;
  pl.lean = readable && a->max_S > 32 * (pl.narrow ? 512 : 1024) && groups >= 4 * a->top_k;
  // A top-k above kStagedTopK has no room for its sort buffer beside a staged row: such calls
  // always take the kernel that stages nothing (with few groups its histogram tier gives way to
  // the exact radix tier over the row in L2).  pl.supported is false if they cannot.
  pl.supported = a->top_k <= kStagedTopK || readable;
  if (a->top_k > kStagedTopK) { pl.lean = readable; pl.narrow = false; }
  return pl;
}

struct Workspace {
  int32_t* status;   // status record: 64-bit tag, then the error code (see report_status)
  float* part_o;     // [B][H_kv][splits][8][128]
  float* part_m;     // [B][H_kv][splits][8]
  float* part_l;     // [B][H_kv][splits][8]
  float* part_smax;  // [B][H_kv][splits][2]  largest K group scale seen (per group)
  float* pmax;       // [B][H_q][page_max_stride] largest approximate score of every pair of 16-token pages (K3V2) / every page (K4V4)
  float* scores;     // [B][H_q][max_S] approximate scores
  uint64_t bytes;
};

__host__ __device__ inline uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }
// entries per row of the page maxima, rounded up to whole float4s: K3V2 one per pair of 16-token
// pages, K4V4 one per page
__host__ __device__ inline int page_max_stride(int mode, int max_S) {
  const int group = (mode == JF_MODE_K3V2) ? 2 * JF_BLOCK_SIZE : JF_BLOCK_SIZE;
  return (((max_S + group - 1) / group) + 3) & ~3;
}

// Sized for the variant with the most splits (bf16 query), so one workspace serves both dtypes.
inline Workspace carve_workspace(void* base, int mode, int B, int H_q, int H_kv, int max_S, int /*top_k*/, bool need_scores) {
  const HeadGeom hg = head_geom(H_q, H_kv);
  const uint64_t splits = scan_splits(mode, JF_DTYPE_BF16, B, hg.H_kv, max_S);
  const uint64_t pairs = static_cast<uint64_t>(B) * hg.H_kv * splits;
  uint64_t off = 0;
  uint8_t* p = static_cast<uint8_t*>(base);
  Workspace w{};
  w.status = reinterpret_cast<int32_t*>(p + off);   off = align_up(off + 256, 256);
  w.part_o = reinterpret_cast<float*>(p + off);     off = align_up(off + pairs * kHeadsPad * JF_HEAD_DIM * 4, 256);
  w.part_m = reinterpret_cast<float*>(p + off);     off = align_up(off + pairs * kHeadsPad * 4, 256);
  w.part_l = reinterpret_cast<float*>(p + off);     off = align_up(off + pairs * kHeadsPad * 4, 256);
  w.part_smax = reinterpret_cast<float*>(p + off);  off = align_up(off + pairs * 2 * 4, 256);
  w.pmax = reinterpret_cast<float*>(p + off);
  off = align_up(off + static_cast<uint64_t>(B) * H_q * page_max_stride(mode, max_S) * 4, 256);
  w.scores = reinterpret_cast<float*>(p + off);
  if (need_scores) off = align_up(off + static_cast<uint64_t>(B) * H_q * max_S * 4, 256);
  w.bytes = off;
  return w;
}

// Status record at the start of the workspace.  A kernel whose bounded wait ran out writes
// the code and then the tag; a record without the tag reads as "no error", so a workspace
// needs no initialisation and no launch has to clear it.  jf_decode_status reads the record
// and clears it.
constexpr unsigned long long kStatusTag = 0x4A46535441545553ull;  // "JFSTATUS"
// Word 4 of the record: written by every scan -- this value if it left page maxima, 0 if not --
// and checked by the select kernel that works from them, so that a select whose arguments do not
// match the scan's reports JF_ERR_STATE (and selects nothing) instead of reading stale maxima.
constexpr int32_t kPageMaxTag = 0x504D4158;  // "PMAX"
#ifdef __CUDACC__
__device__ __forceinline__ void report_status(int32_t* status, int code) {
  status[2] = code;
  __threadfence();
  *reinterpret_cast<unsigned long long*>(status) = kStatusTag;
}
#endif

jf_status_t validate_decode_args(const jf_decode_args* a);
// device address of the library's built-in scratch array on the current device (decode_static.cu)
jf_status_t static_scratch_address(void** out);

}  // namespace jf
