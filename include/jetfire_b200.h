/*
 * jetfire_b200 -- C ABI of the B200-native JetFire decode hot path.
 *
 * Plain pointers and sizes only; no torch or CUDA types.  `stream` arguments are a
 * `cudaStream_t` passed as `void*` (NULL = the legacy default stream).  Every device
 * pointer must belong to the CUDA device that is current on the calling thread.
 * Functions return 0 on success, a negative value for an argument error (nothing was
 * launched) and a positive value for a runtime error.  Nothing here throws, and no
 * function allocates device memory: callers hand in a workspace whose size
 * `jf_decode_workspace_bytes` reports.
 *
 * Each entry point names the JetFire interface it replaces (paths inside the JetFire
 * project).
 */
#ifndef JETFIRE_B200_H_
#define JETFIRE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t jf_status_t;
typedef void*   jf_stream_t;

enum {
  JF_OK               = 0,
  JF_ERR_ARG          = -1, /* null pointer, bad shape, misaligned pointer          */
  JF_ERR_UNSUPPORTED  = -2, /* valid request outside the built envelope              */
  JF_ERR_WORKSPACE    = -3, /* workspace missing or too small                        */
  JF_ERR_STATIC_LIMIT = -4, /* request needs more scratch than the built-in buffer   */
  JF_ERR_CUDA         = 1,  /* a CUDA call failed; see jf_last_cuda_error()          */
  JF_ERR_TIMEOUT      = 2,  /* a bounded wait ran out (device status word or host)   */
  JF_ERR_STATE        = 3   /* object used in the wrong state (host side), or -- through
                               jf_decode_status -- a select whose arguments do not match
                               those of the scan that filled the workspace             */
};

enum { JF_DTYPE_BF16 = 0, JF_DTYPE_FP16 = 1 };

/* Quantisation modes of the release matrix that this library builds
 * (jetfire_vllm/bench/artifact_performance.py:45): K3V2 = SymInt3K_SymInt2V with
 * group 64, K4V4 = SymInt4K_SymInt4V with group 128. */
enum { JF_MODE_K3V2 = 0, JF_MODE_K4V4 = 1 };

/* jf_decode_scan can run the two halves of the reference's pipeline separately, for callers
 * that keep the reference's Stage A / Stage B call structure:
 *   JF_SCAN_K_ONLY  scores (into args->scores and the workspace) and the softmax sums; reads
 *                   q and the K cache only -- with jf_topk_select this is Stage A
 *                   (int3_qk_scores_topk, jetfire_vllm/csrc/int3_qk_scores.cu:562-633);
 *   JF_SCAN_V_ONLY  output partials from the scores in args->scores (an input here) and the
 *                   V cache only -- with jf_decode_finish this is Stage B
 *                   (int2_softmax_v_with_pre_corr_wvs2, csrc/int2_softmax_v.cu:792-901).
 * Both give the bits of the one-pass scan. */
enum { JF_SCAN_ALL = 0, JF_SCAN_K_ONLY = 1, JF_SCAN_V_ONLY = 2 };

/* Weights of the softmax.V product.  JF_STAGE_B_FP32: full-precision weights, the reference's
 * wvs2 / wvs2_scores kernels (csrc/int2_softmax_v.cu:681-705, csrc/int4_softmax_v.cu:599-817).
 * JF_STAGE_B_INT8P (K4V4 only): the reference's plan for a configured batch above 1
 * (jetfire_vllm/adapter/release_policy.py:443-451): per tile of 32 tokens and query head,
 * p * v_scale is rounded to 127 levels of the tile's largest value, tiles laid out over 8
 * splits of ceil(max_S / 8) positions (csrc/int8tc_softmax_v_fused.cu:62, 1049-1053, 1203-1311). */
enum { JF_STAGE_B_FP32 = 0, JF_STAGE_B_INT8P = 1 };

#define JF_HEAD_DIM   128
#define JF_BLOCK_SIZE 16
#define JF_MAX_TOP_K  4096  /* above 2048: only for score rows of whole pages (max_S a multiple of 16,
                               a 16-byte aligned scores pointer), else JF_ERR_UNSUPPORTED */
#define JF_MAX_GROUP  16    /* query heads per KV head: 1..8, or 16 (handled as two halves of 8) */

const char* jf_status_string(jf_status_t st);
int32_t     jf_version(void);
/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
int32_t     jf_last_cuda_error(void);

/* ---------------------------------------------------------------------------------
 * Quantise-on-append.
 * Replaces the Triton writers fused_quant_write_int{2,3,4}_sym
 * (jetfire_vllm/kernels/fused_quant_write.py:242, :337, :746) with the arithmetic of
 * the torch reference quantize_and_pack (jetfire_vllm/kernels/intN_pack.py:60-107):
 * IEEE divide, round-half-even, scale rounded to bf16 before the divide.
 *
 * x_tok      (T, H_kv, 128) bf16/fp16 device, element strides stride_t / stride_h,
 *            innermost contiguous, rows 16-byte aligned (strides multiples of 8 elements)
 * slots      (T,) int64 device; row t goes to out[h, slots[t]]; negative = skip
 * out_data   (H_kv, num_slots, 128*nbits/8) uint8 device
 * out_scales (H_kv, num_slots, 128/group_size) bf16 device
 * ------------------------------------------------------------------------------- */
jf_status_t jf_pack_append(const void* x_tok, int32_t dtype, int64_t T, int32_t H_kv,
                           int64_t stride_t, int64_t stride_h, const int64_t* slots,
                           uint8_t* out_data, void* out_scales, int64_t num_slots,
                           int32_t nbits, int32_t group_size, jf_stream_t stream);

/* K and V of the same tokens in one launch (the reference's
 * fused_quant_write_int4_sym_kv, jetfire_vllm/kernels/fused_quant_write.py:552-617,
 * generalised to any K/V bit pair). */
jf_status_t jf_pack_append_kv(const void* key_tok, const void* value_tok, int32_t dtype,
                              int64_t T, int32_t H_kv,
                              int64_t k_stride_t, int64_t k_stride_h,
                              int64_t v_stride_t, int64_t v_stride_h,
                              const int64_t* slots,
                              uint8_t* k_data, void* k_scales, uint8_t* v_data, void* v_scales,
                              int64_t num_slots, int32_t k_bits, int32_t v_bits,
                              int32_t group_size, jf_stream_t stream);

/* ---------------------------------------------------------------------------------
 * Appending to the host mirror.
 *
 * The reference keeps every appended K/V row in full precision in host memory
 * (k_shadow / v_shadow (H_kv, num_slots, 128) 16-bit, jetfire_vllm/adapter/
 * cache_store.py:311-323) and fills it per append with a device-to-host copy, a host
 * synchronisation and an index_copy_ (:746-756), or under CUDA graphs with pinned staging
 * and a host callback (:616-640; create_shadow_append_submit_ctx and
 * stream_submit_shadow_append, jetfire_vllm/csrc/cpu_topk_attn.cpp:1611-1665, bindings
 * :2509-2663).  Two replacements, both ordered by the stream alone:
 *
 * jf_pack_append_kv_mirror: the packing kernel also stores each live row's 256 raw bytes to
 *   k_mirror / v_mirror, DEVICE-VISIBLE pointers to the mirrors (mapped pinned host memory
 *   from jf_alloc_mapped, or an existing allocation made visible with jf_map_host; device
 *   memory works too).  The mirror's element type is the tokens' (rows are copied bit for
 *   bit).  Rows are in host memory when the stream reaches the point after the launch.
 *
 * jf_stream_mirror_append: for mirrors in ordinary host memory.  A context owns mapped
 *   pinned staging for max_tokens tokens; the call enqueues, per chunk of max_tokens, one
 *   kernel that writes rows, slots and count into the staging and one host callback that
 *   scatters them into the mirror.  Negative or out-of-range slots are skipped.  The
 *   context must outlive the stream work that uses it (synchronise before destroying).
 * ------------------------------------------------------------------------------- */
jf_status_t jf_pack_append_kv_mirror(const void* key_tok, const void* value_tok, int32_t dtype,
                                     int64_t T, int32_t H_kv,
                                     int64_t k_stride_t, int64_t k_stride_h,
                                     int64_t v_stride_t, int64_t v_stride_h,
                                     const int64_t* slots,
                                     uint8_t* k_data, void* k_scales, uint8_t* v_data, void* v_scales,
                                     int64_t num_slots, int32_t k_bits, int32_t v_bits,
                                     int32_t group_size, void* k_mirror, void* v_mirror,
                                     jf_stream_t stream);
jf_status_t jf_mirror_append_ctx_create(void* k_shadow, void* v_shadow, int32_t H_kv,
                                        int64_t num_slots, int64_t max_tokens, int64_t* handle);
jf_status_t jf_mirror_append_ctx_destroy(int64_t handle);
/* rows written / skipped and chunks scattered so far (any pointer may be null) */
jf_status_t jf_mirror_append_ctx_stats(int64_t handle, int64_t* rows_written,
                                       int64_t* rows_skipped, int64_t* chunks);
jf_status_t jf_stream_mirror_append(jf_stream_t stream, int64_t handle, const void* key_tok,
                                    const void* value_tok, int64_t T,
                                    int64_t k_stride_t, int64_t k_stride_h,
                                    int64_t v_stride_t, int64_t v_stride_h,
                                    const int64_t* slots);
/* The reference's own staged form (create_shadow_append_submit_ctx / stream_submit_shadow_append,
 * jetfire_vllm/csrc/cpu_topk_attn.cpp:1611-1665, 2186-2248): the caller owns pinned host staging
 * k_append / v_append (T, H_kv, 128) 16-bit and slots (T,) int64 and fills them with its own
 * stream-ordered copies; `submit` queues a host callback that scatters the staged rows into the
 * mirror (k_shadow / v_shadow (H_kv, num_slots, 128)), skipping negative or out-of-range slots.
 * The context and the buffers must outlive every stream operation that refers to them. */
jf_status_t jf_shadow_append_ctx_create(const void* k_append, const void* v_append,
                                        const int64_t* slots, int64_t T, int32_t H_kv,
                                        void* k_shadow, void* v_shadow, int64_t num_slots,
                                        int64_t* handle);
jf_status_t jf_shadow_append_ctx_destroy(int64_t handle);
jf_status_t jf_shadow_append_ctx_calls(int64_t handle, int64_t* calls);
jf_status_t jf_stream_submit_shadow_append(jf_stream_t stream, int64_t handle);
/* 64-bit store to device-visible memory in stream order (stream_write_value64,
 * jetfire_vllm/csrc/cpu_topk_attn.cpp:1293-1312); device_ptr 8-byte aligned. */
jf_status_t jf_stream_write_value64(jf_stream_t stream, void* device_ptr, int64_t value);
/* Page-lock an existing host allocation and return the pointer the GPU sees it at. */
jf_status_t jf_map_host(void* host_ptr, uint64_t bytes, void** device_ptr);
jf_status_t jf_unmap_host(void* host_ptr);

/* ---------------------------------------------------------------------------------
 * Fused low-bit decode attention.
 *
 * One call of jf_decode_fused does what the reference spreads over Stage A
 * (int3_qk_scores_topk, jetfire_vllm/csrc/int3_qk_scores.cu:562-633;
 * int8tc_qk_scores_topk_stats, csrc/int8tc_qk_scores.cu:2426-2482) and Stage B
 * (int2_softmax_v_with_pre_corr_wvs2, csrc/int2_softmax_v.cu:792-901;
 * int8tc_softmax_v_with_pre_corr_reg_stats, csrc/int8tc_softmax_v_fused.cu:1591-1734),
 * in the single-call shape the reference defines for int2_fused_attn_topk
 * (csrc/int2_fused_attn_topk.cu:404).  The three phases can also be called one by one.
 * ------------------------------------------------------------------------------- */
typedef struct jf_decode_args {
  int32_t mode;          /* JF_MODE_*                                              */
  int32_t q_dtype;       /* JF_DTYPE_* of q                                        */
  int32_t B, H_q, H_kv;  /* H_q / H_kv in 1..8 or 16                               */
  int32_t max_S;         /* positions [0, min(seq_lens[b], max_S)) are attended    */
  int32_t block_size;    /* must be 16                                             */
  int32_t top_k;         /* 1..JF_MAX_TOP_K                                        */
  int32_t max_blocks;    /* row stride of block_table, >= ceil(max_S / 16)         */
  int32_t scan_parts;    /* JF_SCAN_*: what jf_decode_scan computes (0 = everything) */
  float   attn_scale;
  int32_t stage_b;       /* JF_STAGE_B_*: arithmetic of the weights that meet V     */
  int64_t num_slots;     /* slots per KV head in the packed cache                  */
  const void*    q;            /* (B, H_q, 128) contiguous (may be NULL for JF_SCAN_V_ONLY) */
  const uint8_t* k_data;       /* (H_kv, num_slots, 48 | 64)                       */
  const void*    k_scales;     /* (H_kv, num_slots, NG) bf16                       */
  const uint8_t* v_data;       /* (H_kv, num_slots, 32 | 64)                       */
  const void*    v_scales;     /* (H_kv, num_slots, NG) bf16                       */
  const int64_t* block_table;  /* (B, max_blocks)                                  */
  const int32_t* seq_lens;     /* (B,)                                             */
  /* outputs */
  float*   scores;        /* optional (B, H_q, max_S): approximate scores, -inf past the
                             sequence end; NULL keeps them in the workspace only;
                             JF_SCAN_V_ONLY, select and finish read them from here   */
  int64_t* topk_idx;      /* (B, H_q, top_k) positions, (score desc, index asc), -1 pad */
  int64_t* topk_slots;    /* (B, H_q, top_k) physical slots, -1 pad                */
  float*   o_hat;         /* (B, H_q, 128)                                          */
  float*   o_old_unnorm;  /* (B, H_q, 128)                                          */
  float*   W;             /* (B, H_q)                                               */
  float*   softmax_m;     /* optional (B, H_q) reference point of the softmax       */
  float*   softmax_inv_z; /* optional (B, H_q) 1 / sum exp(s - m)                   */
  void*    workspace;     /* >= jf_decode_workspace_bytes(...), 256-byte aligned    */
  uint64_t workspace_bytes;
  int32_t* topk_slots_i32; /* optional (B, H_q, top_k): the selected slots once more, as 32-bit
                              integers (num_slots < 2^31), for a device-to-host copy of half the
                              size; topk_slots may then be NULL.  No counterpart in the reference. */
} jf_decode_args;

uint64_t    jf_decode_workspace_bytes(int32_t mode, int32_t B, int32_t H_q, int32_t H_kv,
                                      int32_t max_S, int32_t top_k);
/* scan: dequantise, Q.K^T, online softmax, P.V over the packed cache; leaves split
 * partials, approximate scores (also in args->scores if given) and, for long rows, the largest
 * score of every group of 16-token pages in the workspace (what the select kernel of the same
 * arguments takes its threshold from). */
jf_status_t jf_decode_scan(const jf_decode_args* args, jf_stream_t stream);
/* select: exact top-k per query head (csrc/int3_qk_scores.cu:426-554 with a
 * deterministic order and tie rule) + slot translation (:399-417).  Works on what the scan of
 * the same arguments left in the same workspace (split statistics, the maxima of groups of pages)
 * and on the scores it wrote -- not on scores from elsewhere. */
jf_status_t jf_topk_select(const jf_decode_args* args, jf_stream_t stream);
/* finish: merge the split partials into o_hat and the softmax statistics, and compute
 * the approximate contribution of the selected set (W, o_old_unnorm;
 * csrc/int2_softmax_v.cu:738-788). */
jf_status_t jf_decode_finish(const jf_decode_args* args, jf_stream_t stream);
jf_status_t jf_decode_fused(const jf_decode_args* args, jf_stream_t stream);
/* The second kernel of jf_decode_fused on its own (select and finish in one launch), for a scan
 * that was launched separately; same outputs, same bits. */
jf_status_t jf_select_finish(const jf_decode_args* args, jf_stream_t stream);
/* Exact row maximum m and 1 / sum exp(s - m) over positions [0, min(seq_lens[b], max_S)) of
 * stored scores (B, H_q, max_S): the two extra outputs of the reference's
 * int8tc_qk_scores_topk_stats (jetfire_vllm/csrc/int8tc_qk_scores.cu:1790-1800, 2426-2482).
 * An empty row gives m = 0 and 1/Z = 0. */
jf_status_t jf_softmax_stats(const float* scores, const int32_t* seq_lens, float* softmax_m,
                             float* softmax_inv_z, int32_t B, int32_t H_q, int32_t max_S,
                             jf_stream_t stream);
/* Reads back (synchronously, after the stream drained) the status record of the
 * workspace: 0, or JF_ERR_TIMEOUT if a bounded wait inside a kernel ran out since the
 * record was last read.  Reading an error clears it.  The workspace needs no
 * initialisation: only a record that a kernel tagged counts.  With args->workspace NULL it
 * reads (and clears) the record of the calls made through jf_decode_fused_static on the
 * current device instead. */
jf_status_t jf_decode_status(const jf_decode_args* args, jf_stream_t stream);
/* The same reading on a HOST copy of the first JF_STATUS_RECORD_BYTES of the workspace (the
 * record sits at its start), for callers that must not synchronise: they copy the record in
 * the stream after the step and look at the copy once that copy has completed.  Clears nothing. */
#define JF_STATUS_RECORD_BYTES 16
jf_status_t jf_decode_status_of_copy(const void* record_copy);

/* ---------------------------------------------------------------------------------
 * jf_decode_fused without a workspace argument.  No counterpart in the reference (its
 * ops allocate their scratch through torch).
 *
 * For callers that cannot allocate device memory themselves -- code living inside a host
 * application that owns all allocations, code on a path where an allocator call or the
 * synchronisation it may imply is not tolerable, or a process whose device memory is fully
 * planned in advance.  Inputs and outputs are still the caller's; `workspace` and
 * `workspace_bytes` of the argument block are ignored.  The scratch is a fixed
 * JF_STATIC_SCRATCH_BYTES array inside the library image: each GPU that loads the library
 * holds it until the process exits.  A request whose jf_decode_workspace_bytes() exceeds it
 * returns JF_ERR_STATIC_LIMIT (roughly: B * H_q * max_S up to ~15 million score slots, e.g.
 * batch 4 x 32 heads x 64k context).  Mode K3V2 only; K4V4 returns JF_ERR_UNSUPPORTED
 * because its launch path keeps a host-side cache that may allocate.
 * All calls on a GPU share the one array and it keeps the previous call's contents, so
 * calls must not overlap on the same GPU (they would race); results do not depend on what
 * was left behind.  The first call on each device resolves the array's address and should
 * be made before any stream capture begins.  Never calls cudaMalloc / cudaFree.
 * A bounded wait that ran out inside one of its kernels is recorded at the start of the
 * array; read it with jf_decode_status on an argument block whose workspace is NULL.
 * ------------------------------------------------------------------------------- */
#define JF_STATIC_SCRATCH_BYTES (64ull << 20)
jf_status_t jf_decode_fused_static(const jf_decode_args* args, jf_stream_t stream);

/* ---------------------------------------------------------------------------------
 * Correction merge: out = dtype(o_hat + W * float(o_new) - o_old_unnorm).
 * Replaces blend_unnorm_into (jetfire_vllm/csrc/blend.cu:229-290).
 * o_new may be device memory or the device alias of mapped pinned host memory.
 * ------------------------------------------------------------------------------- */
jf_status_t jf_merge_correct(const float* o_hat, const float* o_old_unnorm, const float* W,
                             const void* o_new, void* out, int32_t dtype,
                             int32_t B, int32_t H_q, jf_stream_t stream);

/* ---------------------------------------------------------------------------------
 * Host correction: exact attention over the selected rows of the full-precision host
 * mirror.  Replaces cpu_topk_attn (jetfire_vllm/csrc/cpu_topk_attn.cpp:854-956) and the
 * worker pool of jetfire_vllm/csrc/jetfire_pool.h:69-334.
 *
 * q (B,H_q,128), k_shadow/v_shadow (H_kv,num_slots,128), o_new (B,H_q,128): host memory
 * of `dtype`; head_map may be NULL (then h_kv = h_q / (H_q / H_kv)); ts_buf (B,H_q,K)
 * int64 physical slots, invalid (<0 or >= num_slots) entries are skipped.
 * done_flag, if not NULL, is set to 1 (release + store fence) after o_new is complete.
 * ------------------------------------------------------------------------------- */
jf_status_t jf_cpu_topk_attn(const void* q, const void* k_shadow, const void* v_shadow,
                             const int64_t* head_map, const int64_t* ts_buf, void* o_new,
                             int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                             int64_t num_slots, int32_t K, float scale, int64_t* done_flag);
/* The same with the slots as 32-bit integers (jf_decode_args.topk_slots_i32): half the bytes on
 * the device-to-host copy of the selected slots.  No counterpart in the reference (its slot
 * lists are int64 throughout). */
jf_status_t jf_cpu_topk_attn_i32(const void* q, const void* k_shadow, const void* v_shadow,
                                 const int64_t* head_map, const int32_t* ts_buf, void* o_new,
                                 int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                                 int64_t num_slots, int32_t K, float scale, int64_t* done_flag);
/* Host-side wait for a completion flag written by the correction workers (the host half of
 * wait_and_blend_unnorm_into, jetfire_vllm/csrc/blend.cu:320-376): returns JF_OK once *flag is
 * non-zero, JF_ERR_TIMEOUT after timeout_ms.  Does not touch the GPU. */
jf_status_t jf_wait_flag(const int64_t* flag, int32_t timeout_ms);
jf_status_t jf_set_cpu_attn_threads(int32_t n);
int32_t     jf_get_cpu_attn_threads(void);

/* Asynchronous form: submit returns at once, wait blocks up to timeout_ms
 * (JF_ERR_TIMEOUT if jobs are still running; it can be waited on again).  Up to four jobs
 * can be queued (JF_ERR_STATE when the queue is full); workers move from one job to the
 * next without idling.  jf_pool_wait_timeout waits for every queued job, jf_pool_wait_ticket
 * for one.  Jobs that share a done_flag must not be queued together. */
jf_status_t jf_pool_init(int32_t n_threads);
jf_status_t jf_pool_submit(const void* q, const void* k_shadow, const void* v_shadow,
                           const int64_t* head_map, const int64_t* ts_buf, void* o_new,
                           int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                           int64_t num_slots, int32_t K, float scale, int64_t* done_flag);
jf_status_t jf_pool_submit_ticket(const void* q, const void* k_shadow, const void* v_shadow,
                                  const int64_t* head_map, const int64_t* ts_buf, void* o_new,
                                  int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                                  int64_t num_slots, int32_t K, float scale, int64_t* done_flag,
                                  int64_t* ticket);
jf_status_t jf_pool_submit_ticket_i32(const void* q, const void* k_shadow, const void* v_shadow,
                                      const int64_t* head_map, const int32_t* ts_buf, void* o_new,
                                      int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                                      int64_t num_slots, int32_t K, float scale, int64_t* done_flag,
                                      int64_t* ticket);
jf_status_t jf_pool_wait_timeout(int32_t timeout_ms);
jf_status_t jf_pool_wait_ticket(int64_t ticket, int32_t timeout_ms);
jf_status_t jf_pool_shutdown(void);

/* Stream-ordered form (create_cpu_topk_submit_ctx / stream_submit_cpu_topk_attn /
 * stream_wait_cpu_topk_attn, jetfire_vllm/csrc/cpu_topk_attn.cpp:2147-2312): a context fixes
 * the job's buffers; `submit` queues a host callback on the stream that hands the job to the
 * pool when the stream gets there (after the copy of the selected slots to host memory),
 * `wait` queues one that holds the stream until the job is done, so a merge kernel queued
 * after it reads a finished o_new.  Both callbacks wait at most wait_ms (default 30000); a
 * wait that ran out is reported once by jf_submit_ctx_status.  The context must outlive every
 * stream operation (and CUDA graph) that refers to it. */
jf_status_t jf_submit_ctx_create(const void* q, const void* k_shadow, const void* v_shadow,
                                 const int64_t* head_map, const int64_t* ts_buf, void* o_new,
                                 int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                                 int64_t num_slots, int32_t K, float scale, int64_t* done_flag,
                                 int32_t wait_ms, int64_t* handle);
jf_status_t jf_submit_ctx_create_i32(const void* q, const void* k_shadow, const void* v_shadow,
                                     const int64_t* head_map, const int32_t* ts_buf, void* o_new,
                                     int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                                     int64_t num_slots, int32_t K, float scale, int64_t* done_flag,
                                     int32_t wait_ms, int64_t* handle);
jf_status_t jf_submit_ctx_destroy(int64_t handle);
jf_status_t jf_submit_ctx_status(int64_t handle);
jf_status_t jf_stream_submit_cpu_topk_attn(jf_stream_t stream, int64_t handle);
jf_status_t jf_stream_wait_cpu_topk_attn(jf_stream_t stream, int64_t handle);

/* The correction shared between the host's workers and the GPU.  End to end a decode step is
 * bounded by the workers' random gathers from the cold mirror while the GPU and its host link
 * idle; jf_gpu_topk_attn_rows takes a range of the (sequence, query head) rows -- B * H_q of
 * them, row-major -- off the workers: one block per row reads the selected K and V rows from
 * the mirror through its DEVICE-VISIBLE address (mapped pinned memory: jf_alloc_mapped /
 * jf_map_host), one coalesced 256-byte read each, and writes its rows of o_new on the device.
 * Same arithmetic as jf_cpu_topk_attn in another summation order (agreement to rounding).
 * `topk_slots` is the device slot list (int64, or int32 with slots_are_i32).
 * jf_pool_submit_rows is jf_pool_submit_ticket for a non-empty range of rows; the rest of o_new
 * is left alone.  No counterpart on the reference's release path (its GPU-side correction,
 * jetfire_vllm/csrc/fused_correction.cu, works on a device-resident copy of the rows). */
jf_status_t jf_gpu_topk_attn_rows(const void* q, const void* k_mirror_dev, const void* v_mirror_dev,
                                  const void* topk_slots, int32_t slots_are_i32, void* o_new, int32_t dtype,
                                  int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots, int32_t K, float scale,
                                  int64_t row_begin, int64_t row_end, jf_stream_t stream);
jf_status_t jf_pool_submit_rows(const void* q, const void* k_shadow, const void* v_shadow,
                                const int64_t* head_map, const void* ts_buf, int32_t slots_are_i32,
                                void* o_new, int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                                int64_t num_slots, int32_t K, float scale, int64_t* done_flag,
                                int64_t row_begin, int64_t row_end, int64_t* ticket);

/* Host correction started and joined by the GPU through two words in mapped pinned host memory,
 * with no host function in the stream (each costs two thread hand-overs; a layer's pair costs
 * more than the GPU half of the step).  The reference's counterparts are the device-signal and
 * GPU-wait variants of its graph-mode decode (jetfire_vllm/adapter/decode_path.py:2426-2438,
 * :3061-3064: stream_write_value64 / stream_wait_value64 on a mapped flag); here the wait is a
 * polling kernel with a time budget rather than a stream memory operation that never gives up.
 *   jf_submit_ctx_watch       a dispatcher thread polls *trigger_host; non-zero = clear it and queue
 *                             the context's job (whose completion flag is the context's done_flag)
 *   jf_stream_signal_host     kernel: *done_dev = 0, then *trigger_dev = 1 (after the stream's
 *                             earlier copies of the job's inputs have landed on the host)
 *   jf_stream_wait_host_flag  kernel: one thread polls *flag_dev until non-zero, at most timeout_ms;
 *                             a wait that runs out writes JF_ERR_TIMEOUT to the status record given
 *                             (start of the decode workspace, or NULL) and the stream continues
 * All three are capturable: a replayed graph raises the same trigger word again. */
jf_status_t jf_submit_ctx_watch(int64_t handle, int64_t* trigger_host);
/* The context's job covers rows [row_begin, row_end) only (see jf_pool_submit_rows); before use. */
jf_status_t jf_submit_ctx_set_rows(int64_t handle, int64_t row_begin, int64_t row_end);
jf_status_t jf_submit_ctx_unwatch(int64_t handle);
jf_status_t jf_stream_signal_host(jf_stream_t stream, int64_t* done_dev, int64_t* trigger_dev);
jf_status_t jf_stream_wait_host_flag(jf_stream_t stream, const int64_t* flag_dev, int32_t timeout_ms,
                                     void* status_record);

/* Pinned host memory mapped into the device address space
 * (alloc_mapped_pinned_pair, jetfire_vllm/csrc/cpu_topk_attn.cpp:958-1040). */
jf_status_t jf_alloc_mapped(uint64_t bytes, void** host_ptr, void** device_ptr);
jf_status_t jf_free_mapped(void* host_ptr);
/* Asks the operating system to back a host range with 2 MB pages (madvise MADV_HUGEPAGE on the
 * whole huge pages inside it) -- for mirrors in ordinary host memory, before they are first
 * touched: the host correction's random 256-byte row gathers then miss the TLB far less.  No
 * counterpart in the reference.  JF_ERR_UNSUPPORTED if the system refuses; harmless either way. */
jf_status_t jf_advise_huge_pages(void* ptr, uint64_t bytes);

/* ---- NUMA placement of the mirrors and the correction workers ---------------------------------
 * No counterpart in the reference, which leaves placement to first touch.  On a host with more
 * than one memory node the mirror of a GPU and the workers that gather from it belong on the
 * node that GPU is attached to; elsewhere every gathered row crosses the socket interconnect.
 * The layout is read from sysfs (below $JF_SYSFS_ROOT when set, else /sys).
 *
 * jf_numa_node_count      memory nodes online (1 when the system does not say)
 * jf_numa_node_of_device  node of the GPU's PCI function, -1 when unknown
 * jf_numa_node_cpus       processors of a node, ascending; *count = how many exist
 * jf_bind_memory_to_node  mbind(MPOL_BIND) of the whole pages in the range; before the memory is
 *                         first touched or registered.  JF_ERR_UNSUPPORTED if refused.
 * jf_alloc_mapped_on_node jf_alloc_mapped with the block bound to `node` first (-1: no binding);
 *                         a refused binding still returns memory, placed by first touch
 * jf_set_cpu_attn_node    correction workers run only on that node's processors (-1: anywhere);
 *                         takes effect with the next job */
int32_t     jf_numa_node_count(void);
int32_t     jf_numa_node_of_device(int32_t device);
jf_status_t jf_numa_node_cpus(int32_t node, int32_t* cpus, int32_t capacity, int32_t* count);
jf_status_t jf_bind_memory_to_node(void* ptr, uint64_t bytes, int32_t node);
jf_status_t jf_alloc_mapped_on_node(uint64_t bytes, int32_t node, void** host_ptr, void** device_ptr);
jf_status_t jf_set_cpu_attn_node(int32_t node);
int32_t     jf_get_cpu_attn_node(void);

#ifdef __cplusplus
}
#endif
#endif /* JETFIRE_B200_H_ */
