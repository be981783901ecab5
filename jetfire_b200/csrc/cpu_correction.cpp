// Host top-k correction: exact attention over the selected rows of the full-precision
// KV mirror kept in host DRAM.
//
// Keeps the reference's design (jetfire_vllm/csrc/cpu_topk_attn.cpp:316-479, 602-690,
// 854-956; pool: csrc/jetfire_pool.h:69-334): persistent workers over the (b, h_q) rows
// (claimed one by one from a shared counter rather than split evenly), per row: gather K/V rows by slot, s = (q . K) * scale in fp32,
// softmax with exp, o_new = sum p * V in fp32, rounded to the mirror's 16-bit type;
// invalid slots score -inf, an all-invalid row or a non-positive / non-finite
// normaliser gives zeros; a store fence precedes the completion flag so that results
// written to mapped (write-combined) memory are visible to the GPU.
//
// Differences: plain C ABI, no torch types; the AVX-512-BF16 path is selected at run time
// so one binary runs on hosts with and without it; fp16 mirrors are supported; the SIMD
// path makes two prefetched passes (K rows, then V rows) instead of staging V; workers
// park on a condition variable after a short spin.
#include <atomic>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include <immintrin.h>

#include <cuda_runtime_api.h>

#include "../../include/jetfire_b200.h"
#include "numa_place.h"

namespace {

constexpr int D = JF_HEAD_DIM;

inline float bf16_to_f32(uint16_t b) {
  uint32_t u = static_cast<uint32_t>(b) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FC0;  // NaN
  u += 0x7FFFu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}
inline float fp16_to_f32(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      int e = -1;
      do { man <<= 1; ++e; } while (!(man & 0x400u));
      u = sign | ((127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
  else u = sign | ((exp + 112) << 23) | (man << 13);
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline uint16_t f32_to_fp16(float f) {  // RNE
  uint32_t u;
  std::memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  u &= 0x7FFFFFFFu;
  if (u >= 0x7F800000u) return static_cast<uint16_t>(sign | (u > 0x7F800000u ? 0x7E00u : 0x7C00u));
  if (u >= 0x477FF000u) return static_cast<uint16_t>(sign | 0x7C00u);  // rounds to inf
  if (u < 0x38800000u) {  // subnormal half
    if (u < 0x33000000u) return static_cast<uint16_t>(sign);
    const int shift = 126 - static_cast<int>(u >> 23);
    uint32_t man = (u & 0x7FFFFFu) | 0x800000u;
    const uint32_t lsb = 1u << shift, half = lsb >> 1;
    uint32_t r = man >> shift;
    const uint32_t rem = man & (lsb - 1);
    if (rem > half || (rem == half && (r & 1u))) ++r;
    return static_cast<uint16_t>(sign | r);
  }
  uint32_t r = u - 0x38000000u;
  const uint32_t rem = r & 0x1FFFu;
  r >>= 13;
  if (rem > 0x1000u || (rem == 0x1000u && (r & 1u))) ++r;
  return static_cast<uint16_t>(sign | r);
}

struct Job {
  const uint16_t* q;
  const uint16_t* ks;
  const uint16_t* vs;
  const int64_t* head_map;
  const void* ts;     // selected slots, (B, H_q, K): 64-bit integers, or 32-bit ones when ts_i32
  bool ts_i32;
  uint16_t* o;
  int dtype, B, H_q, H_kv, K;
  int64_t num_slots;
  float scale;
  int64_t* done_flag;
  int64_t row_begin = 0;    // the (sequence, query head) rows [row_begin, row_begin + row_count) of the job;
  int64_t row_count = -1;   // -1: all B * H_q of them
};

struct Scratch {
  std::vector<float> scores;
  std::vector<float> vrows;  // K x 128 fp32 copies of the gathered V rows
  std::vector<int64_t> slots;
};

inline int64_t slot_at(const Job& j, int64_t i) {
  return j.ts_i32 ? static_cast<int64_t>(static_cast<const int32_t*>(j.ts)[i]) : static_cast<const int64_t*>(j.ts)[i];
}

inline float load_elem(const uint16_t* p, int dtype) { return dtype == JF_DTYPE_BF16 ? bf16_to_f32(*p) : fp16_to_f32(*p); }

// ---- row kernels --------------------------------------------------------------------

void finish_row(const Job& j, Scratch& sc, uint16_t* o_bh, bool any_valid, float max_score) {
  const int K = j.K;
  float* scores = sc.scores.data();
  if (!any_valid) { std::memset(o_bh, 0, D * 2); return; }
  float denom = 0.f;
  for (int k = 0; k < K; ++k) {
    scores[k] = std::exp(scores[k] - max_score);
    denom += scores[k];
  }
  if (!(denom > 0.f) || !std::isfinite(denom)) { std::memset(o_bh, 0, D * 2); return; }
  const float inv = 1.0f / denom;
  float out[D];
  for (int i = 0; i < D; ++i) out[i] = 0.f;
  const float* vr = sc.vrows.data();
  for (int k = 0; k < K; ++k) {
    const float w = scores[k] * inv;
    if (w == 0.f) continue;
    const float* v = vr + static_cast<size_t>(k) * D;
    for (int i = 0; i < D; ++i) out[i] += w * v[i];
  }
  if (j.dtype == JF_DTYPE_BF16) for (int i = 0; i < D; ++i) o_bh[i] = f32_to_bf16(out[i]);
  else for (int i = 0; i < D; ++i) o_bh[i] = f32_to_fp16(out[i]);
}

// Portable path (any x86-64 / any dtype).
void row_generic(const Job& j, Scratch& sc, int64_t b, int64_t h) {
  const int K = j.K;
  const int64_t bh = b * j.H_q + h;
  const int G = j.H_q / j.H_kv;
  float qf[D];
  for (int i = 0; i < D; ++i) qf[i] = load_elem(j.q + bh * D + i, j.dtype);
  float* scores = sc.scores.data();
  float* vr = sc.vrows.data();
  float max_score = -INFINITY;
  bool any_valid = false;
  for (int k = 0; k < K; ++k) {
    const int64_t slot = slot_at(j, bh * K + k);
    const int64_t hk = j.head_map ? j.head_map[bh * K + k] : h / G;
    if (slot < 0 || slot >= j.num_slots || hk < 0 || hk >= j.H_kv) {
      scores[k] = -INFINITY;
      std::memset(vr + static_cast<size_t>(k) * D, 0, D * 4);
      continue;
    }
    any_valid = true;
    const uint16_t* kr = j.ks + (hk * j.num_slots + slot) * D;
    const uint16_t* vrow = j.vs + (hk * j.num_slots + slot) * D;
    float dot = 0.f;
    for (int i = 0; i < D; ++i) dot += qf[i] * load_elem(kr + i, j.dtype);
    for (int i = 0; i < D; ++i) vr[static_cast<size_t>(k) * D + i] = load_elem(vrow + i, j.dtype);
    const float s = dot * j.scale;
    scores[k] = s;
    if (s > max_score) max_score = s;
  }
  finish_row(j, sc, j.o + bh * D, any_valid, max_score);
}

// AVX-512 path (bf16 mirrors use vdpbf16ps, which accumulates pairs of bf16 products in
// fp32 as the reference's SIMD kernel does; fp16 mirrors convert and use fp32 FMAs).
// Two passes over the selected rows, each with software prefetch running ahead: pass 1
// reads the K rows and produces the scores, pass 2 reads the V rows and accumulates
// sum p * V in eight zmm registers straight from the 16-bit rows, so nothing is staged.
#define JF_AVX512 __attribute__((target("avx512f,avx512bw,avx512vl,avx512bf16")))

// exp(x) for x <= 0 (x = -inf gives 0): x = n ln2 + r, |r| <= ln2 / 2, degree-7 Taylor
// polynomial in r (truncation error 5e-9 relative), scaled by 2^n with vscalefps.
JF_AVX512 inline __m512 exp_nonpos(__m512 x) {
  const __mmask16 dead = _mm512_cmp_ps_mask(x, _mm512_set1_ps(-104.f), _CMP_LT_OQ);
  x = _mm512_max_ps(_mm512_set1_ps(-104.f), x);  // keeps a NaN in x
  const __m512 n = _mm512_roundscale_ps(_mm512_mul_ps(x, _mm512_set1_ps(1.44269504088896341f)),
                                        _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
  __m512 r = _mm512_fnmadd_ps(n, _mm512_set1_ps(0.693145751953125f), x);
  r = _mm512_fnmadd_ps(n, _mm512_set1_ps(1.42860682030941723e-6f), r);
  __m512 p = _mm512_set1_ps(1.f / 5040.f);
  p = _mm512_fmadd_ps(p, r, _mm512_set1_ps(1.f / 720.f));
  p = _mm512_fmadd_ps(p, r, _mm512_set1_ps(1.f / 120.f));
  p = _mm512_fmadd_ps(p, r, _mm512_set1_ps(1.f / 24.f));
  p = _mm512_fmadd_ps(p, r, _mm512_set1_ps(1.f / 6.f));
  p = _mm512_fmadd_ps(p, r, _mm512_set1_ps(0.5f));
  p = _mm512_fmadd_ps(p, r, _mm512_set1_ps(1.f));
  p = _mm512_fmadd_ps(p, r, _mm512_set1_ps(1.f));
  return _mm512_mask_blend_ps(dead, _mm512_scalef_ps(p, n), _mm512_setzero_ps());
}

template <int DT>
JF_AVX512 inline __m512 load16(const uint16_t* p) {
  const __m256i raw = _mm256_loadu_si256(reinterpret_cast<const __m256i*>(p));
  if (DT == JF_DTYPE_BF16) return _mm512_castsi512_ps(_mm512_slli_epi32(_mm512_cvtepu16_epi32(raw), 16));
  return _mm512_cvtph_ps(raw);
}

template <int DT>
JF_AVX512 void row_avx512(const Job& j, Scratch& sc, int64_t b, int64_t h) {
  // rows requested ahead of use: a row is four lines, a dot product over one takes about 10 ns and
  // memory about 100: measured on 15 cores over two 0.5 GB mirrors, 8 / 16 / 32 / 48 / 64 rows ahead
  // give 397 / 364 / 358 / 347 / 349 us for 256 rows of 512 entries
  constexpr int kAhead = 48;
  const int K = j.K;
  const int64_t bh = b * j.H_q + h;
  const int G = j.H_q / j.H_kv;
  const uint16_t* q = j.q + bh * D;
  uint16_t* o_bh = j.o + bh * D;
  float* scores = sc.scores.data();  // padded to a multiple of 16
  int64_t* slots = sc.slots.data();
  // resolve row indices first so that prefetches can run ahead
  bool any_valid = false;
  for (int k = 0; k < K; ++k) {
    const int64_t slot = slot_at(j, bh * K + k);
    const int64_t hk = j.head_map ? j.head_map[bh * K + k] : h / G;
    const bool ok = !(slot < 0 || slot >= j.num_slots || hk < 0 || hk >= j.H_kv);
    slots[k] = ok ? (hk * j.num_slots + slot) * D : -1;
    any_valid |= ok;
  }
  if (!any_valid) { std::memset(o_bh, 0, D * 2); return; }
  auto prefetch_row = [&](const uint16_t* base, int k) {
    if (k < K && slots[k] >= 0) {
      const char* a = reinterpret_cast<const char*>(base + slots[k]);
      for (int l = 0; l < 4; ++l) _mm_prefetch(a + 64 * l, _MM_HINT_T0);
    }
  };

  // pass 1: scores
  __m512bh qb[4];
  __m512 qf[8];
  if (DT == JF_DTYPE_BF16) for (int i = 0; i < 4; ++i) qb[i] = (__m512bh)_mm512_loadu_si512(q + 32 * i);
  else for (int i = 0; i < 8; ++i) qf[i] = load16<DT>(q + 16 * i);
  for (int k = 0; k < kAhead; ++k) prefetch_row(j.ks, k);
  float max_score = -INFINITY;
  for (int k = 0; k < K; ++k) {
    prefetch_row(j.ks, k + kAhead);
    if (k + kAhead < K && slots[k + kAhead] >= 0) {   // V rows on their way to L2 for pass 2
      const char* a = reinterpret_cast<const char*>(j.vs + slots[k + kAhead]);
      for (int l = 0; l < 4; ++l) _mm_prefetch(a + 64 * l, _MM_HINT_T1);
    }
    if (slots[k] < 0) { scores[k] = -INFINITY; continue; }
    const uint16_t* kr = j.ks + slots[k];
    __m512 acc = _mm512_setzero_ps();
    if (DT == JF_DTYPE_BF16) {
      for (int i = 0; i < 4; ++i) acc = _mm512_dpbf16_ps(acc, qb[i], (__m512bh)_mm512_loadu_si512(kr + 32 * i));
    } else {
      __m512 acc2 = _mm512_setzero_ps();
      for (int i = 0; i < 8; i += 2) {
        acc = _mm512_fmadd_ps(qf[i], load16<DT>(kr + 16 * i), acc);
        acc2 = _mm512_fmadd_ps(qf[i + 1], load16<DT>(kr + 16 * i + 16), acc2);
      }
      acc = _mm512_add_ps(acc, acc2);
    }
    const float s = _mm512_reduce_add_ps(acc) * j.scale;
    scores[k] = s;
    if (s > max_score) max_score = s;
  }
  for (int k = 0; k < kAhead; ++k) prefetch_row(j.vs, k);  // overlaps the softmax below

  // softmax weights (a NaN or +inf score leaves a non-finite normaliser: zeros, as the
  // scalar path and the reference give)
  const int K16 = (K + 15) & ~15;
  for (int k = K; k < K16; ++k) scores[k] = -INFINITY;
  const __m512 vmax = _mm512_set1_ps(max_score);
  __m512 vsum = _mm512_setzero_ps();
  for (int k = 0; k < K16; k += 16) {
    const __m512 e = exp_nonpos(_mm512_sub_ps(_mm512_loadu_ps(scores + k), vmax));
    _mm512_storeu_ps(scores + k, e);
    vsum = _mm512_add_ps(vsum, e);
  }
  const float denom = _mm512_reduce_add_ps(vsum);
  if (!(denom > 0.f) || !std::isfinite(denom)) { std::memset(o_bh, 0, D * 2); return; }
  const float inv = 1.0f / denom;

  // pass 2: o = sum p * V
  __m512 out[8];
  for (int i = 0; i < 8; ++i) out[i] = _mm512_setzero_ps();
  for (int k = 0; k < K; ++k) {
    prefetch_row(j.vs, k + kAhead);
    const float w = scores[k] * inv;
    if (slots[k] < 0 || w == 0.f) continue;
    const uint16_t* vrow = j.vs + slots[k];
    const __m512 wv = _mm512_set1_ps(w);
    for (int i = 0; i < 8; ++i) out[i] = _mm512_fmadd_ps(wv, load16<DT>(vrow + 16 * i), out[i]);
  }
  for (int i = 0; i < 8; ++i) {
    __m256i r;
    if (DT == JF_DTYPE_BF16) r = (__m256i)_mm512_cvtneps_pbh(out[i]);
    else r = _mm512_cvtps_ph(out[i], _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
    _mm256_storeu_si256(reinterpret_cast<__m256i*>(o_bh + 16 * i), r);
  }
}

bool have_avx512bf16() {
  static const bool v = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") &&
                        __builtin_cpu_supports("avx512vl") && __builtin_cpu_supports("avx512bf16");
  return v;
}

// One row of the job (rows are claimed one at a time from the job's counter, so a worker that
// loses its core for a while does not hold up the rest).
void run_row(const Job& j, int64_t i, Scratch& sc) {
  if (sc.scores.size() < static_cast<size_t>(j.K) + 16) sc.scores.resize(static_cast<size_t>(j.K) + 16);
  if (sc.slots.size() < static_cast<size_t>(j.K)) sc.slots.resize(j.K);
  const bool simd = have_avx512bf16();
  if (!simd && sc.vrows.size() < static_cast<size_t>(j.K) * D) sc.vrows.resize(static_cast<size_t>(j.K) * D);
  const int64_t b = i / j.H_q, h = i % j.H_q;
  if (!simd) row_generic(j, sc, b, h);
  else if (j.dtype == JF_DTYPE_BF16) row_avx512<JF_DTYPE_BF16>(j, sc, b, h);
  else row_avx512<JF_DTYPE_FP16>(j, sc, b, h);
}

// ---- worker pool: a short queue of jobs ------------------------------------------------
// Up to kQueue jobs can be submitted ahead.  A worker that finds no rows left in a job moves
// on to the next one at once, without waiting for the others, so the workers stay busy across
// job boundaries (with one job at a time every job ended with a tail of idle workers and began
// with a wake-up).  A job is complete when its last row is; its slot is reused when, in
// addition, every worker has left it.
class Pool {
 public:
  static constexpr int kQueue = 4;
  static constexpr int kSpinBeforeParkUs = 400;

  ~Pool() { shutdown(); }
  int size() const { return n_; }
  int node() const { return node_; }
  bool running() const { return n_ > 0; }

  void start(int n) {
    shutdown();
    std::lock_guard<std::mutex> g(api_);
    n_ = n;
    node_ = jf::worker_node();
    stop_ = false;
    submitted_.store(0);
    completed_.store(0);
    for (auto& sl : slots_) { sl.left.store(n); sl.done_id.store(0); }   // "everyone has left": free
    started_.store(0);
    for (int i = 0; i < n; ++i)
      workers_.emplace_back([this] {
        if (node_ >= 0) jf::pin_this_thread_to_node(node_);   // a refusal leaves the worker unconfined
        started_.fetch_add(1, std::memory_order_release);
        loop();
      });
    // every worker is in place (and confined) before the first job is taken
    const auto t_end = std::chrono::steady_clock::now() + std::chrono::seconds(1);
    while (started_.load(std::memory_order_acquire) < n && std::chrono::steady_clock::now() < t_end) std::this_thread::yield();
  }
  void shutdown() {
    std::lock_guard<std::mutex> g(api_);
    if (n_ == 0) return;
    {
      std::lock_guard<std::mutex> l(m_);
      stop_ = true;
    }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
    workers_.clear();
    n_ = 0;
  }
  // Queues the job; false if the queue is full (its oldest slot is still in use).  `ticket`
  // identifies the job for wait_ticket.
  bool submit(const Job& j, uint64_t* ticket = nullptr) {
    const auto t_end = std::chrono::steady_clock::now() + std::chrono::seconds(2);
    for (;;) {
      std::unique_lock<std::mutex> l(m_);
      const uint64_t id = submitted_.load(std::memory_order_relaxed);
      Slot& sl = slots_[id % kQueue];
      if (id >= kQueue && sl.done_id.load(std::memory_order_acquire) != id - kQueue + 1) return false;  // queue full
      if (sl.left.load(std::memory_order_acquire) != n_) {
        // the slot's job is complete but a worker that lost its core has not stepped past it yet
        l.unlock();
        if (std::chrono::steady_clock::now() > t_end) return false;
        std::this_thread::yield();
        continue;
      }
      sl.job = j;
      sl.total = j.row_count >= 0 ? j.row_count : static_cast<int64_t>(j.B) * j.H_q;
      sl.next_row.store(0, std::memory_order_relaxed);
      sl.rows_done.store(0, std::memory_order_relaxed);
      sl.left.store(0, std::memory_order_relaxed);
      submitted_.store(id + 1, std::memory_order_release);
      if (ticket) *ticket = id;
      break;
    }
    cv_.notify_all();
    return true;
  }
  // true when every submitted job is complete within the timeout
  bool wait(int timeout_ms) {
    return wait_until([this] { return completed_.load(std::memory_order_acquire) == submitted_.load(std::memory_order_acquire); },
                      timeout_ms);
  }
  // true when job `ticket` is complete within the timeout
  bool wait_ticket(uint64_t ticket, int timeout_ms) {
    Slot& sl = slots_[ticket % kQueue];
    return wait_until([&sl, ticket] { return sl.done_id.load(std::memory_order_acquire) >= ticket + 1; }, timeout_ms);
  }

 private:
  struct Slot {
    Job job{};
    int64_t total = 0;
    alignas(64) std::atomic<int64_t> next_row{0};
    alignas(64) std::atomic<int64_t> rows_done{0};
    std::atomic<int> left{0};          // workers that have finished with this job
    std::atomic<uint64_t> done_id{0};  // id + 1 of the last job completed in this slot
  };

  template <typename Pred>
  bool wait_until(Pred done, int timeout_ms) {
    const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (int spin = 0; spin < 20000; ++spin) {
      if (done()) return true;
      _mm_pause();
    }
    std::unique_lock<std::mutex> l(m_);
    return done_cv_.wait_until(l, t_end, done);
  }

  void loop() {
    Scratch sc;
    uint64_t my = 0;   // the next job this worker takes part in
    for (;;) {
      // Spin for the next job, then park.  In a decode loop the jobs of consecutive layers are a
      // GPU step apart (a few hundred microseconds at most); parked workers take tens of
      // microseconds to get going again, so the spin outlasts such a gap.
      bool got = false;
      const auto spin_end = std::chrono::steady_clock::now() + std::chrono::microseconds(kSpinBeforeParkUs);
      for (int spin = 0;; ++spin) {
        if (submitted_.load(std::memory_order_acquire) > my) { got = true; break; }
        _mm_pause();
        if ((spin & 63) == 63 && std::chrono::steady_clock::now() > spin_end) break;
      }
      if (!got) {
        std::unique_lock<std::mutex> l(m_);
        cv_.wait(l, [&] { return stop_ || submitted_.load(std::memory_order_acquire) > my; });
      }
      if (submitted_.load(std::memory_order_acquire) <= my) {   // woken to stop, and nothing left to do
        std::lock_guard<std::mutex> l(m_);
        if (stop_) return;
        continue;
      }
      Slot& sl = slots_[my % kQueue];
      const Job j = sl.job;
      const int64_t total = sl.total;
      for (;;) {
        const int64_t i = sl.next_row.fetch_add(1, std::memory_order_relaxed);
        if (i >= total) break;
        run_row(j, j.row_begin + i, sc);
        _mm_sfence();  // results may sit in write-combined mapped memory
        if (sl.rows_done.fetch_add(1, std::memory_order_acq_rel) + 1 == total) {   // the job's last row
          if (j.done_flag) {
            reinterpret_cast<std::atomic<int64_t>*>(j.done_flag)->store(1, std::memory_order_release);
            _mm_sfence();
          }
          sl.done_id.store(my + 1, std::memory_order_release);
          completed_.fetch_add(1, std::memory_order_acq_rel);
          std::lock_guard<std::mutex> l(m_);
          done_cv_.notify_all();
        }
      }
      sl.left.fetch_add(1, std::memory_order_acq_rel);
      ++my;
    }
  }

  std::mutex api_, m_;
  std::condition_variable cv_, done_cv_;
  std::vector<std::thread> workers_;
  Slot slots_[kQueue];
  std::atomic<uint64_t> submitted_{0}, completed_{0};
  std::atomic<int> started_{0};
  bool stop_ = false;
  int n_ = 0;
  int node_ = -1;   // processors the workers were confined to when they started
};

Pool& pool() {
  static Pool p;
  return p;
}
std::atomic<int> g_threads{0};

// One hardware thread is left to the thread that submits jobs and drives the GPU.
int default_threads() {
  int n = static_cast<int>(std::thread::hardware_concurrency()) - 1;
  if (n <= 0) n = 1;
  return n > 64 ? 64 : n;
}

jf_status_t make_job(Job& j, const void* q, const void* ks, const void* vs, const int64_t* hm, const void* ts,
                     void* o, int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots, int32_t K,
                     float scale, int64_t* done_flag, bool ts_i32 = false) {
  if (!q || !ks || !vs || !ts || !o) return JF_ERR_ARG;
  if (B <= 0 || H_q <= 0 || H_kv <= 0 || K <= 0 || num_slots <= 0 || H_q % H_kv != 0) return JF_ERR_ARG;
  if (dtype != JF_DTYPE_BF16 && dtype != JF_DTYPE_FP16) return JF_ERR_UNSUPPORTED;
  if (ts_i32 && num_slots > 0x7FFFFFFFll) return JF_ERR_ARG;
  j = Job{static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(ks), static_cast<const uint16_t*>(vs), hm, ts, ts_i32,
          static_cast<uint16_t*>(o), dtype, B, H_q, H_kv, K, num_slots, scale, done_flag};
  return JF_OK;
}

void ensure_pool() {
  int want = g_threads.load();
  if (want <= 0) want = default_threads();
  if (!pool().running() || pool().size() != want || pool().node() != jf::worker_node()) pool().start(want);
}

// The pool with the configured worker count; a change of the count waits for queued jobs first.
jf_status_t ready_pool() {
  int want = g_threads.load();
  if (want <= 0) want = default_threads();
  if (pool().running() && pool().size() == want && pool().node() == jf::worker_node()) return JF_OK;
  if (pool().running() && !pool().wait(30000)) return JF_ERR_TIMEOUT;
  ensure_pool();
  return JF_OK;
}

jf_status_t submit_job(const Job& j, int64_t* ticket) {
  jf_status_t st = ready_pool();
  if (st != JF_OK) return st;
  if (j.done_flag) reinterpret_cast<std::atomic<int64_t>*>(j.done_flag)->store(0, std::memory_order_release);
  uint64_t t = 0;
  if (!pool().submit(j, &t)) return JF_ERR_STATE;   // queue full
  if (ticket) *ticket = static_cast<int64_t>(t);
  return JF_OK;
}

}  // namespace

// Blocks (spin with pauses, then short sleeps) until *flag is non-zero or the time is up.
extern "C" jf_status_t jf_wait_flag(const int64_t* flag, int32_t timeout_ms) {
  if (!flag) return JF_ERR_ARG;
  const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 0 : timeout_ms);
  const volatile int64_t* f = flag;
  for (int spins = 0;; ++spins) {
    if (*f != 0) {
      std::atomic_thread_fence(std::memory_order_acquire);
      return JF_OK;
    }
    if (spins < 20000) {
      _mm_pause();
    } else {
      if (std::chrono::steady_clock::now() > t_end) return JF_ERR_TIMEOUT;
      std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
    if ((spins & 1023) == 1023 && std::chrono::steady_clock::now() > t_end) return (*f != 0) ? JF_OK : JF_ERR_TIMEOUT;
  }
}

extern "C" jf_status_t jf_set_cpu_attn_threads(int32_t n) {
  if (n <= 0 || n > 1024) return JF_ERR_ARG;
  g_threads.store(n);
  return JF_OK;
}
extern "C" int32_t jf_get_cpu_attn_threads(void) {
  const int n = g_threads.load();
  return n > 0 ? n : default_threads();
}

extern "C" jf_status_t jf_pool_init(int32_t n_threads) {
  if (n_threads > 0) g_threads.store(n_threads);
  if (!pool().wait(30000)) return JF_ERR_TIMEOUT;
  ensure_pool();
  return JF_OK;
}

extern "C" jf_status_t jf_pool_submit(const void* q, const void* k_shadow, const void* v_shadow,
                                      const int64_t* head_map, const int64_t* ts_buf, void* o_new, int32_t dtype,
                                      int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots, int32_t K, float scale,
                                      int64_t* done_flag) {
  Job j;
  jf_status_t st = make_job(j, q, k_shadow, v_shadow, head_map, ts_buf, o_new, dtype, B, H_q, H_kv, num_slots, K,
                            scale, done_flag);
  if (st != JF_OK) return st;
  return submit_job(j, nullptr);
}

extern "C" jf_status_t jf_pool_submit_ticket(const void* q, const void* k_shadow, const void* v_shadow,
                                             const int64_t* head_map, const int64_t* ts_buf, void* o_new,
                                             int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots,
                                             int32_t K, float scale, int64_t* done_flag, int64_t* ticket) {
  if (!ticket) return JF_ERR_ARG;
  Job j;
  jf_status_t st = make_job(j, q, k_shadow, v_shadow, head_map, ts_buf, o_new, dtype, B, H_q, H_kv, num_slots, K,
                            scale, done_flag);
  if (st != JF_OK) return st;
  return submit_job(j, ticket);
}

// A range of the job's (sequence, query head) rows only -- rows [row_begin, row_end) of the B * H_q
// in row-major order; the others are left to someone else (jf_gpu_topk_attn_rows) and their part
// of o_new is not touched.  The range must not be empty.
extern "C" jf_status_t jf_pool_submit_rows(const void* q, const void* k_shadow, const void* v_shadow,
                                           const int64_t* head_map, const void* ts_buf, int32_t slots_are_i32,
                                           void* o_new, int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv,
                                           int64_t num_slots, int32_t K, float scale, int64_t* done_flag,
                                           int64_t row_begin, int64_t row_end, int64_t* ticket) {
  if (!ticket) return JF_ERR_ARG;
  Job j;
  jf_status_t st = make_job(j, q, k_shadow, v_shadow, head_map, ts_buf, o_new, dtype, B, H_q, H_kv, num_slots, K,
                            scale, done_flag, slots_are_i32 != 0);
  if (st != JF_OK) return st;
  if (row_begin < 0 || row_end <= row_begin || row_end > static_cast<int64_t>(B) * H_q) return JF_ERR_ARG;
  j.row_begin = row_begin;
  j.row_count = row_end - row_begin;
  return submit_job(j, ticket);
}

extern "C" jf_status_t jf_pool_wait_ticket(int64_t ticket, int32_t timeout_ms) {
  if (ticket < 0) return JF_ERR_ARG;
  if (!pool().running()) return JF_ERR_STATE;
  return pool().wait_ticket(static_cast<uint64_t>(ticket), timeout_ms < 0 ? 0 : timeout_ms) ? JF_OK : JF_ERR_TIMEOUT;
}

extern "C" jf_status_t jf_pool_wait_timeout(int32_t timeout_ms) {
  if (!pool().running()) return JF_OK;
  return pool().wait(timeout_ms < 0 ? 0 : timeout_ms) ? JF_OK : JF_ERR_TIMEOUT;
}

extern "C" jf_status_t jf_pool_shutdown(void) {
  if (pool().running() && !pool().wait(30000)) return JF_ERR_TIMEOUT;
  pool().shutdown();
  return JF_OK;
}

extern "C" jf_status_t jf_cpu_topk_attn(const void* q, const void* k_shadow, const void* v_shadow,
                                        const int64_t* head_map, const int64_t* ts_buf, void* o_new, int32_t dtype,
                                        int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots, int32_t K,
                                        float scale, int64_t* done_flag) {
  jf_status_t st = jf_pool_submit(q, k_shadow, v_shadow, head_map, ts_buf, o_new, dtype, B, H_q, H_kv, num_slots, K,
                                  scale, done_flag);
  if (st != JF_OK) return st;
  return jf_pool_wait_timeout(30000);
}

// The same three calls for slot lists of 32-bit integers (half the bytes on the device-to-host copy).
extern "C" jf_status_t jf_pool_submit_ticket_i32(const void* q, const void* k_shadow, const void* v_shadow,
                                                 const int64_t* head_map, const int32_t* ts_buf, void* o_new,
                                                 int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots,
                                                 int32_t K, float scale, int64_t* done_flag, int64_t* ticket) {
  if (!ticket) return JF_ERR_ARG;
  Job j;
  jf_status_t st = make_job(j, q, k_shadow, v_shadow, head_map, ts_buf, o_new, dtype, B, H_q, H_kv, num_slots, K,
                            scale, done_flag, true);
  if (st != JF_OK) return st;
  return submit_job(j, ticket);
}

extern "C" jf_status_t jf_cpu_topk_attn_i32(const void* q, const void* k_shadow, const void* v_shadow,
                                            const int64_t* head_map, const int32_t* ts_buf, void* o_new, int32_t dtype,
                                            int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots, int32_t K,
                                            float scale, int64_t* done_flag) {
  int64_t ticket = 0;
  jf_status_t st = jf_pool_submit_ticket_i32(q, k_shadow, v_shadow, head_map, ts_buf, o_new, dtype, B, H_q, H_kv,
                                             num_slots, K, scale, done_flag, &ticket);
  if (st != JF_OK) return st;
  return jf_pool_wait_ticket(ticket, 30000);
}

// ---- stream-ordered submit / wait -----------------------------------------------------
// The reference queues the host correction into the CUDA stream with cudaLaunchHostFunc
// (jetfire_vllm/csrc/cpu_topk_attn.cpp:1268-1290, :2239-2312): one callback hands the job to
// the worker pool when the stream reaches it (the selected slots are in host memory by then),
// a later callback blocks the stream until the job is done, so the merge kernel that follows
// sees o_new.  Callbacks run on a driver thread and call no CUDA API.  Both waits are
// bounded; a wait that runs out is recorded in the context and reported by
// jf_submit_ctx_status.
namespace {

struct SubmitCtx {
  Job job;
  std::atomic<int32_t> error{JF_OK};
  int32_t wait_ms = 30000;
  int64_t* trigger = nullptr;         // watched by the dispatcher thread when set (jf_submit_ctx_watch)
  alignas(64) int64_t own_flag = 0;   // completion flag when the caller gave none
};

void CUDART_CB submit_callback(void* ud) {
  auto* c = static_cast<SubmitCtx*>(ud);
  ensure_pool();
  // single job in flight: an earlier layer's job may still be running
  reinterpret_cast<std::atomic<int64_t>*>(c->job.done_flag)->store(0, std::memory_order_release);
  // the queue may be full: wait for it to drain and try again, within the budget
  const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(c->wait_ms);
  for (;;) {
    if (pool().submit(c->job)) return;
    if (!pool().wait(c->wait_ms) || std::chrono::steady_clock::now() > t_end) { c->error.store(JF_ERR_TIMEOUT); return; }
  }
}

// Contexts whose job is started by the GPU: a kernel in the stream stores a non-zero value to the
// context's trigger word (mapped pinned host memory) once the job's inputs have been copied to the
// host; one dispatcher thread polls the trigger words of all watched contexts, clears the word it
// finds set and queues that context's job.  The completion flag goes the other way: the last
// worker sets it, a kernel in the stream polls it (jf_stream_wait_host_flag).  No host function
// in the stream, whose two thread hand-overs per layer cost more than the GPU half of the step.
class Dispatcher {
 public:
  ~Dispatcher() { stop(); }
  void watch(SubmitCtx* c, int64_t* trigger) {
    std::lock_guard<std::mutex> g(mu_);
    c->trigger = trigger;
    reinterpret_cast<std::atomic<int64_t>*>(trigger)->store(0, std::memory_order_release);
    bool present = false;
    for (auto* x : watched_) present |= (x == c);
    if (!present) watched_.push_back(c);
    if (!running_) {
      running_ = true;
      quit_.store(false);
      thread_ = std::thread([this] { loop(); });
    }
  }
  void unwatch(SubmitCtx* c) {
    std::lock_guard<std::mutex> g(mu_);
    for (size_t i = 0; i < watched_.size(); ++i)
      if (watched_[i] == c) { watched_.erase(watched_.begin() + static_cast<long>(i)); break; }
    c->trigger = nullptr;
  }
  void stop() {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (!running_) return;
      running_ = false;
      quit_.store(true);
    }
    thread_.join();
  }

 private:
  void loop() {
    auto last_hit = std::chrono::steady_clock::now();
    for (uint64_t sweep = 0; !quit_.load(std::memory_order_acquire); ++sweep) {
      bool hit = false;
      {
        std::lock_guard<std::mutex> g(mu_);
        for (SubmitCtx* c : watched_) {
          auto* t = reinterpret_cast<std::atomic<int64_t>*>(c->trigger);
          if (t->load(std::memory_order_acquire) == 0) continue;
          t->store(0, std::memory_order_release);
          submit_callback(c);
          hit = true;
        }
      }
      // busy while steps arrive; after 2 ms without one the sweeps thin out so that an idle process
      // does not hold a core (the first step after a pause then waits up to one nap longer)
      if (hit) { last_hit = std::chrono::steady_clock::now(); continue; }
      _mm_pause();
      if ((sweep & 63) != 63) continue;
      const auto idle = std::chrono::steady_clock::now() - last_hit;
      if (idle > std::chrono::seconds(1)) std::this_thread::sleep_for(std::chrono::milliseconds(1));
      else if (idle > std::chrono::milliseconds(2)) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
  std::mutex mu_;
  std::vector<SubmitCtx*> watched_;
  std::thread thread_;
  std::atomic<bool> quit_{false};
  bool running_ = false;
};

Dispatcher& dispatcher() {
  static Dispatcher d;
  return d;
}

// Waits for THIS context's job (its completion flag), not for an idle pool: the next layer's
// job may already be running by the time this callback gets to look.
void CUDART_CB wait_callback(void* ud) {
  auto* c = static_cast<SubmitCtx*>(ud);
  auto* flag = reinterpret_cast<std::atomic<int64_t>*>(c->job.done_flag);
  const auto t_end = std::chrono::steady_clock::now() + std::chrono::milliseconds(c->wait_ms);
  for (int spin = 0;; ++spin) {
    if (flag->load(std::memory_order_acquire) != 0) return;
    if (c->error.load() != JF_OK) return;   // the submit never happened
    if (spin < 20000) { _mm_pause(); continue; }
    if (std::chrono::steady_clock::now() > t_end) { c->error.store(JF_ERR_TIMEOUT); return; }
    std::this_thread::sleep_for(std::chrono::microseconds(20));
  }
}

}  // namespace

extern "C" jf_status_t jf_submit_ctx_create(const void* q, const void* k_shadow, const void* v_shadow,
                                            const int64_t* head_map, const int64_t* ts_buf, void* o_new,
                                            int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots,
                                            int32_t K, float scale, int64_t* done_flag, int32_t wait_ms,
                                            int64_t* handle) {
  if (!handle) return JF_ERR_ARG;
  auto* c = new SubmitCtx();
  jf_status_t st = make_job(c->job, q, k_shadow, v_shadow, head_map, ts_buf, o_new, dtype, B, H_q, H_kv, num_slots, K,
                            scale, done_flag);
  if (st != JF_OK) { delete c; return st; }
  if (!done_flag) c->job.done_flag = &c->own_flag;
  if (wait_ms > 0) c->wait_ms = wait_ms;
  *handle = static_cast<int64_t>(reinterpret_cast<intptr_t>(c));
  return JF_OK;
}

extern "C" jf_status_t jf_submit_ctx_create_i32(const void* q, const void* k_shadow, const void* v_shadow,
                                            const int64_t* head_map, const int32_t* ts_buf, void* o_new,
                                            int32_t dtype, int32_t B, int32_t H_q, int32_t H_kv, int64_t num_slots,
                                            int32_t K, float scale, int64_t* done_flag, int32_t wait_ms,
                                            int64_t* handle) {
  if (!handle) return JF_ERR_ARG;
  auto* c = new SubmitCtx();
  jf_status_t st = make_job(c->job, q, k_shadow, v_shadow, head_map, ts_buf, o_new, dtype, B, H_q, H_kv, num_slots, K,
                            scale, done_flag, true);
  if (st != JF_OK) { delete c; return st; }
  if (!done_flag) c->job.done_flag = &c->own_flag;
  if (wait_ms > 0) c->wait_ms = wait_ms;
  *handle = static_cast<int64_t>(reinterpret_cast<intptr_t>(c));
  return JF_OK;
}

extern "C" jf_status_t jf_submit_ctx_destroy(int64_t handle) {
  if (!handle) return JF_ERR_ARG;
  auto* c = reinterpret_cast<SubmitCtx*>(static_cast<intptr_t>(handle));
  if (c->trigger) dispatcher().unwatch(c);
  delete c;
  return JF_OK;
}

// From now on a non-zero value stored to *trigger_host (by a kernel in a stream: see
// jf_stream_signal_host) starts the context's job; the dispatcher clears the word when it takes
// it.  The word must stay valid until jf_submit_ctx_unwatch / _destroy.
extern "C" jf_status_t jf_submit_ctx_watch(int64_t handle, int64_t* trigger_host) {
  if (!handle || !trigger_host || (reinterpret_cast<uintptr_t>(trigger_host) & 7)) return JF_ERR_ARG;
  ensure_pool();
  dispatcher().watch(reinterpret_cast<SubmitCtx*>(static_cast<intptr_t>(handle)), trigger_host);
  return JF_OK;
}

// Restricts the context's job to the (sequence, query head) rows [row_begin, row_end) -- the others
// being computed elsewhere (jf_gpu_topk_attn_rows); set before the context is used.
extern "C" jf_status_t jf_submit_ctx_set_rows(int64_t handle, int64_t row_begin, int64_t row_end) {
  if (!handle) return JF_ERR_ARG;
  auto* c = reinterpret_cast<SubmitCtx*>(static_cast<intptr_t>(handle));
  if (row_begin < 0 || row_end <= row_begin || row_end > static_cast<int64_t>(c->job.B) * c->job.H_q) return JF_ERR_ARG;
  c->job.row_begin = row_begin;
  c->job.row_count = row_end - row_begin;
  return JF_OK;
}

extern "C" jf_status_t jf_submit_ctx_unwatch(int64_t handle) {
  if (!handle) return JF_ERR_ARG;
  dispatcher().unwatch(reinterpret_cast<SubmitCtx*>(static_cast<intptr_t>(handle)));
  return JF_OK;
}

extern "C" jf_status_t jf_submit_ctx_status(int64_t handle) {
  if (!handle) return JF_ERR_ARG;
  return static_cast<jf_status_t>(reinterpret_cast<SubmitCtx*>(static_cast<intptr_t>(handle))->error.exchange(JF_OK));
}

extern "C" jf_status_t jf_stream_submit_cpu_topk_attn(jf_stream_t stream, int64_t handle) {
  if (!handle) return JF_ERR_ARG;
  ensure_pool();   // threads are started here, not inside the callback
  const cudaError_t e = cudaLaunchHostFunc(static_cast<cudaStream_t>(stream), submit_callback,
                                           reinterpret_cast<void*>(static_cast<intptr_t>(handle)));
  return e == cudaSuccess ? JF_OK : JF_ERR_CUDA;
}

extern "C" jf_status_t jf_stream_wait_cpu_topk_attn(jf_stream_t stream, int64_t handle) {
  if (!handle) return JF_ERR_ARG;
  const cudaError_t e = cudaLaunchHostFunc(static_cast<cudaStream_t>(stream), wait_callback,
                                           reinterpret_cast<void*>(static_cast<intptr_t>(handle)));
  return e == cudaSuccess ? JF_OK : JF_ERR_CUDA;
}

