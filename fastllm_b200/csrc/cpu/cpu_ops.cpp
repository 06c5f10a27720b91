// Native CPU backend: the operators a decoder needs, in C++ with AVX-512 / AVX2 kernels chosen at run time and a
// persistent thread pool with dynamic task scheduling.  It is the executor for CPU inference (fp32 activations with
// fp32 / bf16 / fp16 / int8 / int4-group weights) and the oracle the GPU kernels are tested against.
//
// Reference components this file stands in for:
//   op registry of the cpu device              src/devices/cpu/cpudevice.cpp:284-394
//   multi-threaded Linear variants             src/devices/cpu/linear.cpp:412-1278
//   spin pool + work stealing                  include/devices/cpu/alivethreadpool.h, include/devices/cpu/computeutils.h:175-201
//   SelectExpert                               src/devices/cpu/cpudevice.cpp:8885-8955
//
// Layout conventions: activations fp32 row-major; weights [out, in] row-major; int8 = per-row (scale, zero) with
// w = scale * (q - zero); int4-group = two values per byte, first value in the HIGH nibble, w = min + scale * q with
// (scale, min) per (row, group).  Paged KV pools are [num_slots, kv_heads, head_dim] fp32, slot = page * page_len + offset.
#include <immintrin.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>

namespace {

// ---------------------------------------------------------------------------------------------------------------
// thread pool: workers poll briefly, then sleep on a condition variable, between parallel regions; inside a region
// tasks are claimed from one atomic counter, so a slow core simply takes fewer tasks
// ---------------------------------------------------------------------------------------------------------------
class Pool {
 public:
  explicit Pool(int n) { resize(n); }
  ~Pool() { stop(); }

  void resize(int n) {
    stop();
    n_threads_ = n < 1 ? 1 : n;
    quit_.store(false);
    for (int i = 1; i < n_threads_; ++i) workers_.emplace_back([this] { loop(); });
  }
  int size() const { return n_threads_; }

  void run(int n_tasks, const std::function<void(int)>& fn) {
    if (n_tasks <= 0) return;
    if (n_threads_ == 1 || n_tasks == 1) {
      for (int i = 0; i < n_tasks; ++i) fn(i);
      return;
    }
    fn_ = &fn;
    n_tasks_ = n_tasks;
    next_.store(0, std::memory_order_relaxed);
    pending_.store(n_threads_ - 1, std::memory_order_relaxed);
    epoch_.fetch_add(1);                         // publishes fn_ / n_tasks_ / next_ (sequentially consistent)
    if (sleepers_.load() > 0) {
      { std::lock_guard<std::mutex> lk(mu_); }   // a worker between its predicate check and its wait holds the mutex
      cv_.notify_all();
    }
    work();
    while (pending_.load(std::memory_order_acquire) != 0) _mm_pause();
    fn_ = nullptr;
  }

 private:
  // Between two operators of a decode step the host spends a few tens of microseconds: workers keep polling for about
  // that long before they block, so consecutive operators start without a futex wake-up.
  static constexpr int SPIN_ITERS = 20000;

  void work() {
    for (;;) {
      const int i = next_.fetch_add(1, std::memory_order_relaxed);
      if (i >= n_tasks_) break;
      (*fn_)(i);
    }
  }
  void loop() {
    uint64_t seen = 0;
    for (;;) {
      bool ready = false;
      for (int i = 0; i < SPIN_ITERS; ++i) {
        if (quit_.load(std::memory_order_relaxed) || epoch_.load(std::memory_order_acquire) != seen) { ready = true; break; }
        _mm_pause();
      }
      if (!ready) {
        std::unique_lock<std::mutex> lk(mu_);
        sleepers_.fetch_add(1);
        cv_.wait(lk, [&] { return quit_.load() || epoch_.load() != seen; });
        sleepers_.fetch_sub(1);
      }
      if (quit_.load()) return;
      seen = epoch_.load(std::memory_order_acquire);
      work();
      pending_.fetch_sub(1, std::memory_order_release);
    }
  }
  void stop() {
    quit_.store(true);
    { std::lock_guard<std::mutex> lk(mu_); }
    cv_.notify_all();
    for (auto& t : workers_) t.join();
    workers_.clear();
  }

  int n_threads_ = 1;
  std::vector<std::thread> workers_;
  std::mutex mu_;
  std::condition_variable cv_;
  const std::function<void(int)>* fn_ = nullptr;
  int n_tasks_ = 0;
  std::atomic<int> next_{0}, pending_{0}, sleepers_{0};
  std::atomic<uint64_t> epoch_{0};
  std::atomic<bool> quit_{false};
};

Pool& pool() {
  static Pool p([] {
    unsigned hc = std::thread::hardware_concurrency();
    int n = hc == 0 ? 4 : (int)hc;
    return n > 32 ? 32 : n;
  }());
  return p;
}

inline bool has_avx512() {
  static const bool v = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl");
  return v;
}

enum WType { W_F32 = 0, W_BF16 = 1, W_F16 = 2, W_INT8 = 3, W_INT4G = 4 };

}  // namespace

#include "cpu_kernels.h"

namespace {

// chunk n items into tasks of at least `min_chunk`, about 4 tasks per thread for balance
inline void split_run(int n, int min_chunk, const std::function<void(int, int)>& fn) {
  if (n <= 0) return;
  const int nt = pool().size();
  int chunk = (n + nt * 4 - 1) / (nt * 4);
  if (chunk < min_chunk) chunk = min_chunk;
  const int tasks = (n + chunk - 1) / chunk;
  pool().run(tasks, [&](int t) {
    const int a = t * chunk, b = a + chunk < n ? a + chunk : n;
    fn(a, b);
  });
}

// rows of `width` floats per task so that a task touches at least ~32K elements (smaller regions run inline)
inline int rows_per_task(int width) { const int r = 32768 / (width > 0 ? width : 1); return r < 1 ? 1 : r; }

#define FB_DISPATCH(fn, ...)                    \
  do {                                          \
    if (has_avx512()) fn##_avx512(__VA_ARGS__); \
    else fn##_avx2(__VA_ARGS__);                \
  } while (0)

}  // namespace

extern "C" {

// reduced-precision-activation kernels of cpu_accel.cpp (VNNI / AVX-512 BF16 / AMX): off unless switched on
int fbx_caps();
void fbx_quant_act_s8(const float* x, int ldx, int M, int K, int deint, int8_t* xq, float* scale, float* sum);
void fbx_to_bf16(const float* x, int ldx, int M, int K, uint16_t* xb);
void fbx_linear_rows_bf16(const FbLinearArgs* a, const uint16_t* xb, int n0, int n1);
void fbx_linear_rows_i8(const FbLinearArgs* a, const int8_t* xq, const float* xscale, const float* xsum, int n0, int n1);
void fbx_amx_pack_i8(const int8_t* xq, int M, int K, int8_t* pk);
void fbx_amx_pack_bf16(const uint16_t* xb, int M, int K, uint16_t* pk);
void fbx_amx_linear_rows_bf16(const FbLinearArgs* a, const uint16_t* pk, int n0, int n1);
void fbx_amx_linear_rows_i8(const FbLinearArgs* a, const int8_t* pk, const float* xscale, const float* xsum, int n0, int n1);

static int g_accel = 0;          // bits requested by fbcpu_set_accel, masked by what the CPU has
// flags: bit 0 VNNI (int8 / int4-group weights with int8 activations), bit 1 AVX-512 BF16, bit 2 AMX.  Returns the bits in effect.
int fbcpu_set_accel(int flags) { g_accel = flags & fbx_caps(); return g_accel; }
int fbcpu_get_accel() { return g_accel; }
int fbcpu_accel_caps() { return fbx_caps(); }

int fbcpu_get_threads() { return pool().size(); }
void fbcpu_set_threads(int n) { pool().resize(n); }
int fbcpu_isa() { return has_avx512() ? 512 : 256; }

// y[M,N] = x[M,K] * W[N,K]^T (+ bias).  Returns 0, or -1 for an unsupported shape.
int fbcpu_linear(const float* x, int ldx, const void* w, int wtype, const float* scale, const float* zero, int group,
                 const float* bias, float* y, int ldy, int M, int N, int K) {
  if (M <= 0 || N <= 0) return 0;
  if (wtype < 0 || wtype > 4) return -1;
  if (wtype == W_INT4G && (group <= 0 || K % group != 0 || group % 16 != 0)) return -1;
  FbLinearArgs a;
  a.x = x; a.ldx = ldx; a.w = w; a.wtype = wtype; a.scale = scale; a.zero = zero; a.group = group; a.bias = bias;
  a.y = y; a.ldy = ldy; a.M = M; a.N = N; a.K = K; a.xsum = nullptr;
  if (g_accel != 0) {
    const bool amx = (g_accel & 4) && M >= 16;
    if (wtype == W_BF16 && (g_accel & 6) && K % 32 == 0) {
      // bf16 weights x bf16 activations: dot-product instructions (two bf16 pairs per lane), or AMX tiles for 16+ rows
      std::vector<uint16_t> xb((size_t)M * K);
      fbx_to_bf16(x, ldx, M, K, xb.data());
      if (amx) {
        std::vector<uint16_t> pk((size_t)((M + 15) / 16 * 16) * K);
        fbx_amx_pack_bf16(xb.data(), M, K, pk.data());
        const int tiles = (N + 15) / 16;
        pool().run(tiles, [&](int t) { fbx_amx_linear_rows_bf16(&a, pk.data(), t * 16, std::min(N, t * 16 + 16)); });
        return 0;
      }
      if (g_accel & 2) {
        split_run(N, 8, [&](int n0, int n1) { fbx_linear_rows_bf16(&a, xb.data(), n0, n1); });
        return 0;
      }
    }
    if ((wtype == W_INT8 || (wtype == W_INT4G && group == 128)) && (g_accel & 1) && K % 128 == 0) {
      const int nb = K / 128;
      std::vector<int8_t> xq((size_t)M * K);
      std::vector<float> xsc((size_t)M * nb), xsm((size_t)M * nb);
      const bool use_amx = amx && wtype == W_INT8;
      fbx_quant_act_s8(x, ldx, M, K, wtype == W_INT4G ? 1 : 0, xq.data(), xsc.data(), xsm.data());
      if (use_amx) {
        std::vector<int8_t> pk((size_t)((M + 15) / 16 * 16) * K);
        fbx_amx_pack_i8(xq.data(), M, K, pk.data());
        const int tiles = (N + 15) / 16;
        pool().run(tiles, [&](int t) { fbx_amx_linear_rows_i8(&a, pk.data(), xsc.data(), xsm.data(), t * 16, std::min(N, t * 16 + 16)); });
        return 0;
      }
      split_run(N, 8, [&](int n0, int n1) { fbx_linear_rows_i8(&a, xq.data(), xsc.data(), xsm.data(), n0, n1); });
      return 0;
    }
  }
  std::vector<float> xsum;
  if (wtype == W_INT8 || wtype == W_INT4G) {
    const int g = wtype == W_INT8 ? K : group;
    xsum.resize((size_t)M * (K / g));
    FB_DISPATCH(fbk_group_sums, x, ldx, M, K, g, xsum.data());
    a.xsum = xsum.data();
  }
  split_run(N, 8, [&](int n0, int n1) { FB_DISPATCH(fbk_linear_rows, &a, n0, n1); });
  return 0;
}

void fbcpu_rmsnorm(const float* x, int ldx, const float* w, float* y, int ldy, int M, int H, float eps, float unit_offset) {
  split_run(M, rows_per_task(H), [&](int r0, int r1) { FB_DISPATCH(fbk_rmsnorm_rows, x, ldx, w, y, ldy, H, eps, unit_offset, r0, r1); });
}

void fbcpu_layernorm(const float* x, int ldx, const float* w, const float* b, float* y, int ldy, int M, int H, float eps) {
  split_run(M, rows_per_task(H), [&](int r0, int r1) { FB_DISPATCH(fbk_layernorm_rows, x, ldx, w, b, y, ldy, H, eps, r0, r1); });
}

void fbcpu_swiglu(const float* gu, int ld, float* out, int ldo, int M, int inter) {
  split_run(M, rows_per_task(inter), [&](int r0, int r1) { FB_DISPATCH(fbk_swiglu_rows, gu, ld, out, ldo, inter, r0, r1); });
}

void fbcpu_activation(float* x, long long n, int kind) {
  const int blocks = (int)((n + 4095) / 4096);
  split_run(blocks, 1, [&](int b0, int b1) {
    const long long a = (long long)b0 * 4096, e = std::min<long long>(n, (long long)b1 * 4096);
    FB_DISPATCH(fbk_act_rows, x + a, (int)(e - a), kind);
  });
}

void fbcpu_softmax(float* x, int ld, int rows, int cols) {
  split_run(rows, rows_per_task(cols), [&](int r0, int r1) { FB_DISPATCH(fbk_softmax_rows, x, ld, cols, r0, r1); });
}

void fbcpu_rope(float* x, int ld, const int* pos, const float* cos_t, const float* sin_t, int rows, int heads, int D, int rot, int mode) {
  if (mode == 0 || rot <= 0) return;
  split_run(rows, rows_per_task(heads * D), [&](int r0, int r1) { FB_DISPATCH(fbk_rope_rows, x, ld, pos, cos_t, sin_t, heads, D, rot, mode, r0, r1); });
}

// append new K / V rows ([T, Hkv*D] with row strides ldk / ldv) into the paged pools at `slots`
void fbcpu_kv_append(const float* k, int ldk, const float* v, int ldv, const int* slots, float* k_pool, float* v_pool, int T, int row_elems) {
  split_run(T, 4, [&](int t0, int t1) {
    for (int t = t0; t < t1; ++t) {
      if (slots[t] < 0) continue;
      std::memcpy(k_pool + (size_t)slots[t] * row_elems, k + (size_t)t * ldk, (size_t)row_elems * 4);
      std::memcpy(v_pool + (size_t)slots[t] * row_elems, v + (size_t)t * ldv, (size_t)row_elems * 4);
    }
  });
}

int fbcpu_attention_paged(const float* q, int ldq, const float* k_pool, const float* v_pool, const int* page_table, int max_pages,
                          const int* kv_lens, const int* cu_q, float* out, int ldo, int B, int Hq, int Hkv, int D, int page_len,
                          float scale, int window, const float* sinks) {
  if (D > 512 || Hkv <= 0 || Hq % Hkv != 0) return -1;
  FbAttnArgs a;
  a.q = q; a.ldq = ldq; a.k_pool = k_pool; a.v_pool = v_pool; a.page_table = page_table; a.max_pages = max_pages;
  a.kv_lens = kv_lens; a.cu_q = cu_q; a.out = out; a.ldo = ldo; a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.page_len = page_len;
  a.scale = scale; a.window = window; a.sinks = sinks;
  split_run(B * Hq, 1, [&](int i0, int i1) { FB_DISPATCH(fbk_attention_items, &a, i0, i1); });
  return 0;
}

void fbcpu_embedding(const float* table, const int* ids, float* out, int T, int H, float scale) {
  split_run(T, 4, [&](int t0, int t1) {
    for (int t = t0; t < t1; ++t) {
      const float* src = table + (size_t)ids[t] * H;
      float* dst = out + (size_t)t * H;
      if (scale == 1.0f) std::memcpy(dst, src, (size_t)H * 4);
      else for (int i = 0; i < H; ++i) dst[i] = src[i] * scale;
    }
  });
}

// Expert selection (reference semantics: top-k on logits + bias, scores taken from the un-biased values, optional renorm,
// times route_scale).  mode 0: scores = softmax(logits), 1: sigmoid(logits), 2: logits as given.
void fbcpu_select_expert(const float* logits, const float* bias, int T, int E, int topk, int mode, int renorm, float route_scale,
                         int* out_idx, float* out_w) {
  split_run(T, 1, [&](int t0, int t1) {
    std::vector<float> sc(E), sel(E);
    for (int t = t0; t < t1; ++t) {
      const float* lg = logits + (size_t)t * E;
      if (mode == 0) {
        float mx = -INFINITY, s = 0.f;
        for (int e = 0; e < E; ++e) mx = std::max(mx, lg[e]);
        for (int e = 0; e < E; ++e) { sc[e] = std::exp(lg[e] - mx); s += sc[e]; }
        for (int e = 0; e < E; ++e) sc[e] /= s;
      } else if (mode == 1) {
        for (int e = 0; e < E; ++e) sc[e] = 1.0f / (1.0f + std::exp(-lg[e]));
      } else {
        for (int e = 0; e < E; ++e) sc[e] = lg[e];
      }
      for (int e = 0; e < E; ++e) sel[e] = sc[e] + (bias ? bias[e] : 0.f);
      float tot = 0.f;
      for (int k = 0; k < topk; ++k) {
        int best = 0;
        for (int e = 1; e < E; ++e)
          if (sel[e] > sel[best]) best = e;          // strict: ties keep the lower expert id
        out_idx[(size_t)t * topk + k] = best;
        out_w[(size_t)t * topk + k] = sc[best];
        tot += sc[best];
        sel[best] = -INFINITY;
      }
      for (int k = 0; k < topk; ++k) {
        float w = out_w[(size_t)t * topk + k];
        if (renorm) w /= (tot + 1e-20f);
        out_w[(size_t)t * topk + k] = w * route_scale;
      }
    }
  });
}

}  // extern "C"
