// Token sampling for sm_100a: repeat penalty, temperature, top-k, top-p and the random draw in ONE launch, one CTA per
// request row, without sorting the vocabulary.
//
// Per row:  (1) penalty on the recently generated ids, in place;  (2) exact k-th largest logit by a 4-pass 8-bit radix
// select over order-preserving integer keys (the row stays L2-resident across the passes);  (3) the <= 1024 survivors are
// gathered into shared memory and bitonic-sorted;  (4) softmax, inclusive scan, nucleus cut, inverse-CDF draw with the
// caller's uniform variate.  top_k <= 0 or > 1024 samples from the 1024 most likely tokens.
//
// Reference behaviour: LLMSampling (src/fastllm.cpp:3037-3138: penalty -> temperature -> top-k -> softmax -> top-p -> draw),
// GPU path FastllmTemperatureSoftmaxKernel / FlashInfer TopKTopPSamplingFromProb (src/devices/cuda/fastllm-cuda.cu:13229-13529).
#include "ptx.cuh"
#include "launch.h"

FB_DEFINE_ERROR_API(sampling)

namespace fb {

constexpr int SM_THREADS = 1024;
constexpr int SM_CAND = 1024;

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

struct SampleParams {
  float* logits; int ld; int V;
  const float* temperature; const int* top_k; const float* top_p; const float* uniform; const float* penalty;
  const int* recent; int recent_w;       // [R, recent_w] de-duplicated ids, -1 padded
  int* out_ids; float* out_prob;         // chosen token and its probability under the truncated distribution
};

__global__ void __launch_bounds__(SM_THREADS, 1) sample_kernel(const SampleParams p) {
  __shared__ uint32_t hist[256];
  __shared__ unsigned long long cand[SM_CAND];
  __shared__ float scan[SM_CAND];
  __shared__ float warp_tot[32];
  __shared__ uint32_t sh_prefix, sh_remaining, sh_count, sh_take_eq;
  __shared__ int sh_n_keep, sh_choice;
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x, tid = threadIdx.x;
  float* lg = p.logits + (size_t)row * p.ld;
  const int V = p.V;

  // ---- (1) repeat penalty, in place ----
  const float pen = p.penalty ? p.penalty[row] : 1.0f;
  if (p.recent != nullptr && fabsf(pen - 1.0f) > 1e-8f) {
    for (int i = tid; i < p.recent_w; i += SM_THREADS) {
      const int id = p.recent[(size_t)row * p.recent_w + i];
      if (id >= 0 && id < V) { const float v = lg[id]; lg[id] = v > 0.f ? v / pen : v * pen; }
    }
    __syncthreads();
  }
  const float inv_t = 1.0f / fmaxf(p.temperature ? p.temperature[row] : 1.0f, 1e-6f);
  int k = p.top_k ? p.top_k[row] : 0;
  if (k <= 0 || k > SM_CAND) k = SM_CAND;
  if (k > V) k = V;

  // ---- (2) radix select: key of the k-th largest scaled logit ----
  if (tid == 0) { sh_prefix = 0; sh_remaining = (uint32_t)k; }
  uint32_t mask = 0;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = sh_prefix;
    for (int i = tid; i < V; i += SM_THREADS) {
      const uint32_t key = order_key(lg[i] * inv_t);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t rem = sh_remaining, acc = 0;
      int b = 255;
      for (; b > 0; --b) {
        if (acc + hist[b] >= rem) break;
        acc += hist[b];
      }
      sh_remaining = rem - acc;                 // how many of bin b (and, after the last pass, of the exact key) to take
      sh_prefix = prefix | ((uint32_t)b << shift);
    }
    mask |= 255u << shift;
    __syncthreads();
  }
  const uint32_t thr = sh_prefix;               // exact key of the k-th largest element
  if (tid == 0) { sh_count = 0; sh_take_eq = sh_remaining; }
  __syncthreads();

  // ---- (3) gather survivors: everything above the threshold, plus as many equal keys as the count needs ----
  for (int i = tid; i < V; i += SM_THREADS) {
    const uint32_t key = order_key(lg[i] * inv_t);
    bool take = key > thr;
    if (!take && key == thr) {
      const uint32_t old = atomicSub(&sh_take_eq, 1u);
      take = old >= 1u && old <= (uint32_t)SM_CAND;       // wrapped below zero: no quota left
    }
    if (take) {
      const uint32_t slot = atomicAdd(&sh_count, 1u);
      if (slot < (uint32_t)SM_CAND) cand[slot] = ((unsigned long long)key << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
    }
  }
  __syncthreads();
  int n = (int)min(sh_count, (uint32_t)SM_CAND);
  for (int i = n + tid; i < SM_CAND; i += SM_THREADS) cand[i] = 0ull;
  __syncthreads();
  // bitonic sort, descending (key, then lower token id first)
  for (int size = 2; size <= SM_CAND; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      const int i = tid, j = i ^ stride;
      if (j > i) {
        const bool desc = (i & size) == 0;
        const unsigned long long a = cand[i], b = cand[j];
        if ((a < b) == desc) { cand[i] = b; cand[j] = a; }
      }
      __syncthreads();
    }
  }

  // ---- (4) softmax over the survivors, inclusive scan, nucleus cut, draw ----
  const float vmax = key_value((uint32_t)(cand[0] >> 32));
  float pr = 0.f;
  if (tid < n) pr = __expf(key_value((uint32_t)(cand[tid] >> 32)) - vmax);
  float incl = pr;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if ((tid & 31) >= o) incl += t;
  }
  if ((tid & 31) == 31) warp_tot[tid >> 5] = incl;
  __syncthreads();
  if (tid < 32) {
    float w = warp_tot[tid];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, w, o);
      if (tid >= o) w += t;
    }
    warp_tot[tid] = w;
  }
  __syncthreads();
  if ((tid >> 5) > 0) incl += warp_tot[(tid >> 5) - 1];
  scan[tid] = incl;
  if (tid == 0) { sh_n_keep = 0; sh_choice = 0; }
  __syncthreads();
  const float total = scan[SM_CAND - 1];
  const float tp = p.top_p ? p.top_p[row] : 1.0f;
  // token i stays while the probability mass before it is below top_p (the most likely token always stays)
  if (tid < n && (tid == 0 || (incl - pr) < tp * total)) atomicAdd(&sh_n_keep, 1);
  __syncthreads();
  const int keep = max(1, sh_n_keep);
  const float kept_total = scan[keep - 1];
  const float target = (p.uniform ? p.uniform[row] : 0.5f) * kept_total;
  if (tid < keep && incl <= target) atomicAdd(&sh_choice, 1);
  __syncthreads();
  if (tid == 0) {
    int c = sh_choice;
    if (c >= keep) c = keep - 1;
    const unsigned long long e = cand[c];
    p.out_ids[row] = (int)(0xFFFFFFFFu - (uint32_t)(e & 0xFFFFFFFFull));
    if (p.out_prob) p.out_prob[row] = (scan[c] - (c > 0 ? scan[c - 1] : 0.f)) / kept_total;
  }
}

}  // namespace fb

using namespace fb;

// logits: fp32 [R, ld] (modified in place by the penalty).  Per-row arrays may be null (defaults: temperature 1,
// top_k 1024, top_p 1, uniform 0.5, no penalty).
extern "C" int fb_sample(float* logits, int ld, int R, int V, const float* temperature, const int* top_k, const float* top_p,
                         const float* uniform, const float* penalty, const int* recent, int recent_w, int* out_ids, float* out_prob,
                         void* stream) {
  if (R <= 0) return 0;
  if (V <= 0 || ld < V) return -1;
  SampleParams p;
  p.logits = logits; p.ld = ld; p.V = V; p.temperature = temperature; p.top_k = top_k; p.top_p = top_p; p.uniform = uniform;
  p.penalty = penalty; p.recent = recent; p.recent_w = recent_w; p.out_ids = out_ids; p.out_prob = out_prob;
  return (int)launch_k(sample_kernel, dim3(R), dim3(SM_THREADS), 0, reinterpret_cast<cudaStream_t>(stream), 0, p);
}
