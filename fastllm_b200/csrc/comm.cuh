// Shared pieces of the tensor-parallel communication kernels: the arena header layout, the per-rank context
// (local / multicast / peer pointers) and the cross-rank arrival / wait helpers.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "ptx.cuh"

namespace fb {

constexpr int MAX_TP = 8;

// arena header layout (bytes from the arena base); each word on its own 128-byte line
constexpr uint32_t OFF_CNT1 = 0, OFF_CNT2 = 128, OFF_EXPECT = 256, OFF_TICKET = 384, OFF_LOCAL1 = 512, OFF_LOCAL2 = 640, OFF_TRACE = 768;   // OFF_TRACE: 8 x u64 phase time stamps of CTA 0

struct CommCtx {
  uint8_t* local;            // this rank's arena
  uint8_t* mc;               // multicast mapping of the arena (nullptr: use peer pointers)
  uint8_t* peer[MAX_TP];     // every rank's arena as seen from this GPU (peer[rank] == local)
  int rank, tp;
};

__device__ __forceinline__ void red_add_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void mc_red_add_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("multimem.red.relaxed.sys.global.add.u32 [%0], %1;\n" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 mc_ld_reduce_f32x4(const void* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];\n"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_b32x4(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};\n"
               ::"l"(p), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// one arrival on counter `off` of every rank
// (one system-scope fence, then relaxed reductions: the fence is the expensive part, do it once)
__device__ __forceinline__ void signal_all(const CommCtx& c, uint32_t off) {
  __threadfence_system();
  if (c.mc) {
    mc_red_add_relaxed_sys(reinterpret_cast<uint32_t*>(c.mc + off), 1u);
  } else {
    for (int r = 0; r < c.tp; ++r) red_add_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[r] + off), 1u);
  }
}
// CTA-level arrival: CTAs of this rank first meet on a local counter; the last one sends ONE arrival to every rank,
// so the cross-GPU counter sees tp arrivals per launch instead of tp x CTAs atomics on one address.
// Ordering: every CTA fences at GPU scope before its local arrival; the last arriver's system-scope fence is
// cumulative over everything it observed through the local counter.
__device__ __forceinline__ void arrive_aggregated(const CommCtx& c, uint32_t off_local, uint32_t off_remote, int n_ctas) {
  __threadfence();
  uint32_t* lc = reinterpret_cast<uint32_t*>(c.local + off_local);
  if (atomicAdd(lc, 1u) == (uint32_t)(n_ctas - 1)) {
    *lc = 0u;                       // nobody reads it again in this launch
    signal_all(c, off_remote);
  }
}
// bounded wait until the local counter has reached `target` (wrap-safe)
__device__ __forceinline__ bool wait_counter(const CommCtx& c, uint32_t off, uint32_t target, int kernel_id, int site) {
  return wait_counter_ge(reinterpret_cast<const uint32_t*>(c.local + off), target, kernel_id, site);
}

inline int sm_count() {
  static int g_sm_count = 0;
  if (g_sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  return g_sm_count;
}

inline void fill_ctx(CommCtx& c, void* local, void* mc, void* const* peers, int rank, int tp) {
  c.local = (uint8_t*)local; c.mc = (uint8_t*)mc; c.rank = rank; c.tp = tp;
  for (int i = 0; i < MAX_TP; ++i) c.peer[i] = i < tp ? (uint8_t*)peers[i] : nullptr;
}


}  // namespace fb
