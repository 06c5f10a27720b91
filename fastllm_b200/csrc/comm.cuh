// Shared pieces of the tensor-parallel communication kernels: the arena header layout, the per-rank context
// (local / multicast / peer pointers) and the cross-rank arrival / wait helpers.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "ptx.cuh"
#include "gemm_smallm.cuh"

namespace fb {

constexpr int KID_GEMM_AR = 30;
constexpr int KID_AR_NORM = 31;
constexpr int KID_ARGMAX_MERGE = 32;
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


struct ArNormParams {
  CommCtx c;
  uint64_t off_part;         // fp32 [tp, M, N]: slot s holds rank s's partial rows (only this rank's own rows are used)
  uint64_t off_h;            // 16-bit [M, N] residual stream (read: own rows; written: all ranks)
  uint64_t off_x;            // 16-bit [M, N] normalised output
  const uint16_t* ln_w;      // RMSNorm weight [N] (nullptr: skip the norm, x is not written)
  const void* src;           // stand-alone kernel: this rank's partial [M, N] to push (nullptr in the GEMM kernel)
  int src_f32;               // src is fp32 (else the 16-bit activation dtype)
  // MoE combine source (src == nullptr, moe_ys != nullptr): partial[row] = sum_k moe_w[row,k] * moe_ys[moe_pos[row,k]] (+ moe_add[row])
  const uint16_t* moe_ys; const int* moe_pos; const float* moe_w; const uint16_t* moe_add; int moe_topk;
  int M, N;
  int has_residual;
  int defer_sync2;           // != 0: end after the broadcast + arrival; the consumer kernel waits on CNT2 >= EXPECT itself
  int trace;                 // != 0: CTA 0 writes globaltimer stamps of each phase to OFF_TRACE
  float eps, unit_offset;
};

// Phases 2.. of the fused all-reduce; called by every thread of every CTA.  `base` = value of the expect word
// read at kernel start; n_ctas = CTAs per rank in this launch.  CTAs come in groups of `csize` (one thread-block
// cluster): a group owns whole rows, each of its CTAs one column slice; the row's sum of squares is exchanged
// through distributed shared memory.
template <bool BF16>
__device__ __forceinline__ void ar_norm_tail(const ArNormParams& p, uint32_t base, int group, int n_groups, int crank,
                                             int csize, int kernel_id) {
  __shared__ float sh_red[16];
  __shared__ float sh_ss;
  __shared__ int sh_ok;
  const CommCtx& c = p.c;
  const int n_ctas = n_groups * csize;
  const uint32_t target = base + (uint32_t)c.tp;      // one aggregated arrival per rank per counter
  const int tid = threadIdx.x, nthr = blockDim.x;
  uint64_t* trace = (p.trace && group == 0 && crank == 0 && tid == 0) ? reinterpret_cast<uint64_t*>(c.local + OFF_TRACE) : nullptr;
  // ---- sync 1: all partials of all ranks are in their arenas ----
  __syncthreads();
  if (tid == 0) {
    if (trace) trace[1] = globaltimer_ns();
    arrive_aggregated(c, OFF_LOCAL1, OFF_CNT1, n_ctas);
    if (trace) trace[2] = globaltimer_ns();
    sh_ok = wait_counter(c, OFF_CNT1, target, kernel_id, 1) ? 1 : 0;
    if (trace) trace[3] = globaltimer_ns();
  }
  __syncthreads();
  const bool ok = sh_ok != 0;      // a CTA that timed out still walks the loop (cluster barriers must match) but moves no data
  // ---- phase 2: own rows ----
  const int rows_per = (p.M + c.tp - 1) / c.tp;
  const int row0 = c.rank * rows_per;
  int row1 = row0 + rows_per; if (row1 > p.M) row1 = p.M;
  const int N = p.N;
  const int chunks = N >> 3;                         // 8 columns per chunk
  const int cpc = (chunks + csize - 1) / csize;      // chunks per CTA of the group
  const int ch0 = crank * cpc;
  int ch1 = ch0 + cpc; if (ch1 > chunks) ch1 = chunks;
  constexpr int MAXC = 12;
  for (int row = row0 + group; row < row1; row += n_groups) {
    uint4 hv[MAXC];
    float ss = 0.f;
    int cnt = 0;
    for (int ch = ch0 + tid; ok && ch < ch1; ch += nthr, ++cnt) {
      const size_t eoff = (size_t)row * N + (size_t)ch * 8;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
      for (int r = 0; r < c.tp; ++r) {
        const float4* src = reinterpret_cast<const float4*>(c.local + p.off_part + (((size_t)r * p.M + row) * N + (size_t)ch * 8) * 4);
        const float4 u = src[0], w = src[1];
        a.x += u.x; a.y += u.y; a.z += u.z; a.w += u.w;
        b.x += w.x; b.y += w.y; b.z += w.z; b.w += w.w;
      }
      if (p.has_residual) {
        const uint4 rv = *reinterpret_cast<const uint4*>(c.local + p.off_h + eoff * 2);
        const float2 r0 = unpack_16<BF16>(rv.x), r1 = unpack_16<BF16>(rv.y), r2 = unpack_16<BF16>(rv.z), r3 = unpack_16<BF16>(rv.w);
        a.x += r0.x; a.y += r0.y; a.z += r1.x; a.w += r1.y;
        b.x += r2.x; b.y += r2.y; b.z += r3.x; b.w += r3.y;
      }
      uint4 o;
      o.x = pack_16<BF16>(a.x, a.y); o.y = pack_16<BF16>(a.z, a.w); o.z = pack_16<BF16>(b.x, b.y); o.w = pack_16<BF16>(b.z, b.w);
      if (cnt < MAXC) hv[cnt] = o;
      // the norm sees the rounded values, exactly what a separate RMSNorm kernel would read back
      const float2 q0 = unpack_16<BF16>(o.x), q1 = unpack_16<BF16>(o.y), q2 = unpack_16<BF16>(o.z), q3 = unpack_16<BF16>(o.w);
      ss += q0.x * q0.x + q0.y * q0.y + q1.x * q1.x + q1.y * q1.y + q2.x * q2.x + q2.y * q2.y + q3.x * q3.x + q3.y * q3.y;
      // The residual stream stays with the row's owner: nobody else reads it (the next collective's phase 2 reads own
      // rows only), so it does not cross NVLink.
      *reinterpret_cast<uint4*>(c.local + p.off_h + eoff * 2) = o;
      if (p.ln_w == nullptr) {
        // no norm: the summed rows themselves are the result every rank needs
        if (c.mc) {
          mc_st_b32x4(c.mc + p.off_x + eoff * 2, o);
        } else {
          for (int r = 0; r < c.tp; ++r) *reinterpret_cast<uint4*>(c.peer[r] + p.off_x + eoff * 2) = o;
        }
      }
    }
    if (p.ln_w != nullptr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      __syncthreads();
      if ((tid & 31) == 0) sh_red[tid >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
      for (int w = 0; w < (nthr >> 5); ++w) tot += sh_red[w];
      if (csize > 1) {
        if (tid == 0) sh_ss = tot;
        cluster_sync_all();
        const uint32_t a_ss = smem_u32(&sh_ss);
        tot = 0.f;
        for (int r = 0; r < csize; ++r) tot += ld_dsmem_f32(mapa_u32(a_ss, (uint32_t)r));
        cluster_sync_all();          // peers have read sh_ss before the next row overwrites it
      }
      const float inv = rsqrtf(tot / (float)N + p.eps);
      cnt = 0;
      for (int ch = ch0 + tid; ok && ch < ch1; ch += nthr, ++cnt) {
        const size_t eoff = (size_t)row * N + (size_t)ch * 8;
        const uint4 h = hv[cnt < MAXC ? cnt : MAXC - 1];
        const uint4 wv = *reinterpret_cast<const uint4*>(p.ln_w + (size_t)ch * 8);
        const float2 h0 = unpack_16<BF16>(h.x), h1 = unpack_16<BF16>(h.y), h2 = unpack_16<BF16>(h.z), h3 = unpack_16<BF16>(h.w);
        const float2 w0 = unpack_16<BF16>(wv.x), w1 = unpack_16<BF16>(wv.y), w2 = unpack_16<BF16>(wv.z), w3 = unpack_16<BF16>(wv.w);
        const float uo = p.unit_offset;
        uint4 o;
        o.x = pack_16<BF16>(h0.x * inv * (w0.x + uo), h0.y * inv * (w0.y + uo));
        o.y = pack_16<BF16>(h1.x * inv * (w1.x + uo), h1.y * inv * (w1.y + uo));
        o.z = pack_16<BF16>(h2.x * inv * (w2.x + uo), h2.y * inv * (w2.y + uo));
        o.w = pack_16<BF16>(h3.x * inv * (w3.x + uo), h3.y * inv * (w3.y + uo));
        if (c.mc) {
          mc_st_b32x4(c.mc + p.off_x + eoff * 2, o);
        } else {
          for (int r = 0; r < c.tp; ++r) *reinterpret_cast<uint4*>(c.peer[r] + p.off_x + eoff * 2) = o;
        }
      }
    }
  }
  // ---- sync 2: every rank's rows have been written everywhere ----
  __syncthreads();
  if (tid == 0) {
    if (trace) trace[4] = globaltimer_ns();
    arrive_aggregated(c, OFF_LOCAL2, OFF_CNT2, n_ctas);
    if (trace) trace[5] = globaltimer_ns();
    if (!p.defer_sync2) wait_counter(c, OFF_CNT2, target, kernel_id, 2);
    if (trace) trace[6] = globaltimer_ns();
    // the last CTA of this rank to get here publishes the new expected value for the next launch
    uint32_t* ticket = reinterpret_cast<uint32_t*>(c.local + OFF_TICKET);
    if (atomicAdd(ticket, 1u) == (uint32_t)(n_ctas - 1)) {
      *ticket = 0u;
      *reinterpret_cast<volatile uint32_t*>(c.local + OFF_EXPECT) = target;
      __threadfence();
    }
  }
}


// ---- host side: the collective's parameters and the GEMM's scatter target, shared by every fused GEMM entry point ----
inline void fill_ar_norm(ArNormParams& p, void* arena_local, void* arena_mc, void* const* peers, int rank, int tp,
                         unsigned long long off_part, unsigned long long off_h, unsigned long long off_x, const void* ln_w, int M, int N,
                         int flags, float eps, float unit_offset) {
  fill_ctx(p.c, arena_local, arena_mc, peers, rank, tp);
  p.off_part = off_part; p.off_h = off_h; p.off_x = off_x; p.ln_w = (const uint16_t*)ln_w; p.M = M; p.N = N;
  p.has_residual = flags & 1; p.trace = (flags >> 1) & 1; p.defer_sync2 = (flags >> 2) & 1; p.eps = eps; p.unit_offset = unit_offset;
  p.src = nullptr; p.src_f32 = 0; p.moe_ys = nullptr; p.moe_pos = nullptr; p.moe_w = nullptr; p.moe_add = nullptr; p.moe_topk = 0;
}
// the GEMM epilogue pushes fp32 row j of this rank's partial to the arena of the rank that owns row j (slot = this rank)
inline void fill_scatter(GemmParams& g, void* arena_local, void* const* peers, unsigned long long off_part, int M, int N, int rank, int tp) {
  g.out = (uint8_t*)arena_local + off_part; g.residual = nullptr; g.ld_out = N; g.ld_res = 0;
  g.scatter_tp = tp; g.scatter_rows = (M + tp - 1) / tp; g.scatter_rank = rank; g.w_row0 = 0; g.x_row0 = 0;
  for (int i = 0; i < 8; ++i) g.scatter_out[i] = i < tp ? reinterpret_cast<float*>((uint8_t*)peers[i] + off_part) : nullptr;
}

}  // namespace fb
