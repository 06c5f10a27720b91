// Bandwidth-regime tensor-parallel collectives for prefill-sized batches (hundreds to thousands of token rows), sm_100a.
//
//  * fb_gemm_ar_norm_big: row-parallel large-M GEMM (tcgen05, persistent, two TMEM accumulators) FUSED with the
//    cross-rank reduction, residual add, RMSNorm and all-gather in ONE kernel.  The GEMM warps write this rank's partial
//    tile (16-bit) into its own arena and post one arrival per epilogue warp on a per-row-block counter in the arena of the
//    block's owner (row block b of 128 tokens belongs to rank b % tp).  Four more warps per CTA are the reducers: they take
//    4-row jobs of the blocks this rank owns from a ticket, wait (bounded) until every rank has posted all tiles of the
//    block, pull the sum of all ranks' partial rows -- `multimem.ld_reduce` with fp32 accumulation, i.e. the addition is
//    done inside NVSwitch and each byte crosses this GPU's link once; plain peer loads when no multicast mapping exists --
//    add the residual row, keep the new residual row locally, normalise and broadcast the normalised row to every rank
//    (`multimem.st`).  Tiles are walked row-block-major, so the reduction of block b runs under the MMAs of the later
//    blocks: the transfer overlaps the math tile by tile.
//  * fb_ar_norm_big: the reducer part alone (all ranks meet on a counter first) for partial sums produced elsewhere:
//    quantised row-parallel projections, mixture-of-experts outputs.
//
// Reference counterpart: the two-stage branch of the custom all-reduce that takes over above 48-512 KiB
// (src/devices/multicuda/fastllm-custom-allreduce.cu:368, thresholds :976-980), a separate launch after a cuBLAS GEMM.
// Every wait here is bounded in time and reports through the error word; a reducer that gave up moves no data.
#include "gemm_largem.cuh"
#include "launch.h"
#include "tmap.h"
#include "comm.cuh"

FB_DEFINE_ERROR_API(comm_prefill)

namespace fb {

constexpr int KID_GEMM_AR_BIG = 33;
constexpr int KID_AR_BIG = 34;
constexpr int BIG_MAX_BLOCKS = 512;            // row blocks of 128 tokens the header has counters for
constexpr int BIG_JOB_ROWS = 4;
constexpr int BIG_JOBS_PER_BLOCK = 128 / BIG_JOB_ROWS;
// second header (32-bit words from off_hdr): ready[512] (remote arrivals) | expect[512] | done[512] | job ticket
constexpr uint32_t BIG_READY = 0, BIG_EXPECT = BIG_MAX_BLOCKS, BIG_DONE = 2 * BIG_MAX_BLOCKS, BIG_JOB_TICKET = 3 * BIG_MAX_BLOCKS;

struct BigArParams {
  CommCtx c;
  uint64_t off_hdr;          // second header (see above)
  uint64_t off_src;          // 16-bit [M, N]: this rank's partial sums (read by every rank)
  uint64_t off_h;            // 16-bit [M, N] residual stream (own row blocks are current)
  uint64_t off_x;            // 16-bit [M, N] normalised rows (all ranks)
  const uint16_t* ln_w;      // RMSNorm weight (nullptr: broadcast the summed rows themselves)
  const void* src;           // stand-alone kernel: partial to place at off_src first (nullptr: already there)
  int src_f32;
  int M, N;
  int has_residual;
  uint32_t ready_inc;        // arrivals per row block per launch in the fused kernel (tp * 4 epilogue warps * n-tiles)
  int trace;                 // != 0: CTA 0 writes globaltimer stamps of its phases to OFF_TRACE
  float eps, unit_offset;
};

template <bool BF16>
__device__ __forceinline__ uint4 mc_ld_reduce_16x8(const void* p) {
  uint4 v;
  if (BF16)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_b128(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// named barrier of one 128-thread group (ids 1 and 2 as immediates: a register operand would reserve all 16 barriers)
__device__ __forceinline__ void group_bar(int id) {
  if (id == 1) asm volatile("bar.sync 1, 128;\n" ::: "memory");
  else asm volatile("bar.sync 2, 128;\n" ::: "memory");
}

// Rows [row0, row0 + nrows) of the all-reduce, done by one group of 128 threads (gtid = 0..127, named barrier bar_id,
// sh_red = 16 floats of shared memory private to the group).  CPT = 16-byte chunks per thread per row (N <= CPT * 1024);
// RPP rows are in flight together, so a thread has RPP * CPT 16-byte loads outstanding per round trip.
// All threads of the group call this with the same arguments; `ok == false` walks the barriers but moves no data.
template <bool BF16, int CPT, int RPP>
__device__ __forceinline__ void big_reduce_rows(const BigArParams& p, int row0, int nrows, int gtid, int bar_id, float* sh_red, bool ok) {
  const CommCtx& c = p.c;
  const int N = p.N, chunks = N >> 3;
  int parity = 0;
  for (int r = 0; r < nrows; r += RPP, parity ^= 1) {
    const int nr = nrows - r < RPP ? nrows - r : RPP;
    uint4 hv[RPP][CPT];
    uint4 rv[RPP][CPT];
    float ss[RPP];
    // ---- loads first (all in flight together), then the arithmetic ----
#pragma unroll
    for (int rr = 0; rr < RPP; ++rr) {
      ss[rr] = 0.f;
#pragma unroll
      for (int k = 0; k < CPT; ++k) {
        const int ch = gtid + k * 128;
        hv[rr][k] = make_uint4(0u, 0u, 0u, 0u);
        rv[rr][k] = make_uint4(0u, 0u, 0u, 0u);
        if (ok && rr < nr && ch < chunks) {
          const size_t boff = ((size_t)(row0 + r + rr) * N + (size_t)ch * 8) * 2;
          if (c.mc) hv[rr][k] = mc_ld_reduce_16x8<BF16>(c.mc + p.off_src + boff);
          if (p.has_residual) rv[rr][k] = *reinterpret_cast<const uint4*>(c.local + p.off_h + boff);
        }
      }
    }
    if (!c.mc) {
      // plain peer loads: one round per rank (rank order: the same sum whoever owns the row), fp32 accumulators
      float acc[RPP][CPT][8];
#pragma unroll
      for (int rr = 0; rr < RPP; ++rr)
#pragma unroll
        for (int k = 0; k < CPT; ++k)
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[rr][k][j] = 0.f;
      // one round trip per rank; two ranks per round was measured slower (8192 x 4096 rows on two GPUs: 108 us against 96 us)
      for (int q = 0; q < c.tp; ++q) {
        const uint8_t* src = c.peer[q] + p.off_src;
#pragma unroll
        for (int rr = 0; rr < RPP; ++rr)
#pragma unroll
          for (int k = 0; k < CPT; ++k) {
            const int ch = gtid + k * 128;
            if (ok && rr < nr && ch < chunks)
              hv[rr][k] = ld_relaxed_sys_b128(src + ((size_t)(row0 + r + rr) * N + (size_t)ch * 8) * 2);
          }
#pragma unroll
        for (int rr = 0; rr < RPP; ++rr)
#pragma unroll
          for (int k = 0; k < CPT; ++k) {
            const uint4 s = hv[rr][k];
            const float2 s0 = unpack_16<BF16>(s.x), s1 = unpack_16<BF16>(s.y), s2 = unpack_16<BF16>(s.z), s3 = unpack_16<BF16>(s.w);
            float* a = acc[rr][k];
            a[0] += s0.x; a[1] += s0.y; a[2] += s1.x; a[3] += s1.y; a[4] += s2.x; a[5] += s2.y; a[6] += s3.x; a[7] += s3.y;
          }
      }
      // round once to the 16-bit format the multicast path delivers (its reduction also accumulates in fp32)
#pragma unroll
      for (int rr = 0; rr < RPP; ++rr)
#pragma unroll
        for (int k = 0; k < CPT; ++k) {
          const float* a = acc[rr][k];
          hv[rr][k] = make_uint4(pack_16<BF16>(a[0], a[1]), pack_16<BF16>(a[2], a[3]), pack_16<BF16>(a[4], a[5]), pack_16<BF16>(a[6], a[7]));
        }
    }
#pragma unroll
    for (int rr = 0; rr < RPP; ++rr) {
#pragma unroll
      for (int k = 0; k < CPT; ++k) {
        const int ch = gtid + k * 128;
        if (ok && rr < nr && ch < chunks) {
          const size_t boff = ((size_t)(row0 + r + rr) * N + (size_t)ch * 8) * 2;
          float v[8];
          const uint4 s = hv[rr][k];
          const float2 s0 = unpack_16<BF16>(s.x), s1 = unpack_16<BF16>(s.y), s2 = unpack_16<BF16>(s.z), s3 = unpack_16<BF16>(s.w);
          v[0] = s0.x; v[1] = s0.y; v[2] = s1.x; v[3] = s1.y; v[4] = s2.x; v[5] = s2.y; v[6] = s3.x; v[7] = s3.y;
          if (p.has_residual) {
            const uint4 q = rv[rr][k];
            const float2 q0 = unpack_16<BF16>(q.x), q1 = unpack_16<BF16>(q.y), q2 = unpack_16<BF16>(q.z), q3 = unpack_16<BF16>(q.w);
            v[0] += q0.x; v[1] += q0.y; v[2] += q1.x; v[3] += q1.y; v[4] += q2.x; v[5] += q2.y; v[6] += q3.x; v[7] += q3.y;
          }
          uint4 o;
          o.x = pack_16<BF16>(v[0], v[1]); o.y = pack_16<BF16>(v[2], v[3]); o.z = pack_16<BF16>(v[4], v[5]); o.w = pack_16<BF16>(v[6], v[7]);
          hv[rr][k] = o;
          // the norm sees the rounded values, exactly what a separate RMSNorm kernel would read back
          const float2 t0 = unpack_16<BF16>(o.x), t1 = unpack_16<BF16>(o.y), t2 = unpack_16<BF16>(o.z), t3 = unpack_16<BF16>(o.w);
          ss[rr] += t0.x * t0.x + t0.y * t0.y + t1.x * t1.x + t1.y * t1.y + t2.x * t2.x + t2.y * t2.y + t3.x * t3.x + t3.y * t3.y;
          *reinterpret_cast<uint4*>(c.local + p.off_h + boff) = o;      // the residual stream stays with the row's owner
          if (p.ln_w == nullptr) {
            if (c.mc) mc_st_b32x4(c.mc + p.off_x + boff, o);
            else for (int q = 0; q < c.tp; ++q) *reinterpret_cast<uint4*>(c.peer[q] + p.off_x + boff) = o;
          }
        }
      }
    }
    if (p.ln_w == nullptr) continue;
#pragma unroll
    for (int rr = 0; rr < RPP; ++rr) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss[rr] += __shfl_xor_sync(0xffffffffu, ss[rr], o);
    }
    float* red = sh_red + parity * 8;                       // [RPP rows][4 warps]; the other parity is still being read
    if ((gtid & 31) == 0) {
#pragma unroll
      for (int rr = 0; rr < RPP; ++rr) red[rr * 4 + (gtid >> 5)] = ss[rr];
    }
    group_bar(bar_id);
    float inv[RPP];
#pragma unroll
    for (int rr = 0; rr < RPP; ++rr) inv[rr] = rsqrtf((red[rr * 4] + red[rr * 4 + 1] + red[rr * 4 + 2] + red[rr * 4 + 3]) / (float)N + p.eps);
#pragma unroll
    for (int rr = 0; rr < RPP; ++rr) {
#pragma unroll
      for (int k = 0; k < CPT; ++k) {
        const int ch = gtid + k * 128;
        if (ok && rr < nr && ch < chunks) {
          const size_t boff = ((size_t)(row0 + r + rr) * N + (size_t)ch * 8) * 2;
          const uint4 h = hv[rr][k];
          const uint4 wv = *reinterpret_cast<const uint4*>(p.ln_w + (size_t)ch * 8);
          const float2 h0 = unpack_16<BF16>(h.x), h1 = unpack_16<BF16>(h.y), h2 = unpack_16<BF16>(h.z), h3 = unpack_16<BF16>(h.w);
          const float2 w0 = unpack_16<BF16>(wv.x), w1 = unpack_16<BF16>(wv.y), w2 = unpack_16<BF16>(wv.z), w3 = unpack_16<BF16>(wv.w);
          const float uo = p.unit_offset, iv = inv[rr];
          uint4 o;
          o.x = pack_16<BF16>(h0.x * iv * (w0.x + uo), h0.y * iv * (w0.y + uo));
          o.y = pack_16<BF16>(h1.x * iv * (w1.x + uo), h1.y * iv * (w1.y + uo));
          o.z = pack_16<BF16>(h2.x * iv * (w2.x + uo), h2.y * iv * (w2.y + uo));
          o.w = pack_16<BF16>(h3.x * iv * (w3.x + uo), h3.y * iv * (w3.y + uo));
          if (c.mc) mc_st_b32x4(c.mc + p.off_x + boff, o);
          else for (int q = 0; q < c.tp; ++q) *reinterpret_cast<uint4*>(c.peer[q] + p.off_x + boff) = o;
        }
      }
    }
  }
}

// End of a big launch, thread 0 of every CTA: one aggregated arrival of this rank on BOTH counters of every rank (the big
// kernels do not wait on the first one, but the other kernels expect both to advance by tp per launch), wait for every
// rank's rows, and the last CTA publishes the new expected value and rewinds the job ticket.
__device__ __forceinline__ void big_finish(const BigArParams& p, uint32_t base, int n_ctas, bool signal_cnt1, int kernel_id) {
  const CommCtx& c = p.c;
  const uint32_t target = base + (uint32_t)c.tp;
  __threadfence();
  uint32_t* lc = reinterpret_cast<uint32_t*>(c.local + OFF_LOCAL2);
  if (atomicAdd(lc, 1u) == (uint32_t)(n_ctas - 1)) {
    *lc = 0u;
    __threadfence_system();
    if (c.mc) {
      if (signal_cnt1) mc_red_add_relaxed_sys(reinterpret_cast<uint32_t*>(c.mc + OFF_CNT1), 1u);
      mc_red_add_relaxed_sys(reinterpret_cast<uint32_t*>(c.mc + OFF_CNT2), 1u);
    } else {
      for (int r = 0; r < c.tp; ++r) {
        if (signal_cnt1) red_add_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[r] + OFF_CNT1), 1u);
        red_add_relaxed_sys(reinterpret_cast<uint32_t*>(c.peer[r] + OFF_CNT2), 1u);
      }
    }
  }
  wait_counter(c, OFF_CNT2, target, kernel_id, 2);
  uint32_t* ticket = reinterpret_cast<uint32_t*>(c.local + OFF_TICKET);
  if (atomicAdd(ticket, 1u) == (uint32_t)(n_ctas - 1)) {
    *ticket = 0u;
    reinterpret_cast<uint32_t*>(c.local + p.off_hdr)[BIG_JOB_TICKET] = 0u;
    *reinterpret_cast<volatile uint32_t*>(c.local + OFF_EXPECT) = target;
    __threadfence();
  }
}

// ---- fused kernel: hooks of the large-M GEMM body ----
template <bool BF16, int CPT>
struct BigArHook {
  const BigArParams& p;
  int tiles_m;
  // row-block-major: the tiles of one row block finish together, early blocks are reduced under the MMAs of later ones
  __device__ __forceinline__ void tile_coords(int t, int tiles_m_, int tiles_n, int& m_tile, int& n_tile) const {
    m_tile = t / tiles_n; n_tile = t - m_tile * tiles_n;
  }
  __device__ __forceinline__ void tile_done(int m_tile, int n_tile, int lane) const {
    __syncwarp();                       // the lanes' row stores are ordered before lane 0's fence
    if (lane == 0) {
      if (p.trace && blockIdx.x == 0 && (threadIdx.x >> 5) == 2) reinterpret_cast<uint64_t*>(p.c.local + OFF_TRACE)[1] = globaltimer_ns();   // last write wins: this CTA's last tile
      __threadfence_system();
      uint32_t* ready = reinterpret_cast<uint32_t*>(p.c.peer[m_tile % p.c.tp] + p.off_hdr) + BIG_READY + m_tile;
      red_add_relaxed_sys(ready, 1u);
    }
  }
  __device__ __forceinline__ void extra_warps(int warp, int lane) const {
    __shared__ int sh_job, sh_ok;
    __shared__ uint32_t sh_target;
    bool gave_up = false;               // thread 0: after one wait ran out the later jobs do not wait again
    __shared__ float sh_red[16];
    const CommCtx& c = p.c;
    const int gtid = (int)threadIdx.x - 192;
    uint32_t* hdr = reinterpret_cast<uint32_t*>(c.local + p.off_hdr);
    const int owned = tiles_m > c.rank ? (tiles_m - c.rank + c.tp - 1) / c.tp : 0;
    const int total = owned * BIG_JOBS_PER_BLOCK;
    while (true) {
      if (gtid == 0) {
        const int j = (int)atomicAdd(hdr + BIG_JOB_TICKET, 1u);
        sh_job = j;
        if (j < total) {
          const int mt = c.rank + (j / BIG_JOBS_PER_BLOCK) * c.tp;
          const uint32_t target = *reinterpret_cast<volatile uint32_t*>(hdr + BIG_EXPECT + mt) + p.ready_inc;
          sh_target = target;
          const bool got = !gave_up && wait_counter_ge(hdr + BIG_READY + mt, target, KID_GEMM_AR_BIG, 1);
          gave_up = !got;
          sh_ok = got ? 1 : 0;
        }
      }
      group_bar(1);
      const int j = sh_job;
      if (j >= total) {
        if (p.trace && blockIdx.x == 0 && gtid == 0) reinterpret_cast<uint64_t*>(c.local + OFF_TRACE)[2] = globaltimer_ns();
        break;
      }
      const bool ok = sh_ok != 0;
      const uint32_t target = sh_target;
      const int mt = c.rank + (j / BIG_JOBS_PER_BLOCK) * c.tp;
      const int row0 = mt * 128 + (j % BIG_JOBS_PER_BLOCK) * BIG_JOB_ROWS;
      int nrows = p.M - row0; if (nrows > BIG_JOB_ROWS) nrows = BIG_JOB_ROWS;
      if (nrows > 0) big_reduce_rows<BF16, CPT, (CPT <= 4 ? 2 : 1)>(p, row0, nrows, gtid, 1, sh_red, ok);
      group_bar(1);                     // rows stored by every thread; sh_job / sh_ok free for the next claim
      if (gtid == 0) {
        __threadfence();
        if (atomicAdd(hdr + BIG_DONE + mt, 1u) == (uint32_t)(BIG_JOBS_PER_BLOCK - 1)) {
          hdr[BIG_DONE + mt] = 0u;
          *reinterpret_cast<volatile uint32_t*>(hdr + BIG_EXPECT + mt) = target;     // every job of the block has read the old value
        }
      }
    }
  }
};

template <int BN, bool BF16, int CPT>
__global__ void __launch_bounds__(320, 1)
gemm_ar_norm_big_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const GemmParams g,
                        const BigArParams p, int tiles_m, int tiles_n) {
  // launched without programmatic dependent launch: the previous collective has ended, its expected value is final
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(p.c.local + OFF_EXPECT);
  uint64_t* trace = (p.trace && blockIdx.x == 0) ? reinterpret_cast<uint64_t*>(p.c.local + OFF_TRACE) : nullptr;
  if (trace && threadIdx.x == 0) trace[0] = globaltimer_ns();
  BigArHook<BF16, CPT> hook{p, tiles_m};
  gemm_largem_device<BN, BF16, BigArHook<BF16, CPT>>(tmX, tmW, g, tiles_m, tiles_n, hook);
  if (threadIdx.x == 0) {
    if (trace) trace[3] = globaltimer_ns();             // this CTA's tiles and reducer jobs are done
    big_finish(p, base, (int)gridDim.x, true, KID_GEMM_AR_BIG);
    if (trace) trace[4] = globaltimer_ns();
  }
}

// ---- stand-alone kernel: 256 threads = two reducer groups, one row in flight per group, two CTAs per SM ----
template <bool BF16, int CPT>
__global__ void __launch_bounds__(256, 2) ar_norm_big_kernel(const BigArParams p) {
  __shared__ float sh_red[2][16];
  __shared__ int sh_ok;
  pdl_launch_dependents();
  pdl_wait();
  const CommCtx& c = p.c;
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(c.local + OFF_EXPECT);
  if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<uint64_t*>(c.local + OFF_TRACE)[0] = globaltimer_ns();
  const int chunks = p.N >> 3;
  if (p.src != nullptr) {
    // four 16-byte pieces per thread per trip, loads before stores
    const long long total = (long long)p.M * chunks;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += 4 * stride) {
      uint4 o[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long i = it + u * stride;
        if (i >= total) continue;
        if (p.src_f32) {
          const float4* sp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.src) + i * 8);
          const float4 a = sp[0], b = sp[1];
          o[u].x = pack_16<BF16>(a.x, a.y); o[u].y = pack_16<BF16>(a.z, a.w); o[u].z = pack_16<BF16>(b.x, b.y); o[u].w = pack_16<BF16>(b.z, b.w);
        } else {
          o[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.src) + i * 8);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const long long i = it + u * stride;
        if (i < total) *reinterpret_cast<uint4*>(c.local + p.off_src + (size_t)i * 16) = o[u];
      }
    }
  }
  uint64_t* trace = (p.trace && blockIdx.x == 0 && threadIdx.x == 0) ? reinterpret_cast<uint64_t*>(c.local + OFF_TRACE) : nullptr;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (trace) trace[1] = globaltimer_ns();
    arrive_aggregated(c, OFF_LOCAL1, OFF_CNT1, (int)gridDim.x);
    sh_ok = wait_counter(c, OFF_CNT1, base + (uint32_t)c.tp, KID_AR_BIG, 1) ? 1 : 0;
    if (trace) trace[2] = globaltimer_ns();
  }
  __syncthreads();
  const bool ok = sh_ok != 0;
  const int group = (int)threadIdx.x >> 7, gtid = (int)threadIdx.x & 127;
  const int tiles_m = (p.M + 127) / 128;
  const int owned = tiles_m > c.rank ? (tiles_m - c.rank + c.tp - 1) / c.tp : 0;
  const int total_jobs = owned * BIG_JOBS_PER_BLOCK;
  for (int j = (int)blockIdx.x * 2 + group; j < total_jobs; j += (int)gridDim.x * 2) {
    const int mt = c.rank + (j / BIG_JOBS_PER_BLOCK) * c.tp;
    const int row0 = mt * 128 + (j % BIG_JOBS_PER_BLOCK) * BIG_JOB_ROWS;
    int nrows = p.M - row0; if (nrows > BIG_JOB_ROWS) nrows = BIG_JOB_ROWS;
    if (nrows > 0) big_reduce_rows<BF16, CPT, 1>(p, row0, nrows, gtid, 1 + group, sh_red[group], ok);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (trace) trace[3] = globaltimer_ns();
    big_finish(p, base, (int)gridDim.x, false, KID_AR_BIG);
    if (trace) trace[4] = globaltimer_ns();
  }
}

static void fill_big(BigArParams& p, void* local, void* mc, void* const* peers, int rank, int tp, unsigned long long off_hdr,
                     unsigned long long off_src, unsigned long long off_h, unsigned long long off_x, const void* ln_w, int M, int N,
                     int has_residual, float eps, float unit_offset) {
  fill_ctx(p.c, local, mc, peers, rank, tp);
  p.off_hdr = off_hdr; p.off_src = off_src; p.off_h = off_h; p.off_x = off_x; p.ln_w = (const uint16_t*)ln_w;
  p.src = nullptr; p.src_f32 = 0; p.M = M; p.N = N; p.has_residual = has_residual & 1; p.trace = (has_residual >> 1) & 1; p.ready_inc = 0;
  p.eps = eps; p.unit_offset = unit_offset;
}

template <int BN, bool BF16, int CPT>
static cudaError_t launch_gemm_ar_big(const CUtensorMap& tmX, const CUtensorMap& tmW, const GemmParams& g, const BigArParams& p,
                                      int tiles_m, int tiles_n, cudaStream_t stream) {
  using Cfg = LargeMCfg<BN>;
  auto kern = gemm_ar_norm_big_kernel<BN, BF16, CPT>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  // every CTA's reducer warps may wait for tiles of any other CTA (of any rank): the whole grid must be resident,
  // which one CTA per SM guarantees
  const long long tiles = (long long)tiles_m * tiles_n;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  kern<<<grid, 320, Cfg::SMEM_BYTES, stream>>>(tmX, tmW, g, p, tiles_m, tiles_n);
  return cudaGetLastError();
}

}  // namespace fb

using namespace fb;

// Row-parallel projection of a prefill-sized batch with the tensor-parallel reduction behind it, one launch:
//   h[own row blocks] (+)= sum over ranks of X @ W^T ;  x[all rows, all ranks] = RMSNorm(h) * ln_w  (or the sums when ln_w is null)
// X [M, K_local] / W [N, K_local] are this rank's shards; bias is passed on one rank only.  off_*: symmetric arena offsets
// (hdr: 3 * 512 + 1 zeroed 32-bit words; src / h / x: 16-bit [M, N]).  256 < M <= 65536, N % 8 == 0, N <= 8192, K % 64 == 0.
extern "C" int fb_gemm_ar_norm_big(const void* X, const void* W, const void* bias, int M, int N, int K, int ldx, int ldw,
                                   void* arena_local, void* arena_mc, void* const* peers, int rank, int tp,
                                   unsigned long long off_hdr, unsigned long long off_src, unsigned long long off_h,
                                   unsigned long long off_x, const void* ln_w, int has_residual, float eps, float unit_offset,
                                   int dtype, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || M > BIG_MAX_BLOCKS * 128 || K % 64 != 0 || N % 8 != 0 || N > 8192 || tp > MAX_TP || tp < 1) return -1;
  const bool bf16 = dtype == 1;
  const int tiles_m = (M + 127) / 128;
  // narrower tiles when 256-wide ones would leave SMs without work
  const int bn = ((long long)tiles_m * ((N + 255) / 256) < sm_count() && N % 128 == 0) ? 128 : 256;
  const int tiles_n = (N + bn - 1) / bn;
  GemmParams g = {};
  g.out = (uint8_t*)arena_local + off_src; g.bias = bias; g.residual = nullptr;
  g.M = M; g.N = N; g.K = K; g.ld_out = N; g.ld_res = 0;
  g.kb_total = K / 64; g.kb_per_split = g.kb_total;
  g.flags = bias ? GEMM_BIAS : 0;
  g.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, bn);
  BigArParams p;
  fill_big(p, arena_local, arena_mc, peers, rank, tp, off_hdr, off_src, off_h, off_x, ln_w, M, N, has_residual, eps, unit_offset);
  p.ready_inc = (uint32_t)(tp * 4 * tiles_n);
  CUtensorMap tmX, tmW;
  if (!make_tmap_2d(&tmX, X, M, K, ldx, 128, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmW, W, N, K, ldw, bn, 64, 2, 3)) return -2;
  const bool wide = N > 4096;
#define FB_GB(BN_, CPT_)                                                                                         \
  return (int)(bf16 ? launch_gemm_ar_big<BN_, true, CPT_>(tmX, tmW, g, p, tiles_m, tiles_n, stream)               \
                    : launch_gemm_ar_big<BN_, false, CPT_>(tmX, tmW, g, p, tiles_m, tiles_n, stream));
  if (bn == 256) { if (wide) { FB_GB(256, 8) } else { FB_GB(256, 4) } }
  if (wide) { FB_GB(128, 8) } else { FB_GB(128, 4) }
#undef FB_GB
}

// All-reduce (+residual, +RMSNorm, all-gather) of this rank's partial [M, N]: `src` (fp32 if src_f32, else the 16-bit dtype) is
// placed at off_src first; src == nullptr means a previous kernel on this stream wrote it there.
extern "C" int fb_ar_norm_big(const void* src, int src_f32, int M, int N, void* arena_local, void* arena_mc, void* const* peers,
                              int rank, int tp, unsigned long long off_hdr, unsigned long long off_src, unsigned long long off_h,
                              unsigned long long off_x, const void* ln_w, int has_residual, float eps, float unit_offset, int dtype,
                              void* stream_) {
  if (M <= 0 || M > BIG_MAX_BLOCKS * 128 || N % 8 != 0 || N > 8192 || tp > MAX_TP || tp < 1) return -1;
  BigArParams p;
  fill_big(p, arena_local, arena_mc, peers, rank, tp, off_hdr, off_src, off_h, off_x, ln_w, M, N, has_residual, eps, unit_offset);
  p.src = src; p.src_f32 = src_f32;
  const int tiles_m = (M + 127) / 128;
  const int owned_max = (tiles_m + tp - 1) / tp;
  const bool bf16 = dtype == 1, wide = N > 4096;
  // the CTAs of a launch meet on a counter: all of them must be resident at once
  int per_sm = 0;
  cudaError_t oe;
  if (bf16) oe = wide ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ar_norm_big_kernel<true, 8>, 256, 0)
                      : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ar_norm_big_kernel<true, 4>, 256, 0);
  else oe = wide ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ar_norm_big_kernel<false, 8>, 256, 0)
                 : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, ar_norm_big_kernel<false, 4>, 256, 0);
  if (oe != cudaSuccess || per_sm < 1) per_sm = 1;
  if (per_sm > 2) per_sm = 2;
  int grid = (owned_max * BIG_JOBS_PER_BLOCK + 1) / 2;
  if (grid > sm_count() * per_sm) grid = sm_count() * per_sm;
  if (grid < 1) grid = 1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (bf16) { if (wide) launch_k(ar_norm_big_kernel<true, 8>, dim3(grid), dim3(256), 0, stream, 0, p); else launch_k(ar_norm_big_kernel<true, 4>, dim3(grid), dim3(256), 0, stream, 0, p); }
  else { if (wide) launch_k(ar_norm_big_kernel<false, 8>, dim3(grid), dim3(256), 0, stream, 0, p); else launch_k(ar_norm_big_kernel<false, 4>, dim3(grid), dim3(256), 0, stream, 0, p); }
  return (int)cudaGetLastError();
}
