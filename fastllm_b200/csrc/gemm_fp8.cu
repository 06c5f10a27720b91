// Block-scaled FP8 (e4m3 x e4m3) small-M GEMM for sm_100a: y = x W^T with 128x128 weight scales and 1x128 activation scales.
//
// Both operands stay FP8 all the way to the tensor core (tcgen05.mma kind::f8f6f4): the weight tile [128 n x 128 k] comes
// straight from the checkpoint layout by TMA, the activation tile [MPAD tokens x 128 k] from a buffer quantised by
// fb_quant_act_fp8 (per token and 128-wide k block).  Swap-AB like the 16-bit decode GEMM: weights are the UMMA A operand.
// One k block (four K=32 MMAs) accumulates into one of two TMEM buffers; the four promotion warps read it back, multiply by
// weight_scale[n tile, k block] * act_scale[token, k block] and add into fp32 registers while the tensor core fills the
// other buffer.  K is split over a thread-block cluster; partial tiles meet in distributed shared memory and the shared
// epilogue (bias -> SwiGLU -> residual -> store) finishes them.
//
// Reference: the W8A8 blockwise CUTLASS path exists only for sm89 / sm120 (src/devices/cuda/linear/fastllm-linear-fp8-cutlass.cu);
// on a B200 the reference runs FP8 weights as W8A16 GEMV / dequant + cuBLAS (fastllm-linear-fp8.cu:1778-1868).
#include "gemm_smallm.cuh"
#include "launch.h"
#include "tmap.h"
#include "comm.cuh"

FB_DEFINE_ERROR_API(gemm_fp8)

namespace fb {

constexpr int KID_GEMM_FP8 = 14;

template <int MPAD>
struct Fp8Cfg {
  static constexpr int A_BYTES = 128 * 128;              // 128 weight rows x 128 fp8
  static constexpr int B_BYTES = MPAD * 128;             // MPAD tokens x 128 fp8
  static constexpr int SC_OFF = A_BYTES + B_BYTES;       // this k block's activation scales (MPAD floats) travel with the tiles
  static constexpr int TX_BYTES = SC_OFF + MPAD * 4;
  static constexpr int STAGE_BYTES = SC_OFF + 1024;      // tiles stay 1024-byte aligned
  static constexpr int MAX_STAGES = (106 * 1024) / STAGE_BYTES;          // two CTAs per SM
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int RED_BYTES = MPAD * 128 * 4;
  static constexpr int PIPE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BODY_BYTES = PIPE_BYTES > RED_BYTES ? PIPE_BYTES : RED_BYTES;
  static constexpr int SMEM_BYTES = BODY_BYTES + 256 + 1024;
  static constexpr int NBUF = MPAD <= 64 ? 4 : 2;        // TMEM accumulator ring
  static constexpr int TMEM_COLS = NBUF * MPAD < 32 ? 32 : NBUF * MPAD;
};

struct Fp8Scales {
  const float* w_scale;      // [N / 128, kb_total]
  const float* a_scale;      // [kb_total, ld_a] (k-block major: one contiguous row of token scales per k block)
  int ld_a;
};

template <int MPAD, bool BF16>
__device__ __forceinline__ void gemm_fp8_device(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const Fp8Scales& sc) {
  using Cfg = Fp8Cfg<MPAD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BODY_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* tm_full = empty_bar + Cfg::STAGES;      // [NBUF] k block accumulated into TMEM buffer b
  uint64_t* tm_empty = tm_full + Cfg::NBUF;         // [NBUF] promotion warps have read buffer b
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tm_empty + Cfg::NBUF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = (int)cluster_ctarank();
  const int nsplit = (int)cluster_nctarank();
  const int n_tile = blockIdx.y;
  const int kb0 = split * p.kb_per_split;           // k blocks of 128
  int kb_cnt = p.kb_total - kb0;
  if (kb_cnt > p.kb_per_split) kb_cnt = p.kb_per_split;
  if (kb_cnt < 0) kb_cnt = 0;
  bool dead = false;
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    // a stage is released by the MMA commit (tiles) and the 128 promotion threads (scale row)
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 129); }
    for (int b = 0; b < Cfg::NBUF; ++b) { mbar_init(&tm_full[b], 1); mbar_init(&tm_empty[b], 128); }
    mbar_init_fence();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      const int pre = kb_cnt < Cfg::STAGES ? kb_cnt : Cfg::STAGES;
      for (int i = 0; i < pre; ++i) {          // weights do not depend on the previous kernel
        mbar_expect_tx(&full_bar[i], Cfg::TX_BYTES);
        tma_load_2d_hint(smem + i * Cfg::STAGE_BYTES, &tmW, &full_bar[i], (kb0 + i) * 128, p.w_row0 + n_tile * 128, pol_w);
      }
      pdl_wait();
      auto load_act = [&](int i, uint8_t* st, uint64_t* bar) {
        tma_load_2d_hint(st + Cfg::A_BYTES, &tmX, bar, (kb0 + i) * 128, p.x_row0, pol_x);
        bulk_load_1d(st + Cfg::SC_OFF, sc.a_scale + (size_t)(kb0 + i) * sc.ld_a + p.x_row0, MPAD * 4, bar);
      };
      for (int i = 0; i < pre; ++i) load_act(i, smem + i * Cfg::STAGE_BYTES, &full_bar[i]);
      for (int i = pre; i < kb_cnt; ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, dead, KID_GEMM_FP8, 1)) break;
        uint8_t* a = smem + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], Cfg::TX_BYTES);
        tma_load_2d_hint(a, &tmW, &full_bar[s], (kb0 + i) * 128, p.w_row0 + n_tile * 128, pol_w);
        load_act(i, a, &full_bar[s]);
      }
    }
    __syncwarp();
    pdl_wait();
  } else if (warp == 1) {
    if (elect_one()) {
      for (int i = 0; i < kb_cnt; ++i) {
        const int s = i % Cfg::STAGES, b = i % Cfg::NBUF;
        const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], ph, dead, KID_GEMM_FP8, 2)) break;
        if (!mbar_wait(&tm_empty[b], ((uint32_t)(i / Cfg::NBUF) & 1u) ^ 1u, dead, KID_GEMM_FP8, 3)) break;
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t da = make_smem_desc(a_addr, 16, 1024, SWZ_128B);
        const uint64_t db = make_smem_desc(a_addr + Cfg::A_BYTES, 16, 1024, SWZ_128B);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8(tmem_base + b * MPAD, da + 2 * k, db + 2 * k, p.idesc, k != 0 ? 1u : 0u);
        umma_commit(&empty_bar[s]);
        umma_commit(&tm_full[b]);
      }
    }
    __syncwarp();
  } else {
    // promotion warps: TMEM lanes [32q, 32q+32) = weight rows; one fp32 accumulator per token in registers
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    float acc[MPAD];
#pragma unroll
    for (int j = 0; j < MPAD; ++j) acc[j] = 0.f;
    pdl_wait();
    const float* wsp = sc.w_scale + (size_t)((p.w_row0 >> 7) + n_tile) * p.kb_total + kb0;
    constexpr int CH = MPAD < 32 ? MPAD : 32;
    for (int i = 0; i < kb_cnt; ++i) {
      const int b = i % Cfg::NBUF, s = i % Cfg::STAGES;
      const float ws = __ldg(wsp + i);               // issued before the waits: the latency overlaps the MMA of this block
      // the scale row is written by a bulk copy that completes on full_bar: observe it in this thread too
      if (!mbar_wait(&full_bar[s], (uint32_t)(i / Cfg::STAGES) & 1u, dead, KID_GEMM_FP8, 5)) break;
      if (!mbar_wait(&tm_full[b], (uint32_t)(i / Cfg::NBUF) & 1u, dead, KID_GEMM_FP8, 4)) break;
      tc_fence_after_sync();
      const float4* asp = reinterpret_cast<const float4*>(smem + s * Cfg::STAGE_BYTES + Cfg::SC_OFF);     // same address in every lane
#pragma unroll
      for (int c0 = 0; c0 < MPAD; c0 += CH) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + b * MPAD + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        if (CH == 32) tmem_ld_32x32b_x32(taddr, r); else tmem_ld_32x32b_x16(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < CH; j += 4) {
          const float4 a4 = asp[(c0 + j) >> 2];
          acc[c0 + j + 0] = fmaf(__uint_as_float(r[j + 0]), ws * a4.x, acc[c0 + j + 0]);
          acc[c0 + j + 1] = fmaf(__uint_as_float(r[j + 1]), ws * a4.y, acc[c0 + j + 1]);
          acc[c0 + j + 2] = fmaf(__uint_as_float(r[j + 2]), ws * a4.z, acc[c0 + j + 2]);
          acc[c0 + j + 3] = fmaf(__uint_as_float(r[j + 3]), ws * a4.w, acc[c0 + j + 3]);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tm_empty[b]);
      mbar_arrive(&empty_bar[s]);
    }
    // every MMA has completed (the last tm_full was observed) and every TMA tile was consumed: the ring becomes P
    float* P = reinterpret_cast<float*>(smem);
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
#pragma unroll
    for (int j = 0; j < MPAD; ++j) P[j * 128 + n_local] = acc[j];
  }
  tc_fence_before_sync();
  cluster_sync_all();
  smallm_reduce_store<BF16>(p, smem, split, nsplit, n_tile);
  cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

// Several output tiles per CTA (16-bit store, plain or SwiGLU; no k-split): the TMA ring, the MMA issue and the TMEM accumulator
// ring run on across the tiles, so a projection with a short k (an expert's projections: 6 to 16 k blocks) does not pay the
// pipeline fill, the barrier / TMEM set-up and the drain once per 128 output rows.  Tiles tile0 .. tile0 + ntile - 1 of the weight
// rows p.w_row0 + ...; activations as in gemm_fp8_device.  SwiGLU: rows 0..63 of a tile are gate rows and rows 64..127 the up rows
// of the same 64 output columns, so the two upper promotion warps hand their sums to the two lower ones through shared memory;
// that buffer takes the place of the last pipeline stage.
template <int MPAD, bool BF16>
__device__ __forceinline__ void gemm_fp8_multi_device(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const Fp8Scales& sc,
                                                      int tile0, int ntile, bool swiglu) {
  using Cfg = Fp8Cfg<MPAD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BODY_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* tm_full = empty_bar + Cfg::STAGES;
  uint64_t* tm_empty = tm_full + Cfg::NBUF;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tm_empty + Cfg::NBUF);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_cnt = p.kb_total;
  const int total = ntile * kb_cnt;
  const int nst = swiglu ? Cfg::STAGES - 1 : Cfg::STAGES;
  bool dead = false;
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 129); }
    for (int b = 0; b < Cfg::NBUF; ++b) { mbar_init(&tm_full[b], 1); mbar_init(&tm_empty[b], 128); }
    mbar_init_fence();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      for (int g = 0; g < total; ++g) {
        const int t = g / kb_cnt, i = g - t * kb_cnt;
        const int s = g % nst;
        if (g >= nst && !mbar_wait(&empty_bar[s], ((uint32_t)(g / nst) & 1u) ^ 1u, dead, KID_GEMM_FP8, 11)) break;
        uint8_t* a = smem + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], Cfg::TX_BYTES);
        tma_load_2d_hint(a, &tmW, &full_bar[s], i * 128, p.w_row0 + (tile0 + t) * 128, pol_w);
        tma_load_2d_hint(a + Cfg::A_BYTES, &tmX, &full_bar[s], i * 128, p.x_row0, pol_x);
        bulk_load_1d(a + Cfg::SC_OFF, sc.a_scale + (size_t)i * sc.ld_a + p.x_row0, MPAD * 4, &full_bar[s]);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      for (int g = 0; g < total; ++g) {
        const int s = g % nst, b = g % Cfg::NBUF;
        if (!mbar_wait(&full_bar[s], (uint32_t)(g / nst) & 1u, dead, KID_GEMM_FP8, 12)) break;
        if (!mbar_wait(&tm_empty[b], ((uint32_t)(g / Cfg::NBUF) & 1u) ^ 1u, dead, KID_GEMM_FP8, 13)) break;
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t da = make_smem_desc(a_addr, 16, 1024, SWZ_128B);
        const uint64_t db = make_smem_desc(a_addr + Cfg::A_BYTES, 16, 1024, SWZ_128B);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f8(tmem_base + b * MPAD, da + 2 * k, db + 2 * k, p.idesc, k != 0 ? 1u : 0u);
        umma_commit(&empty_bar[s]);
        umma_commit(&tm_full[b]);
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    constexpr int CH = MPAD < 32 ? MPAD : 32;
    uint16_t* outp = reinterpret_cast<uint16_t*>(p.out);
    float* X = reinterpret_cast<float*>(smem + nst * Cfg::STAGE_BYTES);      // [MPAD][64] up sums (SwiGLU only)
    int g = 0;
    for (int t = 0; t < ntile; ++t) {        // a thread whose wait ran out still walks the tiles: it meets the named barriers below
      float acc[MPAD];
#pragma unroll
      for (int j = 0; j < MPAD; ++j) acc[j] = 0.f;
      const float* wsp = sc.w_scale + (size_t)((p.w_row0 >> 7) + tile0 + t) * p.kb_total;
      for (int i = 0; i < kb_cnt; ++i, ++g) {
        const int b = g % Cfg::NBUF, s = g % nst;
        const float ws = __ldg(wsp + i);
        if (!mbar_wait(&full_bar[s], (uint32_t)(g / nst) & 1u, dead, KID_GEMM_FP8, 15)) break;
        if (!mbar_wait(&tm_full[b], (uint32_t)(g / Cfg::NBUF) & 1u, dead, KID_GEMM_FP8, 14)) break;
        tc_fence_after_sync();
        const float4* asp = reinterpret_cast<const float4*>(smem + s * Cfg::STAGE_BYTES + Cfg::SC_OFF);
#pragma unroll
        for (int c0 = 0; c0 < MPAD; c0 += CH) {
          uint32_t r[32];
          const uint32_t taddr = tmem_base + b * MPAD + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
          if (CH == 32) tmem_ld_32x32b_x32(taddr, r); else tmem_ld_32x32b_x16(taddr, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CH; j += 4) {
            const float4 a4 = asp[(c0 + j) >> 2];
            acc[c0 + j + 0] = fmaf(__uint_as_float(r[j + 0]), ws * a4.x, acc[c0 + j + 0]);
            acc[c0 + j + 1] = fmaf(__uint_as_float(r[j + 1]), ws * a4.y, acc[c0 + j + 1]);
            acc[c0 + j + 2] = fmaf(__uint_as_float(r[j + 2]), ws * a4.z, acc[c0 + j + 2]);
            acc[c0 + j + 3] = fmaf(__uint_as_float(r[j + 3]), ws * a4.w, acc[c0 + j + 3]);
          }
        }
        tc_fence_before_sync();
        mbar_arrive(&tm_empty[b]);
        mbar_arrive(&empty_bar[s]);
      }
      if (swiglu) {
        // producer / consumer named barriers: 2 = "up sums of this tile are in X", 1 = "X has been read"
        if (q >= 2) {
          if (t > 0) asm volatile("bar.sync 1, 128;\n" ::: "memory");
#pragma unroll
          for (int j = 0; j < MPAD; ++j) X[j * 64 + n_local - 64] = acc[j];
          asm volatile("bar.arrive 2, 128;\n" ::: "memory");
        } else {
          asm volatile("bar.sync 2, 128;\n" ::: "memory");
          const int n_out = (tile0 + t) * 64 + n_local;
          const bool live = !dead && n_out < (p.N >> 1);
#pragma unroll
          for (int j = 0; j < MPAD; ++j) {
            const float u = X[j * 64 + n_local];
            if (live && j < p.M) outp[(size_t)j * p.ld_out + n_out] = (uint16_t)(pack_16<BF16>(silu_f(acc[j]) * u, 0.f) & 0xFFFFu);
          }
          if (t + 1 < ntile) asm volatile("bar.arrive 1, 128;\n" ::: "memory");
        }
        continue;
      }
      if (dead) continue;
      // a lane owns one output column; consecutive lanes write consecutive columns of a token's row
      const int n = (tile0 + t) * 128 + n_local;
      if (n < p.N) {
#pragma unroll
        for (int j = 0; j < MPAD; ++j)
          if (j < p.M) outp[(size_t)j * p.ld_out + n] = (uint16_t)(pack_16<BF16>(acc[j], 0.f) & 0xFFFFu);
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int MPAD, bool BF16>
__global__ void __launch_bounds__(192, (MPAD <= 64 ? 2 : 1))
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams p, const Fp8Scales sc) {
  gemm_fp8_device<MPAD, BF16>(tmW, tmX, p, sc);
}

// Row-parallel projection of a tensor-parallel rank FUSED with the collective behind it: the epilogue pushes the fp32 partial
// rows to their owners' arenas, then the shared tail (csrc/comm.cuh) meets the other ranks, reduces, adds the residual,
// normalises and broadcasts -- one launch instead of GEMM + all-reduce kernel.
template <int MPAD, bool BF16>
__global__ void __launch_bounds__(192, (MPAD <= 64 ? 2 : 1))
gemm_fp8_ar_norm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams g,
                        const Fp8Scales sc, const ArNormParams p) {
  const uint64_t t_start = p.trace ? globaltimer_ns() : 0;
  gemm_fp8_device<MPAD, BF16>(tmW, tmX, g, sc);
  // every thread has passed the dependency wait inside the GEMM: the expect word written by the previous collective is final
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(p.c.local + OFF_EXPECT);
  if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) reinterpret_cast<uint64_t*>(p.c.local + OFF_TRACE)[0] = t_start;
  ar_norm_tail<BF16>(p, base, blockIdx.y, gridDim.y, blockIdx.x, gridDim.x, KID_GEMM_AR);
}

// Grouped (mixture-of-experts) variant over the expert-sorted activation buffer: blockIdx.z = expert * chunks + chunk.
struct Fp8GroupInfo {
  const int* counts; const int* offsets;
  int rows_per_chunk, chunks, n_rows_w;
  int n_local, compact;        // compact: grid.z enumerates existing (expert, chunk) pairs (moe_find_item)
  int tiles_per_cta;           // > 1: blockIdx.y walks this many 128-row output tiles (plain store, see gemm_fp8_multi_device)
};

template <int MPAD, bool BF16>
__global__ void __launch_bounds__(192, (MPAD <= 64 ? 2 : 1))
moe_grouped_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams base,
                       const Fp8Scales sbase, const Fp8GroupInfo gi) {
  int e = blockIdx.z / gi.chunks, chunk = blockIdx.z - e * gi.chunks;
  pdl_launch_dependents();
  pdl_wait();                         // counts / offsets come from the plan kernel
  if (gi.compact && !moe_find_item(gi.counts, gi.n_local, gi.rows_per_chunk, (int)blockIdx.z, e, chunk)) return;
  const int cnt = gi.counts[e];
  const int row0 = chunk * gi.rows_per_chunk;
  if (row0 >= cnt) return;            // uniform over the cluster (same blockIdx.z)
  GemmParams p = base;
  const int seg = gi.offsets[e] + row0;
  p.M = cnt - row0 < gi.rows_per_chunk ? cnt - row0 : gi.rows_per_chunk;
  p.x_row0 = seg;
  p.w_row0 = e * gi.n_rows_w;         // stacked weights: the weight-scale tile index (w_row0 / 128 + n_tile) follows from it
  p.out = reinterpret_cast<uint16_t*>(base.out) + (size_t)seg * base.ld_out;
  if (gi.tiles_per_cta > 1) {
    const int tile0 = blockIdx.y * gi.tiles_per_cta, n_tiles = p.N >> 7;
    const int nt = n_tiles - tile0 < gi.tiles_per_cta ? n_tiles - tile0 : gi.tiles_per_cta;
    gemm_fp8_multi_device<MPAD, BF16>(tmW, tmX, p, sbase, tile0, nt, (p.flags & GEMM_SWIGLU) != 0);
    return;
  }
  gemm_fp8_device<MPAD, BF16>(tmW, tmX, p, sbase);
}

// ---- activation quantisation: x [M, K] 16-bit -> xq [M, K] e4m3 + scales [K / 128, ld_a] ------------------------------------

template <bool BF16>
__global__ void quant_act_fp8_kernel(const uint16_t* __restrict__ x, int ldx, uint8_t* __restrict__ xq, int ldq, float* __restrict__ scales,
                                     int ld_a, int M, int kb_total, const int* __restrict__ rows_used) {
  pdl_launch_dependents();
  pdl_wait();
  const int wpb = blockDim.x >> 5;
  const int gw = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int m = gw / kb_total, kb = gw - m * kb_total;
  if (m >= M) return;
  if (rows_used != nullptr && m >= *rows_used) return;         // expert-sorted buffers: rows behind the last routed token
  const uint2 v = *reinterpret_cast<const uint2*>(x + (size_t)m * ldx + kb * 128 + lane * 4);
  const float2 a = unpack_16<BF16>(v.x), b = unpack_16<BF16>(v.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 448.0f;
  const float inv = 1.0f / scale;
  *reinterpret_cast<uint32_t*>(xq + (size_t)m * ldq + kb * 128 + lane * 4) = pack_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
  if (lane == 0) scales[(size_t)kb * ld_a + m] = scale;
}

// Rounds activations to the values the 8-bit-activation GEMMs see (per token and 128-wide k block; INT8: round(x / s) * s with
// s = amax / 127, else e4m3 with s = amax / 448) and writes them back as 16-bit numbers.  Batches too large for the small-M
// 8-bit kernels run the 16-bit-activation kernels on these values, so a request gets the same numerics at every batch size.
template <bool BF16, bool INT8>
__global__ void round_act_kernel(const uint16_t* __restrict__ x, int ldx, uint16_t* __restrict__ out, int ldo, int M, int kb_total) {
  pdl_launch_dependents();
  pdl_wait();
  const int wpb = blockDim.x >> 5;
  const int gw = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int m = gw / kb_total, kb = gw - m * kb_total;
  if (m >= M) return;
  const uint2 v = *reinterpret_cast<const uint2*>(x + (size_t)m * ldx + kb * 128 + lane * 4);
  const float2 a = unpack_16<BF16>(v.x), b = unpack_16<BF16>(v.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  float r0, r1, r2, r3;
  if (INT8) {
    const float scale = fmaxf(amax, 1e-12f) / 127.0f, inv = 1.0f / scale;
    r0 = rintf(a.x * inv) * scale; r1 = rintf(a.y * inv) * scale; r2 = rintf(b.x * inv) * scale; r3 = rintf(b.y * inv) * scale;
  } else {
    const float scale = fmaxf(amax, 1e-12f) / 448.0f, inv = 1.0f / scale;
    const uint32_t q = pack_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
    uint32_t h01, h23;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h01) : "h"((uint16_t)(q & 0xFFFFu)));
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h23) : "h"((uint16_t)(q >> 16)));
    const float2 f01 = __half22float2(*reinterpret_cast<const __half2*>(&h01)), f23 = __half22float2(*reinterpret_cast<const __half2*>(&h23));
    r0 = f01.x * scale; r1 = f01.y * scale; r2 = f23.x * scale; r3 = f23.y * scale;
  }
  uint2 o;
  o.x = pack_16<BF16>(r0, r1);
  o.y = pack_16<BF16>(r2, r3);
  *reinterpret_cast<uint2*>(out + (size_t)m * ldo + kb * 128 + lane * 4) = o;
}

// Gather for the grouped expert GEMM fused with the activation quantisation: row pos[pair] of the expert-sorted FP8 buffer
// receives token pair / topk, quantised per 128-wide k block.  One CTA per (token, k) pair, one warp per k block.
template <bool BF16>
__global__ void moe_gather_quant_fp8_kernel(const uint16_t* __restrict__ x, const int* __restrict__ pos, uint8_t* __restrict__ xq,
                                            float* __restrict__ scales, int ld_a, int topk, int H) {
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x;
  const int r = pos[pair];
  if (r < 0) return;
  const int t = pair / topk;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int kb = warp; kb < (H >> 7); kb += nw) {
    const uint2 v = *reinterpret_cast<const uint2*>(x + (size_t)t * H + kb * 128 + lane * 4);
    const float2 a = unpack_16<BF16>(v.x), b = unpack_16<BF16>(v.y);
    float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax, 1e-12f) / 448.0f;
    const float inv = 1.0f / scale;
    *reinterpret_cast<uint32_t*>(xq + (size_t)r * H + kb * 128 + lane * 4) = pack_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
    if (lane == 0) scales[(size_t)kb * ld_a + r] = scale;
  }
}

}  // namespace fb

using namespace fb;

extern "C" int fb_gemm_pick_split(int M, int N, int K, int slots);

extern "C" int fb_moe_gather_quant_fp8(const void* x, const int* pos, void* xq, float* scales, int ld_a, int T, int topk, int H, int dtype,
                                       void* stream) {
  if (T <= 0) return 0;
  if (H % 128 != 0) return -1;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1)
    launch_k(moe_gather_quant_fp8_kernel<true>, dim3(T * topk), dim3(128), 0, s, 0, (const uint16_t*)x, pos, (uint8_t*)xq, scales, ld_a, topk, H);
  else
    launch_k(moe_gather_quant_fp8_kernel<false>, dim3(T * topk), dim3(128), 0, s, 0, (const uint16_t*)x, pos, (uint8_t*)xq, scales, ld_a, topk, H);
  return (int)cudaGetLastError();
}

// mode 0: int8 grid, 1: e4m3 grid.  x, out: [M, K] 16-bit (row strides ldx, ldo elements, multiples of 4); K % 128 == 0.
extern "C" int fb_round_act(const void* x, int ldx, void* out, int ldo, int M, int K, int dtype, int mode, void* stream) {
  if (M <= 0) return 0;
  if (K % 128 != 0 || ldx % 4 != 0 || ldo % 4 != 0 || (mode != 0 && mode != 1)) return -1;
  const int kb_total = K / 128, wpb = 8;
  const long long warps = (long long)M * kb_total;
  const dim3 grid((unsigned)((warps + wpb - 1) / wpb)), block(wpb * 32);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  auto xi = (const uint16_t*)x;
  auto xo = (uint16_t*)out;
  if (dtype == 1) {
    if (mode == 0) launch_k(round_act_kernel<true, true>, grid, block, 0, s, 0, xi, ldx, xo, ldo, M, kb_total);
    else launch_k(round_act_kernel<true, false>, grid, block, 0, s, 0, xi, ldx, xo, ldo, M, kb_total);
  } else {
    if (mode == 0) launch_k(round_act_kernel<false, true>, grid, block, 0, s, 0, xi, ldx, xo, ldo, M, kb_total);
    else launch_k(round_act_kernel<false, false>, grid, block, 0, s, 0, xi, ldx, xo, ldo, M, kb_total);
  }
  return (int)cudaGetLastError();
}

extern "C" int fb_quant_act_fp8(const void* x, int ldx, void* xq, int ldq, float* scales, int ld_a, int M, int K, int dtype,
                                const int* rows_used, void* stream) {
  if (M <= 0) return 0;
  if (K % 128 != 0 || ldx % 4 != 0 || ldq % 4 != 0) return -1;
  const int kb_total = K / 128, wpb = 8;
  const int warps = M * kb_total;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1)
    launch_k(quant_act_fp8_kernel<true>, dim3((warps + wpb - 1) / wpb), dim3(wpb * 32), 0, s, 0, (const uint16_t*)x, ldx, (uint8_t*)xq, ldq, scales, ld_a, M, kb_total, rows_used);
  else
    launch_k(quant_act_fp8_kernel<false>, dim3((warps + wpb - 1) / wpb), dim3(wpb * 32), 0, s, 0, (const uint16_t*)x, ldx, (uint8_t*)xq, ldq, scales, ld_a, M, kb_total, rows_used);
  return (int)cudaGetLastError();
}

template <int MPAD, bool BF16>
static cudaError_t launch_fp8(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const Fp8Scales& sc, int nsplit,
                              int n_tiles, cudaStream_t stream) {
  using Cfg = Fp8Cfg<MPAD>;
  auto kern = gemm_fp8_kernel<MPAD, BF16>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, n_tiles, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nsplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = add_pdl_attr(attr, 1);
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, sc);
}

template <int MPAD, bool BF16>
static cudaError_t launch_fp8_ar(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& g, const Fp8Scales& sc,
                                 const ArNormParams& p, int nsplit, int n_tiles, cudaStream_t stream) {
  using Cfg = Fp8Cfg<MPAD>;
  auto kern = gemm_fp8_ar_norm_kernel<MPAD, BF16>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, n_tiles, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nsplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = add_pdl_attr(attr, 1);
  // all CTAs wait for each other across ranks: they must all be resident at once
  int max_clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters <= 0 || n_tiles > max_clusters)
    return cudaErrorLaunchOutOfResources;
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, g, sc, p);
}

// Fused form of fb_gemm_fp8 for a row-parallel projection under tensor parallelism (see fb_gemm_ar_norm in comm.cu for the arena
// arguments and `flags`: bit 0 residual, bit 1 trace, bit 2 deferred all-gather wait).  N = hidden size, M <= 128.
// Returns cudaErrorLaunchOutOfResources (701) when the grid cannot be co-resident: the caller runs GEMM + collective then.
extern "C" int fb_gemm_fp8_ar_norm(const void* xq, int ldq, const float* a_scale, int ld_a, const void* Wq, const float* w_scale,
                                   const void* bias, int M, int N, int K, void* arena_local, void* arena_mc, void* const* peers, int rank,
                                   int tp, unsigned long long off_part, unsigned long long off_h, unsigned long long off_x,
                                   const void* ln_w, int flags, float eps, float unit_offset, int dtype, void* stream_) {
  if (M <= 0 || M > 128 || K % 128 != 0 || N % 8 != 0 || N > 18432 || tp > MAX_TP || tp < 1) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int mpad = 16;
  while (mpad < M) mpad <<= 1;
  const int n_tiles = (N + 127) / 128;
  const int kb_total = K / 128;
  const int slots = sm_count() * (mpad <= 64 ? 2 : 1);
  int nsplit = 1;
  while (nsplit < 8 && n_tiles * nsplit * 2 <= slots && kb_total / (nsplit * 2) >= 4) nsplit <<= 1;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, Wq, (uint64_t)N, (uint64_t)K, (uint64_t)K, 128, 128, 1, 3)) return -2;
  if (!make_tmap_2d(&tmX, xq, (uint64_t)M, (uint64_t)K, (uint64_t)ldq, mpad, 128, 1, 3)) return -2;
  GemmParams g = {};
  g.bias = bias; g.M = M; g.N = N; g.K = K;
  g.kb_total = kb_total; g.kb_per_split = (kb_total + nsplit - 1) / nsplit; g.flags = GEMM_OUT_F32 | (bias ? GEMM_BIAS : 0);
  g.idesc = make_idesc(0, 0, 0, 0, 128, mpad);
  fill_scatter(g, arena_local, peers, off_part, M, N, rank, tp);
  Fp8Scales sc;
  sc.w_scale = w_scale; sc.a_scale = a_scale; sc.ld_a = ld_a;
  ArNormParams p;
  fill_ar_norm(p, arena_local, arena_mc, peers, rank, tp, off_part, off_h, off_x, ln_w, M, N, flags, eps, unit_offset);
  cudaError_t e;
#define FB_F8A(MP)                                                                                       \
  e = dtype == 1 ? launch_fp8_ar<MP, true>(tmW, tmX, g, sc, p, nsplit, n_tiles, stream)                   \
                 : launch_fp8_ar<MP, false>(tmW, tmX, g, sc, p, nsplit, n_tiles, stream);                 \
  break;
  for (;;) {            // a k-split whose clusters cannot all be resident at once is halved until they can
    g.kb_per_split = (kb_total + nsplit - 1) / nsplit;
    switch (mpad) {
      case 16: FB_F8A(16)
      case 32: FB_F8A(32)
      case 64: FB_F8A(64)
      default: FB_F8A(128)
    }
    if (e != cudaErrorLaunchOutOfResources || nsplit == 1) break;
    nsplit >>= 1;
  }
#undef FB_F8A
  return (int)e;
}

// xq: [M, K] e4m3 (row stride ldq bytes), a_scale: [K / 128, ld_a]; Wq: [N, K] e4m3, w_scale: [ceil(N / 128), K / 128].
// out / bias / residual are 16-bit (dtype 0 = fp16, 1 = bf16) unless GEMM_OUT_F32.  M <= 128.
extern "C" int fb_gemm_fp8(const void* xq, int ldq, const float* a_scale, int ld_a, const void* Wq, const float* w_scale, void* out,
                           const void* bias, const void* residual, int M, int N, int K, int ld_out, int ld_res, int dtype, int flags,
                           int nsplit, void* stream_) {
  if (M <= 0) return 0;
  if (M > 128 || K % 128 != 0 || N % 8 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int mpad = 16;
  while (mpad < M) mpad <<= 1;
  const int n_tiles = (N + 127) / 128;
  const int kb_total = K / 128;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (nsplit <= 0) {
    nsplit = 1;
    const int slots = sm_count * (mpad <= 64 ? 2 : 1);
    while (nsplit < 8 && n_tiles * nsplit * 2 <= slots && kb_total / (nsplit * 2) >= 4) nsplit <<= 1;
  }
  if ((flags & GEMM_SWIGLU) && nsplit > 8) nsplit = 8;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, Wq, (uint64_t)N, (uint64_t)K, (uint64_t)K, 128, 128, 1, 3)) return -2;
  if (!make_tmap_2d(&tmX, xq, (uint64_t)M, (uint64_t)K, (uint64_t)ldq, mpad, 128, 1, 3)) return -2;
  GemmParams p = {};
  p.out = out; p.bias = bias; p.residual = residual; p.M = M; p.N = N; p.K = K; p.ld_out = ld_out; p.ld_res = ld_res;
  p.kb_total = kb_total; p.kb_per_split = (kb_total + nsplit - 1) / nsplit; p.flags = flags;
  p.idesc = make_idesc(0, 0, 0, 0, 128, mpad);
  Fp8Scales sc;
  sc.w_scale = w_scale; sc.a_scale = a_scale; sc.ld_a = ld_a;
  cudaError_t e;
#define FB_F8(MP)                                                                                        \
  e = dtype == 1 ? launch_fp8<MP, true>(tmW, tmX, p, sc, nsplit, n_tiles, stream)                        \
                 : launch_fp8<MP, false>(tmW, tmX, p, sc, nsplit, n_tiles, stream);                      \
  break;
  switch (mpad) {
    case 16: FB_F8(16)
    case 32: FB_F8(32)
    case 64: FB_F8(64)
    default: FB_F8(128)
  }
#undef FB_F8
  return (int)e;
}

template <int MPAD, bool BF16>
static cudaError_t launch_grouped_fp8(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const Fp8Scales& sc,
                                      const Fp8GroupInfo& gi, int nsplit, int n_tiles, int nz, cudaStream_t stream) {
  using Cfg = Fp8Cfg<MPAD>;
  auto kern = moe_grouped_fp8_kernel<MPAD, BF16>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, n_tiles, nz);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nsplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = add_pdl_attr(attr, 1);
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, sc, gi);
}

// Grouped expert GEMM over the expert-sorted, FP8-quantised activation buffer xq [rows_cap, K]; stacked weights
// Wq [E_local * N, K] with scales [E_local, ceil(N / 128), K / 128].  max_rows: low 16 bits = most rows an expert can hold,
// high 16 bits = rows per chunk hint (0: derived).
// Output tiles per CTA of the plain grouped projection: 0 picks from the grid size, 1 keeps one tile per CTA, n >= 2 forces n.
static int g_moe_fp8_tiles = [] { const char* e = getenv("FB_MOE_FP8_TILES"); return e ? atoi(e) : 0; }();
extern "C" int fb_moe_grouped_fp8_set_tiles(int tiles) {
  const int old = g_moe_fp8_tiles;
  g_moe_fp8_tiles = tiles < 0 ? 0 : tiles;
  return old;
}

extern "C" int fb_moe_grouped_gemm_fp8(const void* xq, int ldq, const float* a_scale, int ld_a, const void* Wq, const float* w_scale,
                                       void* out, const int* counts, const int* offsets, int n_local, int N, int K, int rows_cap,
                                       int ld_out, int dtype, int flags, int max_rows, int total_rows, void* stream_) {
  // total_rows > 0: upper bound of the routed rows over all local experts; the grid then has one slot per existing row chunk
  if (n_local <= 0 || rows_cap <= 0) return 0;
  if (K % 128 != 0 || N % 128 != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int hint = (max_rows >> 16) & 0xFFFF;
  max_rows &= 0xFFFF;
  if (max_rows <= 0) max_rows = rows_cap;
  int mpad = 16;
  const int want = hint > 0 ? hint : max_rows;
  while (mpad < want && mpad < 64) mpad <<= 1;
  const int chunks = (max_rows + mpad - 1) / mpad;
  const int n_tiles = N / 128, kb_total = K / 128;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, Wq, (uint64_t)n_local * N, (uint64_t)K, (uint64_t)K, 128, 128, 1, 3)) return -2;
  if (!make_tmap_2d(&tmX, xq, (uint64_t)rows_cap, (uint64_t)K, (uint64_t)ldq, mpad, 128, 1, 3)) return -2;
  GemmParams p = {};
  p.out = out; p.M = mpad; p.N = N; p.K = K; p.ld_out = ld_out; p.flags = flags;
  p.kb_total = kb_total; p.kb_per_split = kb_total;
  p.idesc = make_idesc(0, 0, 0, 0, 128, mpad);
  Fp8Scales sc;
  sc.w_scale = w_scale; sc.a_scale = a_scale; sc.ld_a = ld_a;
  Fp8GroupInfo gi;
  gi.counts = counts; gi.offsets = offsets; gi.rows_per_chunk = mpad; gi.chunks = chunks; gi.n_rows_w = N;
  gi.n_local = n_local; gi.compact = 0; gi.tiles_per_cta = 1;
  int nz = n_local * chunks;
  if (total_rows > 0) {
    const int bound = n_local + (total_rows + mpad - 1) / mpad;       // sum of ceil(count / mpad) <= experts + rows / mpad
    if (bound < nz) { nz = bound; gi.compact = 1; }
  }
  int grid_y = n_tiles;
  const bool multi_kind = flags == 0 || flags == GEMM_SWIGLU;
  if (multi_kind && g_moe_fp8_tiles >= 2) {
    gi.tiles_per_cta = g_moe_fp8_tiles < n_tiles ? g_moe_fp8_tiles : n_tiles;
    grid_y = (n_tiles + gi.tiles_per_cta - 1) / gi.tiles_per_cta;
  } else if (multi_kind && g_moe_fp8_tiles == 0 && kb_total <= 32) {
    // an expert's projections have a short k: a CTA walks several output tiles, as many as leave about one CTA per slot of the
    // GPU (two CTAs per SM).  The number of (expert, row chunk) items that exist is estimated between its bounds.
    static int slots = 0;
    if (slots == 0) {
      int dev = 0, sms = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      slots = 2 * sms;
    }
    int est = total_rows > 0 ? n_local + total_rows / (2 * mpad) : nz;
    if (est > nz) est = nz;
    int gy = (slots + est / 2) / est;
    gy = gy < 1 ? 1 : (gy > n_tiles ? n_tiles : gy);
    const int nt = (n_tiles + gy - 1) / gy;
    gi.tiles_per_cta = nt;
    grid_y = (n_tiles + nt - 1) / nt;
  }
  cudaError_t e;
#define FB_G8(MP)                                                                                                         \
  e = dtype == 1 ? launch_grouped_fp8<MP, true>(tmW, tmX, p, sc, gi, 1, grid_y, nz, stream)                               \
                 : launch_grouped_fp8<MP, false>(tmW, tmX, p, sc, gi, 1, grid_y, nz, stream);                             \
  break;
  switch (mpad) {
    case 16: FB_G8(16)
    case 32: FB_G8(32)
    default: FB_G8(64)
  }
#undef FB_G8
  return (int)e;
}
