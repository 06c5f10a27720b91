// Integer small-M GEMM for sm_100a: 8-bit activations x int8 / int4-group weights on the tensor core (tcgen05.mma kind::i8).
//
// The 16-bit-activation kernels for these weight formats (gemm_quant.cu) convert every weight tile to bf16 in shared memory
// and are bound by that conversion (slower than the plain bf16 GEMM at decode sizes).  Here the weights reach the tensor core
// as signed bytes: int8 weights directly by TMA (stored as q - 128), int4-group weights after a nibble -> byte unpack that is
// four bit operations per eight values.  Activations are quantised per token and 128-wide k block to int8 by
// fb_quant_act_i8, which also records the block sums of the quantised values (needed for zero points / group minima).
// One k block = four K=32 MMAs into one buffer of a TMEM ring (exact int32 sums); the promotion warps turn it into fp32:
//     int8 per channel  (w = s_n (q - z_n)):        acc[m] += sum * a[m,kb];   T[m] += xs[m,kb] * a[m,kb]   finally s_n (acc - z'_n T)
//     int4 group g = kb (w = min_ng + s_ng q):      acc[m] += (sum * s_ng + min_ng * xs[m,kb]) * a[m,kb]     ((s, min) as [kb, n] pairs)
// with z' = z - 128, xs = sum of the quantised activations of the block, a = activation scale.  The a / xs rows of a k block
// travel with its tiles (bulk copy into the stage), so the promotion reads them from shared memory instead of waiting on L2
// once per k block.  Split-K clusters and the epilogue are the ones of the 16-bit decode GEMM.
//
// Reference kernels for these formats: CUDA-core GEMV / dequant + cuBLAS (src/devices/cuda/linear/fastllm-linear-int8.cu,
// fastllm-linear-int4group.cu) and Marlin mma.sync (fastllm-marlin.cu).
#include "gemm_smallm.cuh"
#include "launch.h"
#include "tmap.h"
#include "comm.cuh"

FB_DEFINE_ERROR_API(gemm_i8)

namespace fb {

constexpr int KID_GEMM_I8 = 15;
constexpr int WK_INT8 = 1, WK_INT4G = 2;

template <int MPAD, int WK>
struct I8Cfg {
  static constexpr int A_BYTES = 128 * 128;                              // 128 weight rows x 128 int8 (MMA operand)
  static constexpr int RAW_BYTES = WK == WK_INT4G ? 128 * 64 : 0;        // packed nibbles of one k block
  static constexpr int B_BYTES = MPAD * 128;
  static constexpr int W_BYTES = WK == WK_INT4G ? RAW_BYTES : A_BYTES;
  static constexpr int SC_OFF = B_BYTES + W_BYTES;                       // activation scales, then block sums (MPAD floats each)
  static constexpr int TX_BYTES = SC_OFF + 2 * MPAD * 4;
  // int8: the TMA tile is the operand.  int4g: TMA brings the packed tile, the unpack fills one of two operand slots.
  static constexpr int STAGE_BYTES = SC_OFF + 1024;
  static constexpr int DQ_SLOTS = WK == WK_INT4G ? 2 : 0;
  static constexpr int BUDGET = 106 * 1024 - DQ_SLOTS * A_BYTES;      // two CTAs per SM
  static constexpr int MAX_STAGES = BUDGET / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 8 ? 8 : MAX_STAGES;
  static constexpr int RED_BYTES = MPAD * 128 * 4;
  static constexpr int PIPE_BYTES = DQ_SLOTS * A_BYTES + STAGES * STAGE_BYTES;
  static constexpr int BODY_BYTES = PIPE_BYTES > RED_BYTES ? PIPE_BYTES : RED_BYTES;
  static constexpr int SMEM_BYTES = BODY_BYTES + 1024 + 1024;          // barriers (256 B) + zero-point sums T (MPAD floats at +512)
  // int4g with few rows: four extra warps do nothing but unpack nibbles, so the unpack of block i + 1 and the promotion of
  // block i run side by side instead of one after the other in the same four warps (102 registers per thread at two CTAs
  // per SM are enough for sixteen accumulators)
  static constexpr bool SPLIT = WK == WK_INT4G && MPAD <= 16;
  static constexpr int THREADS = SPLIT ? 320 : 192;
  static constexpr int NBUF = MPAD <= 64 ? 4 : 2;                        // TMEM accumulator ring
  static constexpr int TMEM_COLS = NBUF * MPAD < 32 ? 32 : NBUF * MPAD;
};

struct I8Scales {
  const float* w_scale;      // int8: [N];  int4g: float2 (scale, min) [kb_total, n_rows] (a warp reads one line per k block)
  const float* w_zero;       // int8: zero point - 128 [N];  int4g: unused
  int n_rows;                // int4g: rows of the (scale, min) table = weight rows of this matrix
  const float* a_scale;      // [kb_total, ld_a]
  const float* a_sum;        // [kb_total, ld_a]  sums of the quantised activations per block
  int ld_a;
};

__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// instruction descriptor for kind::i8: D = s32 (2), A and B = signed 8 bit (1), both K-major
__host__ __device__ constexpr uint32_t make_idesc_i8(uint32_t M, uint32_t N) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// int32 block sum -> float without the conversion pipe: |v| < 2^22 (127 * 128 * 128 at most), so v + 0x4B400000 is the bit
// pattern of 1.5 * 2^23 + v
__device__ __forceinline__ float sum_to_float(uint32_t v) { return __uint_as_float(v + 0x4B400000u) - 12582912.0f; }

// int4g: unpack the packed tile of k block i into operand slot i & 1 (thread t of 128 handles 16-byte chunks t, t + 128, ...)
template <class Cfg>
__device__ __forceinline__ void unpack_int4_tile(int i, int tid, uint8_t* stages, uint8_t* dq, uint64_t* full_bar, uint64_t* empty_bar,
                                                 uint64_t* dq_full, uint64_t* dq_empty, bool& dead) {
  const int s = i % Cfg::STAGES, b = i & 1;
  const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u, bph = ((uint32_t)i >> 1) & 1u;
  if (!mbar_wait(&full_bar[s], ph, dead, KID_GEMM_I8, 6)) return;
  if (!mbar_wait(&dq_empty[b], bph ^ 1u, dead, KID_GEMM_I8, 7)) return;
  const uint8_t* raw = stages + s * Cfg::STAGE_BYTES + Cfg::B_BYTES;
  uint8_t* out = dq + b * Cfg::A_BYTES;
  uint4 pk[4];                                         // all four loads first: the stores below must not serialise them
#pragma unroll
  for (int it = 0; it < 4; ++it) pk[it] = *reinterpret_cast<const uint4*>(raw + (tid + it * 128) * 16);
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int idx = tid + it * 128;                  // 512 chunks of 16 packed bytes
    const int row = idx >> 2, c4 = idx & 3;
    uint32_t o[8];
    const uint32_t w4[4] = {pk[it].x, pk[it].y, pk[it].z, pk[it].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const uint32_t hi = (w4[e] >> 4) & 0x0F0F0F0Fu, lo = w4[e] & 0x0F0F0F0Fu;      // first value of a byte = high nibble
      o[2 * e] = __byte_perm(hi, lo, 0x5140);
      o[2 * e + 1] = __byte_perm(hi, lo, 0x7362);
    }
    uint8_t* rowp = out + row * 128;
    const int c0 = 2 * c4, c1 = 2 * c4 + 1;
    *reinterpret_cast<uint4*>(rowp + ((c0 ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(rowp + ((c1 ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
  }
  fence_proxy_async_smem();
  mbar_arrive(&dq_full[b]);
  if (Cfg::SPLIT) mbar_arrive(&empty_bar[s]);          // dedicated unpack warps: the packed tile is theirs to release
}

template <int MPAD, bool BF16, int WK>
__device__ __forceinline__ void gemm_i8_device(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const I8Scales& sc) {
  using Cfg = I8Cfg<MPAD, WK>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* dq = smem;                                               // int4g: two unpacked operand slots (1024-aligned)
  uint8_t* stages = smem + Cfg::DQ_SLOTS * Cfg::A_BYTES;            // per stage: [activation tile | weight tile (int8) or packed tile (int4g)]
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BODY_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;     // MMA commit + 128 promotion arrivals (scales read, packed tile unpacked)
  uint64_t* tm_full = empty_bar + Cfg::STAGES;      // [NBUF]
  uint64_t* tm_empty = tm_full + Cfg::NBUF;         // [NBUF]
  uint64_t* dq_full = tm_empty + Cfg::NBUF;         // [2] int4g: operand slot unpacked (128 arrivals)
  uint64_t* dq_empty = dq_full + 2;                 // [2] int4g: MMA of that slot committed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(dq_empty + 2);
  // activation tiles must start on 1024-byte boundaries (128-byte swizzle): B first in every stage, stage sizes are multiples of 1024
  static_assert(Cfg::STAGE_BYTES % 1024 == 0, "stage size");

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
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], Cfg::SPLIT ? 257 : 129); }
    for (int b = 0; b < Cfg::NBUF; ++b) { mbar_init(&tm_full[b], 1); mbar_init(&tm_empty[b], 128); }
    for (int b = 0; b < 2; ++b) { mbar_init(&dq_full[b], 128); mbar_init(&dq_empty[b], 1); }
    mbar_init_fence();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  constexpr int WBYTES = WK == WK_INT4G ? 64 : 128;       // weight bytes per row and k block in global memory

  if (warp == 0) {
    if (elect_one()) {
      const uint64_t pol_w = l2_policy_evict_first();
      const uint64_t pol_x = l2_policy_evict_last();
      const int pre = kb_cnt < Cfg::STAGES ? kb_cnt : Cfg::STAGES;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], Cfg::TX_BYTES);
        tma_load_2d_hint(stages + i * Cfg::STAGE_BYTES + Cfg::B_BYTES, &tmW, &full_bar[i], (kb0 + i) * WBYTES, p.w_row0 + n_tile * 128, pol_w);
      }
      pdl_wait();
      auto load_act = [&](int i, uint8_t* st, uint64_t* bar) {
        tma_load_2d_hint(st, &tmX, bar, (kb0 + i) * 128, p.x_row0, pol_x);
        const size_t off = (size_t)(kb0 + i) * sc.ld_a + p.x_row0;
        bulk_load_1d(st + Cfg::SC_OFF, sc.a_scale + off, MPAD * 4, bar);
        bulk_load_1d(st + Cfg::SC_OFF + MPAD * 4, sc.a_sum + off, MPAD * 4, bar);
      };
      for (int i = 0; i < pre; ++i) load_act(i, stages + i * Cfg::STAGE_BYTES, &full_bar[i]);
      for (int i = pre; i < kb_cnt; ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, dead, KID_GEMM_I8, 1)) break;
        uint8_t* st = stages + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], Cfg::TX_BYTES);
        tma_load_2d_hint(st + Cfg::B_BYTES, &tmW, &full_bar[s], (kb0 + i) * WBYTES, p.w_row0 + n_tile * 128, pol_w);
        load_act(i, st, &full_bar[s]);
      }
    }
    __syncwarp();
    pdl_wait();
  } else if (warp == 1) {
    if (elect_one()) {
      for (int i = 0; i < kb_cnt; ++i) {
        const int s = i % Cfg::STAGES, b = i % Cfg::NBUF, d = i & 1;
        const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u, bph = (uint32_t)(i / Cfg::NBUF) & 1u, dph = ((uint32_t)i >> 1) & 1u;
        if (!mbar_wait(&full_bar[s], ph, dead, KID_GEMM_I8, 2)) break;
        if (WK == WK_INT4G && !mbar_wait(&dq_full[d], dph, dead, KID_GEMM_I8, 5)) break;
        if (!mbar_wait(&tm_empty[b], bph ^ 1u, dead, KID_GEMM_I8, 3)) break;
        tc_fence_after_sync();
        const uint32_t x_addr = smem_u32(stages + s * Cfg::STAGE_BYTES);
        const uint32_t w_addr = WK == WK_INT4G ? smem_u32(dq + d * Cfg::A_BYTES) : x_addr + Cfg::B_BYTES;
        const uint64_t da = make_smem_desc(w_addr, 16, 1024, SWZ_128B);
        const uint64_t db = make_smem_desc(x_addr, 16, 1024, SWZ_128B);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_i8(tmem_base + b * MPAD, da + 2 * k, db + 2 * k, p.idesc, k != 0 ? 1u : 0u);
        umma_commit(&empty_bar[s]);
        if (WK == WK_INT4G) umma_commit(&dq_empty[d]);
        umma_commit(&tm_full[b]);
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // dedicated unpack warps (SPLIT configurations only)
    const int tid = threadIdx.x - 192;
    for (int i = 0; i < kb_cnt; ++i) unpack_int4_tile<Cfg>(i, tid, stages, dq, full_bar, empty_bar, dq_full, dq_empty, dead);
  } else {
    const int q = warp & 3;
    const int n_local = q * 32 + lane;
    const int tid = threadIdx.x - 64;                    // 0..127 among the four promotion warps
    float acc[MPAD];
    float tsum = 0.f;                                    // int8: T[m] of token m = tid over this CTA's k range
#pragma unroll
    for (int j = 0; j < MPAD; ++j) acc[j] = 0.f;
    pdl_wait();
    const int n_glob = p.w_row0 + n_tile * 128 + n_local;
    const bool n_ok = n_tile * 128 + n_local < p.N;
    float zrow = 0.f, srow = 1.f;
    if (WK == WK_INT8 && n_ok) { zrow = sc.w_zero[n_glob]; srow = sc.w_scale[n_glob]; }
    constexpr int CH = MPAD < 32 ? MPAD : 32;

    if (WK == WK_INT4G && !Cfg::SPLIT && kb_cnt > 0) unpack_int4_tile<Cfg>(0, tid, stages, dq, full_bar, empty_bar, dq_full, dq_empty, dead);
    for (int i = 0; i < kb_cnt; ++i) {
      if (WK == WK_INT4G && !Cfg::SPLIT && i + 1 < kb_cnt) unpack_int4_tile<Cfg>(i + 1, tid, stages, dq, full_bar, empty_bar, dq_full, dq_empty, dead);
      const int b = i % Cfg::NBUF, s = i % Cfg::STAGES;
      float wa = 1.f, wb = 0.f;
      if (WK == WK_INT4G && n_ok) {                 // issued before the wait: the latency overlaps the MMA of this block
        const float2 sm = __ldg(reinterpret_cast<const float2*>(sc.w_scale) + (size_t)(kb0 + i) * sc.n_rows + n_tile * 128 + n_local);
        wa = sm.x; wb = sm.y;
      }
      // the scale rows are written by the bulk copies that complete on full_bar: observe it in this thread too
      if ((WK == WK_INT8 || Cfg::SPLIT) && !mbar_wait(&full_bar[s], (uint32_t)(i / Cfg::STAGES) & 1u, dead, KID_GEMM_I8, 8)) break;
      if (!mbar_wait(&tm_full[b], (uint32_t)(i / Cfg::NBUF) & 1u, dead, KID_GEMM_I8, 4)) break;
      tc_fence_after_sync();
      const float4* asp = reinterpret_cast<const float4*>(stages + s * Cfg::STAGE_BYTES + Cfg::SC_OFF);      // same address in every lane
      const float4* xsp = asp + MPAD / 4;
      if (WK == WK_INT8 && tid < MPAD)
        tsum = fmaf(reinterpret_cast<const float*>(xsp)[tid], reinterpret_cast<const float*>(asp)[tid], tsum);
#pragma unroll
      for (int c0 = 0; c0 < MPAD; c0 += CH) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + b * MPAD + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        if (CH == 32) tmem_ld_32x32b_x32(taddr, r); else tmem_ld_32x32b_x16(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < CH; j += 4) {
          const float4 a4 = asp[(c0 + j) >> 2];
          if (WK == WK_INT8) {
            acc[c0 + j + 0] = fmaf(sum_to_float(r[j + 0]), a4.x, acc[c0 + j + 0]);
            acc[c0 + j + 1] = fmaf(sum_to_float(r[j + 1]), a4.y, acc[c0 + j + 1]);
            acc[c0 + j + 2] = fmaf(sum_to_float(r[j + 2]), a4.z, acc[c0 + j + 2]);
            acc[c0 + j + 3] = fmaf(sum_to_float(r[j + 3]), a4.w, acc[c0 + j + 3]);
          } else {
            const float4 x4 = xsp[(c0 + j) >> 2];
            acc[c0 + j + 0] = fmaf(fmaf(sum_to_float(r[j + 0]), wa, wb * x4.x), a4.x, acc[c0 + j + 0]);
            acc[c0 + j + 1] = fmaf(fmaf(sum_to_float(r[j + 1]), wa, wb * x4.y), a4.y, acc[c0 + j + 1]);
            acc[c0 + j + 2] = fmaf(fmaf(sum_to_float(r[j + 2]), wa, wb * x4.z), a4.z, acc[c0 + j + 2]);
            acc[c0 + j + 3] = fmaf(fmaf(sum_to_float(r[j + 3]), wa, wb * x4.w), a4.w, acc[c0 + j + 3]);
          }
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&tm_empty[b]);
      mbar_arrive(&empty_bar[s]);
    }
    float* P = reinterpret_cast<float*>(smem);
    float* Tsm = reinterpret_cast<float*>(smem + Cfg::BODY_BYTES + 512);
    if (WK == WK_INT8 && tid < MPAD) Tsm[tid] = tsum;
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
#pragma unroll
    for (int j = 0; j < MPAD; ++j) {
      const float v = WK == WK_INT8 ? fmaf(-zrow, Tsm[j], acc[j]) : acc[j];
      P[j * 128 + n_local] = n_ok ? v * srow : 0.f;
    }
  }
  tc_fence_before_sync();
  cluster_sync_all();
  smallm_reduce_store<BF16>(p, smem, split, nsplit, n_tile);
  cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int MPAD, bool BF16, int WK>
__global__ void __launch_bounds__((I8Cfg<MPAD, WK>::THREADS), (MPAD <= 64 ? 2 : 1))
gemm_i8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams p, const I8Scales sc) {
  gemm_i8_device<MPAD, BF16, WK>(tmW, tmX, p, sc);
}

// Row-parallel projection of a tensor-parallel rank fused with the collective behind it (see gemm_fp8_ar_norm_kernel).
template <int MPAD, bool BF16, int WK>
__global__ void __launch_bounds__((I8Cfg<MPAD, WK>::THREADS), (MPAD <= 64 ? 2 : 1))
gemm_i8_ar_norm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams g,
                       const I8Scales sc, const ArNormParams p) {
  const uint64_t t_start = p.trace ? globaltimer_ns() : 0;
  gemm_i8_device<MPAD, BF16, WK>(tmW, tmX, g, sc);
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(p.c.local + OFF_EXPECT);
  if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) reinterpret_cast<uint64_t*>(p.c.local + OFF_TRACE)[0] = t_start;
  ar_norm_tail<BF16>(p, base, blockIdx.y, gridDim.y, blockIdx.x, gridDim.x, KID_GEMM_AR);
}

struct I8GroupInfo {
  const int* counts; const int* offsets;
  int rows_per_chunk, chunks, n_rows_w;
  int n_local, compact;        // compact: grid.z enumerates existing (expert, chunk) pairs (moe_find_item)
};

template <int MPAD, bool BF16, int WK>
__global__ void __launch_bounds__((I8Cfg<MPAD, WK>::THREADS), (MPAD <= 64 ? 2 : 1))
moe_grouped_i8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams base,
                      const I8Scales sbase, const I8GroupInfo gi) {
  int e = blockIdx.z / gi.chunks, chunk = blockIdx.z - e * gi.chunks;
  pdl_launch_dependents();
  pdl_wait();
  if (gi.compact && !moe_find_item(gi.counts, gi.n_local, gi.rows_per_chunk, (int)blockIdx.z, e, chunk)) return;
  const int cnt = gi.counts[e];
  const int row0 = chunk * gi.rows_per_chunk;
  if (row0 >= cnt) return;
  GemmParams p = base;
  const int seg = gi.offsets[e] + row0;
  p.M = cnt - row0 < gi.rows_per_chunk ? cnt - row0 : gi.rows_per_chunk;
  p.x_row0 = seg;
  p.w_row0 = e * gi.n_rows_w;         // per-row scale tables of the stacked experts are indexed by w_row0 + row
  p.out = reinterpret_cast<uint16_t*>(base.out) + (size_t)seg * base.ld_out;
  I8Scales sc = sbase;
  if (WK == WK_INT4G) sc.w_scale = sbase.w_scale + (size_t)e * base.kb_total * gi.n_rows_w * 2;      // [E, kb_total, N, 2]
  gemm_i8_device<MPAD, BF16, WK>(tmW, tmX, p, sc);
}

// ---- activation quantisation: x [M, K] 16-bit -> int8 [M, K], scales and block sums [K / 128, ld_a] ------------------------
template <bool BF16>
__global__ void quant_act_i8_kernel(const uint16_t* __restrict__ x, int ldx, int8_t* __restrict__ xq, int ldq, float* __restrict__ scales,
                                    float* __restrict__ sums, int ld_a, int M, int kb_total, const int* __restrict__ rows_used,
                                    const int* __restrict__ pos, int topk) {
  pdl_launch_dependents();
  pdl_wait();
  const int wpb = blockDim.x >> 5;
  const int gw = blockIdx.x * wpb + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int m = gw / kb_total, kb = gw - m * kb_total;
  if (m >= M) return;
  int src = m, dst = m;
  if (pos != nullptr) {                 // gather mode: m enumerates (token, k) pairs, the row goes to pos[m] of the sorted buffer
    dst = pos[m];
    if (dst < 0) return;
    src = m / topk;
  } else if (rows_used != nullptr && m >= *rows_used) {
    return;
  }
  const uint2 v = *reinterpret_cast<const uint2*>(x + (size_t)src * ldx + kb * 128 + lane * 4);
  const float2 a = unpack_16<BF16>(v.x), b = unpack_16<BF16>(v.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 127.0f;
  const float inv = 1.0f / scale;
  const int q0 = __float2int_rn(a.x * inv), q1 = __float2int_rn(a.y * inv), q2 = __float2int_rn(b.x * inv), q3 = __float2int_rn(b.y * inv);
  *reinterpret_cast<uint32_t*>(xq + (size_t)dst * ldq + kb * 128 + lane * 4) =
      (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
  int s = q0 + q1 + q2 + q3;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) { scales[(size_t)kb * ld_a + dst] = scale; sums[(size_t)kb * ld_a + dst] = (float)s; }
}

}  // namespace fb

using namespace fb;

// pos == null: quantise rows [0, M) (or [0, *rows_used)).  pos != null: M = tokens * topk pairs, row pos[pair] <- token pair / topk.
extern "C" int fb_quant_act_i8(const void* x, int ldx, void* xq, int ldq, float* scales, float* sums, int ld_a, int M, int K, int dtype,
                               const int* rows_used, const int* pos, int topk, void* stream) {
  if (M <= 0) return 0;
  if (K % 128 != 0 || ldx % 4 != 0 || ldq % 4 != 0) return -1;
  const int kb_total = K / 128, wpb = 8;
  const int warps = M * kb_total;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1)
    launch_k(quant_act_i8_kernel<true>, dim3((warps + wpb - 1) / wpb), dim3(wpb * 32), 0, s, 0, (const uint16_t*)x, ldx, (int8_t*)xq, ldq,
             scales, sums, ld_a, M, kb_total, rows_used, pos, topk);
  else
    launch_k(quant_act_i8_kernel<false>, dim3((warps + wpb - 1) / wpb), dim3(wpb * 32), 0, s, 0, (const uint16_t*)x, ldx, (int8_t*)xq, ldq,
             scales, sums, ld_a, M, kb_total, rows_used, pos, topk);
  return (int)cudaGetLastError();
}

template <int MPAD, bool BF16, int WK>
static cudaError_t launch_i8(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const I8Scales& sc, const I8GroupInfo* gi,
                             int nsplit, int n_tiles, int nz, cudaStream_t stream) {
  using Cfg = I8Cfg<MPAD, WK>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, n_tiles, nz);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nsplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = add_pdl_attr(attr, 1);
  if (gi == nullptr) {
    auto kern = gemm_i8_kernel<MPAD, BF16, WK>;
    static DeviceOnce configured;
    if (configured.need()) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
      if (e != cudaSuccess) return e;
    }
    return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, sc);
  }
  auto kern = moe_grouped_i8_kernel<MPAD, BF16, WK>;
  static DeviceOnce configured_g;
  if (configured_g.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, sc, *gi);
}

template <int WK>
static int dispatch_i8(int mpad, int dtype, const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const I8Scales& sc,
                       const I8GroupInfo* gi, int nsplit, int n_tiles, int nz, cudaStream_t stream) {
  cudaError_t e;
#define FB_I8(MP)                                                                                                  \
  e = dtype == 1 ? launch_i8<MP, true, WK>(tmW, tmX, p, sc, gi, nsplit, n_tiles, nz, stream)                       \
                 : launch_i8<MP, false, WK>(tmW, tmX, p, sc, gi, nsplit, n_tiles, nz, stream);                     \
  break;
  switch (mpad) {
    case 16: FB_I8(16)
    case 32: FB_I8(32)
    case 64: FB_I8(64)
    default: FB_I8(128)
  }
#undef FB_I8
  return (int)e;
}

template <int MPAD, bool BF16, int WK>
static cudaError_t launch_i8_ar(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& g, const I8Scales& sc,
                                const ArNormParams& p, int nsplit, int n_tiles, cudaStream_t stream) {
  using Cfg = I8Cfg<MPAD, WK>;
  auto kern = gemm_i8_ar_norm_kernel<MPAD, BF16, WK>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, n_tiles, 1);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nsplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = add_pdl_attr(attr, 1);
  int max_clusters = 0;                 // all CTAs wait for each other across ranks: they must all be resident at once
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) != cudaSuccess || max_clusters <= 0 || n_tiles > max_clusters)
    return cudaErrorLaunchOutOfResources;
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, g, sc, p);
}

template <int WK>
static int dispatch_i8_ar(int mpad, int dtype, const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& g, const I8Scales& sc,
                          const ArNormParams& p, int nsplit, int n_tiles, cudaStream_t stream) {
  cudaError_t e;
#define FB_I8A(MP)                                                                                                 \
  e = dtype == 1 ? launch_i8_ar<MP, true, WK>(tmW, tmX, g, sc, p, nsplit, n_tiles, stream)                          \
                 : launch_i8_ar<MP, false, WK>(tmW, tmX, g, sc, p, nsplit, n_tiles, stream);                        \
  break;
  switch (mpad) {
    case 16: FB_I8A(16)
    case 32: FB_I8A(32)
    case 64: FB_I8A(64)
    default: FB_I8A(128)
  }
#undef FB_I8A
  return (int)e;
}

// Fused form of fb_gemm_i8 (plain, not grouped) for a row-parallel projection under tensor parallelism; arena arguments and
// `flags` as in fb_gemm_ar_norm (comm.cu).  Returns 701 when the grid cannot be co-resident.
extern "C" int fb_gemm_i8_ar_norm(const void* xq, int ldq, const float* a_scale, const float* a_sum, int ld_a, const void* Wq,
                                  const float* w_scale, const float* w_zero, const void* bias, int M, int N, int K, int wkind,
                                  void* arena_local, void* arena_mc, void* const* peers, int rank, int tp, unsigned long long off_part,
                                  unsigned long long off_h, unsigned long long off_x, const void* ln_w, int flags, float eps,
                                  float unit_offset, int dtype, void* stream_) {
  if (M <= 0 || M > 128 || K % 128 != 0 || N % 8 != 0 || N > 18432 || tp > MAX_TP || tp < 1) return -1;
  if (wkind != WK_INT8 && wkind != WK_INT4G) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int kb_total = K / 128;
  const int wbytes = wkind == WK_INT4G ? K / 2 : K;
  int mpad = 16;
  while (mpad < M) mpad <<= 1;
  const int n_tiles = (N + 127) / 128;
  const int slots = sm_count() * (mpad <= 64 ? 2 : 1);
  int nsplit = 1;
  while (nsplit < 8 && n_tiles * nsplit * 2 <= slots && kb_total / (nsplit * 2) >= 4) nsplit <<= 1;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, Wq, (uint64_t)N, (uint64_t)wbytes, (uint64_t)wbytes, 128, wkind == WK_INT4G ? 64 : 128, 1, wkind == WK_INT4G ? 0 : 3)) return -2;
  if (!make_tmap_2d(&tmX, xq, (uint64_t)M, (uint64_t)K, (uint64_t)ldq, mpad, 128, 1, 3)) return -2;
  GemmParams g = {};
  g.bias = bias; g.M = M; g.N = N; g.K = K; g.kb_total = kb_total; g.kb_per_split = (kb_total + nsplit - 1) / nsplit;
  g.flags = GEMM_OUT_F32 | (bias ? GEMM_BIAS : 0);
  g.idesc = make_idesc_i8(128, mpad);
  fill_scatter(g, arena_local, peers, off_part, M, N, rank, tp);
  I8Scales sc;
  sc.w_scale = w_scale; sc.w_zero = w_zero; sc.a_scale = a_scale; sc.a_sum = a_sum; sc.ld_a = ld_a; sc.n_rows = N;
  ArNormParams p;
  fill_ar_norm(p, arena_local, arena_mc, peers, rank, tp, off_part, off_h, off_x, ln_w, M, N, flags, eps, unit_offset);
  for (;;) {            // a k-split whose clusters cannot all be resident at once is halved until they can
    g.kb_per_split = (kb_total + nsplit - 1) / nsplit;
    const int rc = wkind == WK_INT8 ? dispatch_i8_ar<WK_INT8>(mpad, dtype, tmW, tmX, g, sc, p, nsplit, n_tiles, stream)
                                    : dispatch_i8_ar<WK_INT4G>(mpad, dtype, tmW, tmX, g, sc, p, nsplit, n_tiles, stream);
    if (rc != (int)cudaErrorLaunchOutOfResources || nsplit == 1) return rc;
    nsplit >>= 1;
  }
}

// wkind: 1 = int8 per channel (Wq int8 = q - 128, w_scale [N], w_zero = zero - 128 [N]);
//        2 = int4 group 128 (Wq packed [N, K / 2], w_scale = float2 (scale, min) [K / 128, N], per expert when grouped; w_zero unused).
// counts == null: plain GEMM, M <= 128.  counts != null: grouped over the expert-sorted buffer (rows_cap rows, n_local experts,
// M = upper bound of the routed rows or 0,
// max_rows: low 16 bits = most rows of one expert, high 16 bits = rows-per-chunk hint).
extern "C" int fb_gemm_i8(const void* xq, int ldq, const float* a_scale, const float* a_sum, int ld_a, const void* Wq, const float* w_scale,
                          const float* w_zero, void* out, const void* bias, const void* residual, int M, int N, int K, int ld_out,
                          int ld_res, int dtype, int flags, int wkind, int nsplit, const int* counts, const int* offsets, int n_local,
                          int rows_cap, int max_rows, void* stream_) {
  if (M <= 0 && counts == nullptr) return 0;
  if (K % 128 != 0 || N % 8 != 0 || (wkind != WK_INT8 && wkind != WK_INT4G)) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int kb_total = K / 128;
  const int wbytes = wkind == WK_INT4G ? K / 2 : K;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  GemmParams p = {};
  p.out = out; p.bias = bias; p.residual = residual; p.N = N; p.K = K; p.ld_out = ld_out; p.ld_res = ld_res; p.flags = flags;
  p.kb_total = kb_total;
  I8Scales sc;
  sc.w_scale = w_scale; sc.w_zero = w_zero; sc.a_scale = a_scale; sc.a_sum = a_sum; sc.ld_a = ld_a; sc.n_rows = N;
  CUtensorMap tmW, tmX;
  int mpad = 16;
  if (counts == nullptr) {
    if (M > 128) return -1;
    while (mpad < M) mpad <<= 1;
    const int n_tiles = (N + 127) / 128;
    if (nsplit <= 0) {
      nsplit = 1;
      const int slots = sm_count * (mpad <= 64 ? 2 : 1);
      while (nsplit < 8 && n_tiles * nsplit * 2 <= slots && kb_total / (nsplit * 2) >= 4) nsplit <<= 1;
    }
    if (!make_tmap_2d(&tmW, Wq, (uint64_t)N, (uint64_t)wbytes, (uint64_t)wbytes, 128, wkind == WK_INT4G ? 64 : 128, 1, wkind == WK_INT4G ? 0 : 3)) return -2;
    if (!make_tmap_2d(&tmX, xq, (uint64_t)M, (uint64_t)K, (uint64_t)ldq, mpad, 128, 1, 3)) return -2;
    p.M = M; p.kb_per_split = (kb_total + nsplit - 1) / nsplit;
    p.idesc = make_idesc_i8(128, mpad);
    return wkind == WK_INT8 ? dispatch_i8<WK_INT8>(mpad, dtype, tmW, tmX, p, sc, nullptr, nsplit, n_tiles, 1, stream)
                            : dispatch_i8<WK_INT4G>(mpad, dtype, tmW, tmX, p, sc, nullptr, nsplit, n_tiles, 1, stream);
  }
  if (N % 128 != 0 || n_local <= 0 || rows_cap <= 0) return -1;
  const int hint = (max_rows >> 16) & 0xFFFF;
  max_rows &= 0xFFFF;
  if (max_rows <= 0) max_rows = rows_cap;
  const int want = hint > 0 ? hint : max_rows;
  while (mpad < want && mpad < 64) mpad <<= 1;
  const int chunks = (max_rows + mpad - 1) / mpad;
  const int n_tiles = N / 128;
  if (!make_tmap_2d(&tmW, Wq, (uint64_t)n_local * N, (uint64_t)wbytes, (uint64_t)wbytes, 128, wkind == WK_INT4G ? 64 : 128, 1, wkind == WK_INT4G ? 0 : 3)) return -2;
  if (!make_tmap_2d(&tmX, xq, (uint64_t)rows_cap, (uint64_t)K, (uint64_t)ldq, mpad, 128, 1, 3)) return -2;
  p.M = mpad; p.kb_per_split = kb_total;
  p.idesc = make_idesc_i8(128, mpad);
  I8GroupInfo gi;
  gi.counts = counts; gi.offsets = offsets; gi.rows_per_chunk = mpad; gi.chunks = chunks; gi.n_rows_w = N;
  gi.n_local = n_local; gi.compact = 0;
  int nz = n_local * chunks;
  if (M > 0) {                        // grouped call: M = upper bound of the routed rows over all local experts
    const int bound = n_local + (M + mpad - 1) / mpad;
    if (bound < nz) { nz = bound; gi.compact = 1; }
  }
  return wkind == WK_INT8 ? dispatch_i8<WK_INT8>(mpad, dtype, tmW, tmX, p, sc, &gi, 1, n_tiles, nz, stream)
                          : dispatch_i8<WK_INT4G>(mpad, dtype, tmW, tmX, p, sc, &gi, 1, n_tiles, nz, stream);
}
