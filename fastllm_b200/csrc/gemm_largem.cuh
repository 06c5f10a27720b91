// Large-M ("prefill") 16-bit GEMM body for sm_100a, shared by the plain kernel and by the kernel that fuses the
// cross-rank reduction behind it.  Included after gemm_smallm.cuh (GemmParams, flags, pack/unpack helpers).
#pragma once
#include "gemm_smallm.cuh"

namespace fb {

// ---------------------------------------------------------------------------------------------------
// large-M kernel: tile 128 tokens x BN out-features, BK = 64
// ---------------------------------------------------------------------------------------------------
template <int BN>
struct LargeMCfg {
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (196 * 1024) / STAGE_BYTES > 8 ? 8 : (196 * 1024) / STAGE_BYTES;
  static constexpr int BODY_BYTES = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BYTES = BODY_BYTES + 256 + 1024;
  static constexpr int TMEM_COLS = 2 * BN;              // two accumulators: epilogue of tile i overlaps the MMAs of tile i + 1
};

// Epilogue of one 128-token x BN-feature tile: TMEM lanes [32q, 32q+32) of accumulator `tmem_acc` -> bias / residual / SwiGLU ->
// 16-bit or fp32 rows in global memory.  A thread owns one token row and writes 64 / 128 contiguous bytes per 32-column step.
template <int BN, bool BF16>
__device__ __forceinline__ void largem_epilogue(const GemmParams& p, uint32_t tmem_acc, int m_tile, int n_tile, int q, int lane) {
    const int m = m_tile * 128 + q * 32 + lane;
    const bool swiglu = (p.flags & GEMM_SWIGLU) != 0;
    const uint16_t* bias16 = reinterpret_cast<const uint16_t*>(p.bias);
    if (!swiglu) {
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        __syncwarp();
        tmem_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
        const int n0 = n_tile * BN + c0;
        if (m >= p.M || n0 >= p.N) continue;
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (p.flags & GEMM_BIAS) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float2 b = unpack_16<BF16>(*reinterpret_cast<const uint32_t*>(bias16 + n0 + j));
            v[j] += b.x; v[j + 1] += b.y;
          }
        }
        if (p.flags & GEMM_RESIDUAL) {
          const uint4* rp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.residual) + (size_t)m * p.ld_res + n0);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 rv = rp[g];
            float2 a0 = unpack_16<BF16>(rv.x), a1 = unpack_16<BF16>(rv.y), a2 = unpack_16<BF16>(rv.z), a3 = unpack_16<BF16>(rv.w);
            v[g * 8 + 0] += a0.x; v[g * 8 + 1] += a0.y; v[g * 8 + 2] += a1.x; v[g * 8 + 3] += a1.y;
            v[g * 8 + 4] += a2.x; v[g * 8 + 5] += a2.y; v[g * 8 + 6] += a3.x; v[g * 8 + 7] += a3.y;
          }
        }
        if (p.flags & GEMM_OUT_F32) {
          float4* op = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)m * p.ld_out + n0);
#pragma unroll
          for (int g = 0; g < 8; ++g) op[g] = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
        } else {
          uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + (size_t)m * p.ld_out + n0);
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_16<BF16>(v[g * 8 + 0], v[g * 8 + 1]); o.y = pack_16<BF16>(v[g * 8 + 2], v[g * 8 + 3]);
            o.z = pack_16<BF16>(v[g * 8 + 4], v[g * 8 + 5]); o.w = pack_16<BF16>(v[g * 8 + 6], v[g * 8 + 7]);
            op[g] = o;
          }
        }
      }
    } else {
      // gate columns [128b, 128b+64), up columns [128b+64, 128b+128) of this tile -> out columns 64*(tile) + ...
#pragma unroll 1
      for (int blk = 0; blk < BN / 128; ++blk) {
#pragma unroll 1
        for (int c0 = 0; c0 < 64; c0 += 32) {
          uint32_t g[32], u[32];
          __syncwarp();
          tmem_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(blk * 128 + c0), g);
          tmem_ld_32x32b_x32(tmem_acc + ((uint32_t)(q * 32) << 16) + (uint32_t)(blk * 128 + 64 + c0), u);
          tmem_ld_wait();
          const int nin = n_tile * BN + blk * 128 + c0;            // gate row index in W
          const int nout = (n_tile * BN + blk * 128) / 2 + c0;
          if (m >= p.M || nout >= (p.N >> 1)) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float gv = __uint_as_float(g[j]), uv = __uint_as_float(u[j]);
            if (p.flags & GEMM_BIAS) {
              gv += BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias16)[nin + j])
                         : __half2float(reinterpret_cast<const __half*>(bias16)[nin + j]);
              uv += BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(bias16)[nin + 64 + j])
                         : __half2float(reinterpret_cast<const __half*>(bias16)[nin + 64 + j]);
            }
            v[j] = silu_f(gv) * uv;
          }
          uint4* op = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + (size_t)m * p.ld_out + nout);
#pragma unroll
          for (int gq = 0; gq < 4; ++gq) {
            uint4 o;
            o.x = pack_16<BF16>(v[gq * 8 + 0], v[gq * 8 + 1]); o.y = pack_16<BF16>(v[gq * 8 + 2], v[gq * 8 + 3]);
            o.z = pack_16<BF16>(v[gq * 8 + 4], v[gq * 8 + 5]); o.w = pack_16<BF16>(v[gq * 8 + 6], v[gq * 8 + 7]);
            op[gq] = o;
          }
        }
      }
    }
}


// Hook of the plain kernel: weight-tile-major order (m fastest: the CTAs of a wave share a few weight tiles through L2),
// nothing to do after a tile, no extra warps.
struct LargeMPlainHook {
  __device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& m_tile, int& n_tile) const {
    n_tile = t / tiles_m; m_tile = t - n_tile * tiles_m;
  }
  __device__ __forceinline__ void tile_done(int m_tile, int n_tile, int lane) const {}
  __device__ __forceinline__ void extra_warps(int warp, int lane) const {}
};

// Persistent, warp-specialised large-M kernel body.  One CTA per SM walks the output tiles in the hook's order; warp 0 streams
// operand tiles by TMA through a ring that keeps running across tile boundaries, warp 1 issues the UMMAs, warps 2..5 run the
// epilogue; warps 6.. (if the launch has them) run hook.extra_warps.  TMEM holds two accumulators: while the epilogue warps
// drain tile i the tensor core already accumulates tile i + 1, so the tensor pipe does not idle during epilogues and the
// per-tile prologue (TMEM allocation, barrier set-up, pipeline fill) is paid once per CTA instead of once per tile.
// hook.tile_done(m_tile, n_tile, lane) runs in every epilogue warp after that warp's rows of the tile are stored.
template <int BN, bool BF16, class Hook>
__device__ __forceinline__ void gemm_largem_device(const CUtensorMap& tmX, const CUtensorMap& tmW, const GemmParams& p,
                                                   int tiles_m, int tiles_n, const Hook& hook) {
  using Cfg = LargeMCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BODY_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* acc_full = empty_bar + Cfg::STAGES;        // [2] accumulator ready for the epilogue
  uint64_t* acc_empty = acc_full + 2;                  // [2] accumulator drained (4 epilogue warps arrive)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_cnt = p.kb_total;
  const int tiles = tiles_m * tiles_n;
  bool dead = false;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
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
      int it = 0;                                          // k-block counter across all of this CTA's tiles
      for (int t = blockIdx.x; t < tiles; t += gridDim.x) {
        int m_tile, n_tile;
        hook.tile_coords(t, tiles_m, tiles_n, m_tile, n_tile);
        for (int i = 0; i < kb_cnt; ++i, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
          if (!mbar_wait(&empty_bar[s], ph ^ 1u, dead, KID_GEMM_LARGEM, 1)) break;
          uint8_t* a = smem + s * Cfg::STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
          tma_load_2d(a, &tmX, &full_bar[s], i * 64, m_tile * 128);
          tma_load_2d(a + Cfg::A_BYTES, &tmW, &full_bar[s], i * 64, n_tile * BN);
        }
        if (dead) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      int it = 0, u = 0;                                   // u: tiles done by this CTA
      for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++u) {
        const int buf = u & 1;
        const uint32_t use = (uint32_t)(u >> 1) & 1u;      // how often this buffer has been used, parity
        if (!mbar_wait(&acc_empty[buf], use ^ 1u, dead, KID_GEMM_LARGEM, 4)) break;     // first use passes at once
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + (uint32_t)(buf * BN);
        for (int i = 0; i < kb_cnt; ++i, ++it) {
          const int s = it % Cfg::STAGES;
          const uint32_t ph = (uint32_t)(it / Cfg::STAGES) & 1u;
          if (!mbar_wait(&full_bar[s], ph, dead, KID_GEMM_LARGEM, 2)) break;
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
          const uint64_t da = make_smem_desc(a_addr, 16, 1024, SWZ_128B);
          const uint64_t db = make_smem_desc(a_addr + Cfg::A_BYTES, 16, 1024, SWZ_128B);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(acc, da + 2 * k, db + 2 * k, p.idesc, (i | k) != 0 ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        if (dead) break;
        umma_commit(&acc_full[buf]);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    const int q = warp & 3;
    int u = 0;
    for (int t = blockIdx.x; t < tiles; t += gridDim.x, ++u) {
      int m_tile, n_tile;
      hook.tile_coords(t, tiles_m, tiles_n, m_tile, n_tile);
      const int buf = u & 1;
      const uint32_t use = (uint32_t)(u >> 1) & 1u;
      if (!mbar_wait(&acc_full[buf], use, dead, KID_GEMM_LARGEM, 3)) break;
      tc_fence_after_sync();
      largem_epilogue<BN, BF16>(p, tmem_base + (uint32_t)(buf * BN), m_tile, n_tile, q, lane);
      tc_fence_before_sync();                              // this warp's TMEM reads are done before the buffer is handed back
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      hook.tile_done(m_tile, n_tile, lane);
    }
  } else {
    hook.extra_warps(warp, lane);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

}  // namespace fb
