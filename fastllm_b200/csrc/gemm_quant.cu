// Weight-only-quantised small-M GEMM for sm_100a:  Y[M,N] = X[M,K] * dequant(Wq)[N,K]^T  (+ bias, residual, SwiGLU)
//
// Formats (reference numerics, include/fastllm.h:239-306):
//   int8   per-output-channel asymmetric      w = scale[n] * (q - zero[n])
//   int4g  group-wise asymmetric, 2 per byte, first value in the HIGH nibble      w = min[n,g] + scale[n,g] * q
//   fp8    FP8-E4M3 with one fp32 scale per 128x128 block                          w = scale[n/128,k/128] * q
//   fp4    e2m1, 2 per byte, first value in the LOW nibble, one bf16 scale per 16 (NVFP4: e4m3-valued scales and a
//          per-tensor fp32 factor) or 32 (MXFP4: power-of-two scales) k elements    w = global * scale[n,k/g] * q
// The reference serves these with CUDA-core GEMV kernels for small batches and dequant-to-fp16 + cublasGemmEx
// otherwise (src/devices/cuda/linear/fastllm-linear-int8.cu, -int4group.cu:1919-2054, -fp8.cu:1778-1868).
//
// Here: same swap-AB tcgen05 kernel as the dense decode GEMM, with a dequant stage between TMA and MMA.
//   warp 0     TMA: packed weight tile [128 n x 64 k] (4 KB int4 / 8 KB int8,fp8) + activation tile -> raw ring
//   warps 2-5  dequant: raw -> 16-bit in the 128-byte-swizzled K-major layout UMMA reads (int -> fp16 through the
//              0x6400 "1024 + q" bit trick, FP8 through cvt.f16x2.e4m3x2), group scale/min applied here,
//              per-channel int8 scale applied in the epilogue (q - zero is exact in fp16)
//   warp 1     UMMA: A = de-quantised weights in the activations' 16-bit type, B = activations, fp32 accumulate
//   then the shared cluster split-K reduce + epilogue (gemm_smallm.cuh)
// Weight bytes cross HBM once, in packed form: the kernel is bound by 0.5 / 1 byte per weight.
#include "gemm_smallm.cuh"
#include "launch.h"
#include "tmap.h"

FB_DEFINE_ERROR_API(gemm_quant)

namespace fb {

constexpr int KID_GEMM_QUANT = 3;
enum QMode : int { Q_INT8 = 1, Q_INT4G = 2, Q_FP8 = 3, Q_FP4 = 4 };

struct QuantParams {
  const float* scale;     // int8: [N]; fp8: [ceil(N/128), kb128]; int4g: float2 (scale, min) [groups, N]; fp4: bf16 [N, groups]
  const float* zero;      // int8: [N]; fp4: one per-tensor factor (null: 1)
  int group_k;            // int4g: k elements per group (multiple of 64); fp8: 128; fp4: 16 or 32
  int groups;             // int4g: groups per row; fp8: scale columns
  uint32_t xor_mask;      // int8: 0x80808080 when the bytes are stored as q - 128 (operand form of the integer path), else 0;
                          // fp4: 1 when the scale table lies within fp16's range (fp16 activations: half2 de-quantiser)
};

// OCC: CTAs per SM the shared-memory budget is sized for (2 doubles the dequant warps working per SM)
template <int MPAD, int QM, int OCC = (MPAD <= 64 ? 2 : 1)>
struct QuantCfg {
  static constexpr int RAW_BYTES = (QM == Q_INT4G || QM == Q_FP4) ? 128 * 32 : 128 * 64;
  static constexpr int B_BYTES = MPAD * 128;
  static constexpr int STAGE_BYTES = RAW_BYTES + B_BYTES;            // bytes TMA delivers per stage
  static constexpr int PITCH = (STAGE_BYTES + 1023) / 1024 * 1024;   // stage pitch: keeps the swizzled activation tile 1024-aligned
  static constexpr int DQ_SLOTS = 3;
  static constexpr int DQ_BYTES = 128 * 128;
  static constexpr int RED_BYTES = MPAD * 128 * 4;
  static constexpr int BUDGET = (196 * 1024) / OCC - DQ_SLOTS * DQ_BYTES;
  static constexpr int STAGES_RAW = BUDGET / PITCH > 12 ? 12 : BUDGET / PITCH;
  static constexpr int STAGES = STAGES_RAW < 2 ? 2 : STAGES_RAW;
  static constexpr int PIPE_BYTES = DQ_SLOTS * DQ_BYTES + STAGES * PITCH;
  static constexpr int BODY_BYTES = PIPE_BYTES > RED_BYTES ? PIPE_BYTES : RED_BYTES;
  static constexpr int SMEM_BYTES = BODY_BYTES + 512 + 1024;
  static constexpr int TMEM_COLS = MPAD < 32 ? 32 : MPAD;
  // dequant warps: four per CTA with two CTAs per SM; eight when the tile leaves room for one CTA only (the conversion is
  // a dependent load - convert - store chain per thread, so its rate follows the number of warps in flight)
  static constexpr int DQ_WARPS = (MPAD <= 64 && QM != Q_FP4) ? 4 : 8;      // fp4: the longest conversion chain per value
  static constexpr int DQ_THREADS = DQ_WARPS * 32;
  static constexpr int THREADS = 64 + DQ_THREADS;
};

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
// weights are produced in the activations' own 16-bit type (both UMMA operands share one format)
template <bool BF16>
__device__ __forceinline__ uint32_t out16(__half2 h) {
  if (!BF16) return h2_as_u32(h);
  const float2 f = __half22float2(h);
  return pack_bf16(f.x, f.y);
}

// two unsigned bytes (values < 1024) -> half2 (lo, hi) exactly, via the 0x6400 | v == 1024 + v representation
__device__ __forceinline__ __half2 u8x2_to_h2(uint32_t lo, uint32_t hi, __half2 sub) {
  const uint32_t bits = 0x64006400u | lo | (hi << 16);
  return __hsub2(*reinterpret_cast<const __half2*>(&bits), sub);
}

template <int MPAD, bool BF16, int QM>
__device__ __forceinline__ void gemm_quant_device(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p,
                                                  const QuantParams& qp) {
  using Cfg = QuantCfg<MPAD, QM>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* dq = smem;                                            // DQ_SLOTS x 16 KB, 1024-aligned
  uint8_t* stages = smem + Cfg::DQ_SLOTS * Cfg::DQ_BYTES;        // per stage: activation tile first (1024-aligned), raw weights after
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::BODY_BYTES);
  uint64_t* full_bar = bars;                       // [STAGES]   TMA landed (raw + X)
  uint64_t* empty_bar = full_bar + Cfg::STAGES;    // [STAGES]   1 UMMA commit + 128 dequant arrivals
  uint64_t* dq_full = empty_bar + Cfg::STAGES;     // [DQ_SLOTS] 128 dequant arrivals
  uint64_t* dq_empty = dq_full + Cfg::DQ_SLOTS;    // [DQ_SLOTS] UMMA commit
  uint64_t* accum_bar = dq_empty + Cfg::DQ_SLOTS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
  constexpr int PITCH = Cfg::PITCH;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = (int)cluster_ctarank();
  const int nsplit = (int)cluster_nctarank();
  const int n_tile = blockIdx.y;
  const int kb0 = split * p.kb_per_split;
  int kb_cnt = p.kb_total - kb0;
  if (kb_cnt > p.kb_per_split) kb_cnt = p.kb_per_split;
  if (kb_cnt < 0) kb_cnt = 0;
  bool dead = false;
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], Cfg::DQ_THREADS + 1); }
    for (int s = 0; s < Cfg::DQ_SLOTS; ++s) { mbar_init(&dq_full[s], Cfg::DQ_THREADS); mbar_init(&dq_empty[s], 1); }
    mbar_init(accum_bar, 1);
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
      constexpr int KBYTES = (QM == Q_INT4G || QM == Q_FP4) ? 32 : 64;            // packed bytes per 64-wide k block
      // packed weights are independent of the kernel before this one: request the first ring before the dependency wait
      const int pre = kb_cnt < Cfg::STAGES ? kb_cnt : Cfg::STAGES;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], Cfg::STAGE_BYTES);
        tma_load_2d_hint(stages + i * PITCH + Cfg::B_BYTES, &tmW, &full_bar[i], (kb0 + i) * KBYTES, p.w_row0 + n_tile * 128, pol_w);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) tma_load_2d_hint(stages + i * PITCH, &tmX, &full_bar[i], (kb0 + i) * 64, p.x_row0, pol_x);
      for (int i = pre; i < kb_cnt; ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, dead, KID_GEMM_QUANT, 1)) break;
        uint8_t* xb = stages + s * PITCH;
        mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
        tma_load_2d_hint(xb, &tmX, &full_bar[s], (kb0 + i) * 64, p.x_row0, pol_x);
        tma_load_2d_hint(xb + Cfg::B_BYTES, &tmW, &full_bar[s], (kb0 + i) * KBYTES, p.w_row0 + n_tile * 128, pol_w);
      }
    }
    __syncwarp();
    pdl_wait();
  } else if (warp == 1) {
    if (elect_one()) {
      for (int i = 0; i < kb_cnt; ++i) {
        const int s = i % Cfg::STAGES, t = i % Cfg::DQ_SLOTS;
        const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u, tph = (uint32_t)(i / Cfg::DQ_SLOTS) & 1u;
        if (!mbar_wait(&full_bar[s], ph, dead, KID_GEMM_QUANT, 6)) break;
        if (!mbar_wait(&dq_full[t], tph, dead, KID_GEMM_QUANT, 2)) break;
        tc_fence_after_sync();
        const uint64_t da = make_smem_desc(smem_u32(dq + t * Cfg::DQ_BYTES), 16, 1024, SWZ_128B);
        const uint64_t db = make_smem_desc(smem_u32(stages + s * PITCH), 16, 1024, SWZ_128B);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(tmem_base, da + 2 * k, db + 2 * k, p.idesc, (i | k) != 0 ? 1u : 0u);
        umma_commit(&empty_bar[s]);
        umma_commit(&dq_empty[t]);
      }
      umma_commit(accum_bar);
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    const int tid = threadIdx.x - 64;                 // 0..DQ_THREADS-1
    constexpr int DQT = Cfg::DQ_THREADS;
    // ------------------------------ dequant stage ------------------------------
    // fp4: the block scales of a k block come from global memory; they are requested one k block ahead, so that their
    // latency is not part of the chain barrier -> convert -> store
    constexpr int FP4_UNITS = QM == Q_FP4 ? 256 / DQT : 1;
    uint32_t fp4_s[FP4_UNITS];
    auto fp4_fetch = [&](int kb) {
#pragma unroll
      for (int it = 0; it < FP4_UNITS; ++it) {
        const int u = tid + DQT * it, row = u >> 1, ch = u & 1;
        const int n = n_tile * 128 + row;
        fp4_s[it] = 0u;
        if (n < p.N) {
          const uint16_t* sp = reinterpret_cast<const uint16_t*>(qp.scale) + (size_t)n * qp.groups + (kb * 64 + ch * 32) / qp.group_k;
          fp4_s[it] = qp.group_k == 16 ? *reinterpret_cast<const uint32_t*>(sp) : (uint32_t)sp[0] * 0x10001u;
        }
      }
    };
    if (QM == Q_FP4 && kb_cnt > 0) fp4_fetch(kb0);
    for (int i = 0; i < kb_cnt; ++i) {
      const int s = i % Cfg::STAGES, t = i % Cfg::DQ_SLOTS;
      const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u, tph = (uint32_t)(i / Cfg::DQ_SLOTS) & 1u;
      mbar_wait(&full_bar[s], ph, dead, KID_GEMM_QUANT, 4);
      mbar_wait(&dq_empty[t], tph ^ 1u, dead, KID_GEMM_QUANT, 5);
      const uint8_t* raw = stages + s * PITCH + Cfg::B_BYTES;
      uint8_t* out = dq + t * Cfg::DQ_BYTES;
      const int kb = kb0 + i;
      if (QM == Q_INT4G) {
        const int g = (kb * 64) / qp.group_k;
#pragma unroll
        for (int it = 0; it < 256 / DQT; ++it) {
          const int u = tid + DQT * it, row = u >> 1, ch = u & 1;
          const int n = n_tile * 128 + row;
          float2 sm = make_float2(0.f, 0.f);
          if (n < p.N) sm = reinterpret_cast<const float2*>(qp.scale)[(size_t)g * p.N + n];
          const __half2 sc = __float2half2_rn(sm.x), mn = __float2half2_rn(sm.y);
          const __half2 k1024 = __float2half2_rn(1024.f);
          const uint4 w = *reinterpret_cast<const uint4*>(raw + row * 32 + ch * 16);
          const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {            // one 32-bit word = 8 values = one 16-byte chunk of fp16
            const uint32_t x = ws[j];
            uint32_t o[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
              const uint32_t byte = (x >> (8 * b)) & 0xFFu;
              const __half2 v = u8x2_to_h2(byte >> 4, byte & 0xFu, k1024);      // first value = high nibble
              o[b] = out16<BF16>(__hfma2(v, sc, mn));
            }
            const int chunk = ch * 4 + j;
            *reinterpret_cast<uint4*>(out + row * 128 + ((chunk ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      } else if (QM == Q_FP4) {
#pragma unroll
        for (int it = 0; it < 256 / DQT; ++it) {
          const int u = tid + DQT * it, row = u >> 1, ch = u & 1;           // 32 k values = 16 packed bytes per unit
          // scales of the unit's two 16-value halves (two bf16 values in one word)
          const float s0 = __uint_as_float(fp4_s[it] << 16), s1 = __uint_as_float(fp4_s[it] & 0xFFFF0000u);
          const uint4 w = *reinterpret_cast<const uint4*>(raw + row * 32 + ch * 16);
          const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {            // one 32-bit word = 8 values = one 16-byte chunk of 16-bit operands
            uint32_t h[4];
            asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
                "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
                "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}\n"
                : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(ws[j]));
            const float sc = j < 2 ? s0 : s1;
            uint32_t o[4];
            if (!BF16 && qp.xor_mask != 0u) {
              // fp16 activations: the product e2m1 x scale is exact in fp16 while the scale table stays inside fp16's range,
              // which the host has checked -- one multiply per value pair.  (Both operands of one MMA must have the same 16-bit
              // format: an fp16 weight operand beside bf16 activations raises an illegal-instruction error.)
              const __half2 sc2 = __float2half2_rn(sc);
#pragma unroll
              for (int b = 0; b < 4; ++b) o[b] = h2_as_u32(__hmul2(*reinterpret_cast<const __half2*>(&h[b]), sc2));
            } else {
#pragma unroll
              for (int b = 0; b < 4; ++b) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[b]));
                o[b] = BF16 ? pack_bf16(f.x * sc, f.y * sc) : h2_as_u32(__floats2half2_rn(f.x * sc, f.y * sc));
              }
            }
            const int chunk = ch * 4 + j;
            *reinterpret_cast<uint4*>(out + row * 128 + ((chunk ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        if (i + 1 < kb_cnt) fp4_fetch(kb + 1);
      } else {
        float bscale = 1.f;
        if (QM == Q_FP8) bscale = qp.scale[(size_t)n_tile * qp.groups + (kb * 64) / 128];
        const __half2 bs2 = __float2half2_rn(bscale);
        uint4 wv[512 / DQT];
#pragma unroll
        for (int it = 0; it < 512 / DQT; ++it) {
          const int u = tid + DQT * it;
          wv[it] = *reinterpret_cast<const uint4*>(raw + (u >> 2) * 64 + (u & 3) * 16);
        }
#pragma unroll
        for (int it = 0; it < 512 / DQT; ++it) {
          const int u = tid + DQT * it, row = u >> 2, ch = u & 3;
          const int n = n_tile * 128 + row;
          const uint32_t ws[4] = {wv[it].x, wv[it].y, wv[it].z, wv[it].w};
          uint32_t o[8];
          if (QM == Q_INT8) {
            const float z = n < p.N ? qp.zero[n] : 0.f;
            const __half2 sub = __float2half2_rn(1024.f + z);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t w = ws[j] ^ qp.xor_mask;
              o[2 * j] = out16<BF16>(u8x2_to_h2(w & 0xFFu, (w >> 8) & 0xFFu, sub));
              o[2 * j + 1] = out16<BF16>(u8x2_to_h2((w >> 16) & 0xFFu, w >> 24, sub));
            }
          } else if (BF16) {
            // e4m3 -> bf16 by bit placement: sign to bit 15, the 7 exponent+mantissa bits to bits 10..4; the value comes out
            // scaled by 2^-120 (exponent bias 7 vs 127), exact also for subnormals; one fp32 multiply applies 2^120 * block scale
            const float fs = bscale * 1.329227995784916e36f;     // 2^120
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t x = ws[j];
#pragma unroll
              for (int hw = 0; hw < 2; ++hw) {
                const uint32_t b0 = (x >> (16 * hw)) & 0xFFu, b1 = (x >> (16 * hw + 8)) & 0xFFu;
                const float f0 = __uint_as_float((((b0 & 0x80u) << 8) | ((b0 & 0x7Fu) << 4)) << 16) * fs;
                const float f1 = __uint_as_float((((b1 & 0x80u) << 8) | ((b1 & 0x7Fu) << 4)) << 16) * fs;
                o[2 * j + hw] = pack_bf16(f0, f1);
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t lo, hi;
              asm("{\n\t.reg .b16 a, b;\n\tmov.b32 {a, b}, %2;\n\tcvt.rn.f16x2.e4m3x2 %0, a;\n\tcvt.rn.f16x2.e4m3x2 %1, b;\n\t}\n"
                  : "=r"(lo), "=r"(hi) : "r"(ws[j]));
              o[2 * j] = h2_as_u32(__hmul2(*reinterpret_cast<__half2*>(&lo), bs2));
              o[2 * j + 1] = h2_as_u32(__hmul2(*reinterpret_cast<__half2*>(&hi), bs2));
            }
          }
          const int c0 = ch * 2;
          *reinterpret_cast<uint4*>(out + row * 128 + ((c0 ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(out + row * 128 + (((c0 + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&dq_full[t]);
      mbar_arrive(&empty_bar[s]);
    }
    // ------------------------------ epilogue: TMEM -> fp32 partial tile ------------------------------
    pdl_wait();
    float* P = reinterpret_cast<float*>(smem);
    const int n_local = q * 32 + lane;
    float row_scale = 1.f;
    if (QM == Q_INT8) { const int n = n_tile * 128 + n_local; row_scale = n < p.N ? qp.scale[n] : 0.f; }
    if (QM == Q_FP4 && qp.zero != nullptr) row_scale = qp.zero[0];
    if (warp >= 6) {
      // extra dequant warps: no TMEM lane quarter of their own
    } else if (kb_cnt > 0) {
      mbar_wait(accum_bar, 0, dead, KID_GEMM_QUANT, 3);
      tc_fence_after_sync();
      constexpr int CH = MPAD < 32 ? MPAD : 32;
#pragma unroll 1
      for (int c0 = 0; c0 < MPAD; c0 += CH) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        if (CH == 32) tmem_ld_32x32b_x32(taddr, r); else tmem_ld_32x32b_x16(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < CH; ++j) P[(c0 + j) * 128 + n_local] = __uint_as_float(r[j]) * row_scale;
      }
    } else {
      for (int j = 0; j < MPAD; ++j) P[j * 128 + n_local] = 0.f;
    }
  }
  tc_fence_before_sync();
  cluster_sync_all();
  smallm_reduce_store<BF16>(p, smem, split, nsplit, n_tile);
  cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}

template <int MPAD, bool BF16, int QM>
__global__ void __launch_bounds__((QuantCfg<MPAD, QM>::THREADS), (MPAD <= 64 ? 2 : 1))
gemm_quant_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams p,
                  const QuantParams qp) {
  gemm_quant_device<MPAD, BF16, QM>(tmW, tmX, p, qp);
}

// Grouped (mixture-of-experts) variant: blockIdx.z = expert * chunks + chunk; weights / scales are stacked per expert.
struct QuantGroupInfo {
  const int* counts; const int* offsets;
  int rows_per_chunk, chunks, n_rows_w;
  long long scale_stride_e, zero_stride_e;      // floats per expert
  int n_local, compact;                         // compact: grid.z enumerates existing (expert, chunk) pairs (moe_find_item)
};

template <int MPAD, bool BF16, int QM>
__global__ void __launch_bounds__((QuantCfg<MPAD, QM>::THREADS), (MPAD <= 64 ? 2 : 1))
moe_grouped_quant_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams base,
                         const QuantParams qbase, const QuantGroupInfo gi) {
  int e = blockIdx.z / gi.chunks, chunk = blockIdx.z - e * gi.chunks;
  pdl_launch_dependents();
  pdl_wait();   // counts / offsets come from the plan kernel
  if (gi.compact && !moe_find_item(gi.counts, gi.n_local, gi.rows_per_chunk, (int)blockIdx.z, e, chunk)) return;
  const int cnt = gi.counts[e];
  const int row0 = chunk * gi.rows_per_chunk;
  if (row0 >= cnt) return;
  GemmParams p = base;
  const int seg = gi.offsets[e] + row0;
  p.M = cnt - row0 < gi.rows_per_chunk ? cnt - row0 : gi.rows_per_chunk;
  p.x_row0 = seg;
  p.w_row0 = e * gi.n_rows_w;
  p.out = reinterpret_cast<uint16_t*>(base.out) + (size_t)seg * base.ld_out;
  QuantParams qp = qbase;
  qp.scale = qbase.scale + (size_t)e * gi.scale_stride_e;
  if (qbase.zero != nullptr) qp.zero = qbase.zero + (size_t)e * gi.zero_stride_e;
  gemm_quant_device<MPAD, BF16, QM>(tmW, tmX, p, qp);
}

}  // namespace fb

using namespace fb;

extern "C" int fb_gemm_pick_split(int M, int N, int K, int slots);

template <int MPAD, bool BF16, int QM>
static cudaError_t launch_quant(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const QuantParams& qp,
                                int nsplit, int n_tiles, cudaStream_t stream) {
  using Cfg = QuantCfg<MPAD, QM>;
  auto kern = gemm_quant_kernel<MPAD, BF16, QM>;
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
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, qp);
}

// qmode: 1 = int8 (Wq uint8 [N,K], scale [N], zero [N]), 2 = int4g (Wq uint8 [N,K/2], scale = float2 (scale,min) [groups,N]),
// 3 = fp8 block 128 (Wq e4m3 [N,K], scale [ceil(N/128), ceil(K/128)]), 4 = fp4 (Wq uint8 [N,K/2], scale = bf16 [N, K/group_k],
// group_k 16 or 32, zero = one per-tensor factor or null).  X dtype: 0 = fp16, 1 = bf16.  M <= 256.
// int8 with group_k < 0: the bytes hold q - 128 (two's complement), zero still refers to q.
extern "C" int fb_gemm_quant(const void* X, const void* Wq, const float* scale, const float* zero, void* out, const void* bias,
                             const void* residual, int M, int N, int K, int ldx, int ld_out, int ld_res, int dtype, int qmode,
                             int group_k, int flags, int nsplit, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (M > 256 || K % 64 != 0 || N % 8 != 0 || (dtype != 0 && dtype != 1)) return -1;
  if (qmode == Q_INT4G && (group_k <= 0 || group_k % 64 != 0 || K % group_k != 0)) return -1;
  if (qmode == Q_FP8 && K % 128 != 0) return -1;
  if (qmode == Q_FP4 && group_k != 16 && group_k != 32) return -1;
  if ((flags & GEMM_SWIGLU) && (N % 128 != 0)) return -1;
  GemmParams p;
  p.out = out; p.bias = bias; p.residual = residual;
  p.M = M; p.N = N; p.K = K; p.ld_out = ld_out; p.ld_res = ld_res;
  p.kb_total = K / 64; p.flags = flags;
  p.scatter_tp = 0; p.scatter_rows = 1; p.scatter_rank = 0; p.w_row0 = 0; p.x_row0 = 0;
  for (int i = 0; i < 8; ++i) p.scatter_out[i] = nullptr;
  QuantParams qp;
  qp.scale = scale; qp.zero = zero;
  qp.group_k = (qmode == Q_INT4G || qmode == Q_FP4) ? group_k : 128;
  qp.groups = (qmode == Q_INT4G || qmode == Q_FP4) ? K / group_k : (K + 127) / 128;
  qp.xor_mask = (qmode == Q_INT8 && group_k < 0) ? 0x80808080u : 0u;      // int8 with group_k < 0: bytes hold q - 128
  const bool bf16 = dtype == 1;
  if (qmode == Q_FP4 && (flags & GEMM_FP4_F16W) != 0 && !bf16) qp.xor_mask = 1u;
  const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  if (nsplit <= 0) nsplit = fb_gemm_pick_split(M, N, K, sm_count);
  if (nsplit != 1 && nsplit != 2 && nsplit != 4 && nsplit != 8) return -1;
  p.kb_per_split = (p.kb_total + nsplit - 1) / nsplit;
  if (qmode == Q_INT4G) {
    // a cluster rank must start on a group boundary only in the sense that a k block never straddles groups: group_k % 64 == 0
  }
  p.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, mpad);
  const bool nib = qmode == Q_INT4G || qmode == Q_FP4;
  const int kbytes = nib ? K / 2 : K;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, Wq, N, kbytes, kbytes, 128, nib ? 32 : 64, 1, 0)) return -2;
  if (!make_tmap_2d(&tmX, X, M, K, ldx, mpad, 64, 2, 3)) return -2;
  const int n_tiles = (N + 127) / 128;
#define FB_Q2(MP, QMV)                                                                                   \
  return (int)(bf16 ? launch_quant<MP, true, QMV>(tmW, tmX, p, qp, nsplit, n_tiles, stream)               \
                    : launch_quant<MP, false, QMV>(tmW, tmX, p, qp, nsplit, n_tiles, stream));
#define FB_Q(MP)                                                                                          \
  { if (qmode == Q_INT8) { FB_Q2(MP, Q_INT8) } else if (qmode == Q_INT4G) { FB_Q2(MP, Q_INT4G) } else if (qmode == Q_FP8) { FB_Q2(MP, Q_FP8) } else if (qmode == Q_FP4) { FB_Q2(MP, Q_FP4) } else return -1; }
  switch (mpad) {
    case 16: FB_Q(16)
    case 32: FB_Q(32)
    case 64: FB_Q(64)
    case 128: FB_Q(128)
    default: FB_Q(256)
  }
#undef FB_Q
#undef FB_Q2
}

template <int MPAD, bool BF16, int QM>
static cudaError_t launch_grouped_quant(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const QuantParams& qp,
                                        const QuantGroupInfo& gi, int nsplit, int n_tiles, int nz, cudaStream_t stream) {
  using Cfg = QuantCfg<MPAD, QM>;
  auto kern = moe_grouped_quant_kernel<MPAD, BF16, QM>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, n_tiles, nz);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nsplit; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = add_pdl_attr(attr, 1);
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, qp, gi);
}

// Grouped quantised expert GEMM over the expert-sorted buffer; stacked Wq [E_local * N, K bytes], stacked scales.
extern "C" int fb_moe_grouped_gemm_quant(const void* Xs, const void* Wq, const float* scale, const float* zero, void* out,
                                         const int* counts, const int* offsets, int rows_cap, int E_local, int N, int K, int ld_out,
                                         int max_rows_per_expert, int dtype, int qmode, int group_k, int flags, int total_rows,
                                         void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (E_local <= 0 || rows_cap <= 0) return 0;
  if (K % 64 != 0 || N % 128 != 0 || (dtype != 0 && dtype != 1)) return -1;
  if (qmode == Q_INT4G && (group_k <= 0 || group_k % 64 != 0 || K % group_k != 0)) return -1;
  if (qmode == Q_FP8 && K % 128 != 0) return -1;
  if (qmode == Q_FP4 && ((group_k != 16 && group_k != 32) || ((long long)N * (K / group_k)) % 2 != 0)) return -1;
  const bool bf16 = dtype == 1;
  const int hint = max_rows_per_expert >> 16;       // high 16 bits: chunk size hint, low 16 bits: most rows an expert can get
  max_rows_per_expert &= 0xFFFF;
  int mpad = max_rows_per_expert <= 16 ? 16 : max_rows_per_expert <= 32 ? 32 : max_rows_per_expert <= 64 ? 64 : 128;
  if (hint == 16 || hint == 32 || hint == 64 || hint == 128) mpad = hint < mpad ? hint : mpad;
  const int chunks = (max_rows_per_expert + mpad - 1) / mpad;
  GemmParams p;
  p.out = out; p.bias = nullptr; p.residual = nullptr;
  p.M = 0; p.N = N; p.K = K; p.ld_out = ld_out; p.ld_res = 0;
  p.kb_total = K / 64; p.flags = flags;
  p.scatter_tp = 0; p.scatter_rows = 1; p.scatter_rank = 0; p.w_row0 = 0; p.x_row0 = 0;
  for (int i = 0; i < 8; ++i) p.scatter_out[i] = nullptr;
  const int n_tiles = N / 128;
  int nsplit = 1;
  while (nsplit < 4 && n_tiles * E_local * nsplit < 148 && (p.kb_total / (nsplit * 2)) >= 8) nsplit *= 2;
  p.kb_per_split = (p.kb_total + nsplit - 1) / nsplit;
  p.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, mpad);
  QuantParams qp;
  qp.scale = scale; qp.zero = zero;
  qp.group_k = (qmode == Q_INT4G || qmode == Q_FP4) ? group_k : 128;
  qp.groups = (qmode == Q_INT4G || qmode == Q_FP4) ? K / group_k : (K + 127) / 128;
  qp.xor_mask = (qmode == Q_INT8 && group_k < 0) ? 0x80808080u : 0u;      // int8 with group_k < 0: bytes hold q - 128
  if (qmode == Q_FP4 && (flags & GEMM_FP4_F16W) != 0 && !bf16) qp.xor_mask = 1u;
  QuantGroupInfo gi;
  gi.counts = counts; gi.offsets = offsets; gi.rows_per_chunk = mpad; gi.chunks = chunks; gi.n_rows_w = N;
  // strides in floats; the fp4 scale table holds bf16 values (two per float), its per-tensor factor is one float per expert
  gi.scale_stride_e = qmode == Q_INT8 ? N : qmode == Q_INT4G ? (long long)qp.groups * N * 2
                    : qmode == Q_FP4 ? (long long)qp.groups * N / 2 : (long long)(N / 128) * qp.groups;
  gi.zero_stride_e = qmode == Q_FP4 ? 1 : N;
  const bool nib = qmode == Q_INT4G || qmode == Q_FP4;
  const int kbytes = nib ? K / 2 : K;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, Wq, (uint64_t)E_local * N, kbytes, kbytes, 128, nib ? 32 : 64, 1, 0)) return -2;
  if (!make_tmap_2d(&tmX, Xs, rows_cap, K, K, mpad, 64, 2, 3)) return -2;
  int nz = E_local * chunks;
  gi.n_local = E_local; gi.compact = 0;
  if (total_rows > 0) {               // upper bound of the routed rows: one grid slot per existing row chunk
    const int bound = E_local + (total_rows + mpad - 1) / mpad;
    if (bound < nz) { nz = bound; gi.compact = 1; }
  }
  if (nz > 65535) return -1;
#define FB_GQ2(MP, QMV)                                                                                          \
  return (int)(bf16 ? launch_grouped_quant<MP, true, QMV>(tmW, tmX, p, qp, gi, nsplit, n_tiles, nz, stream)       \
                    : launch_grouped_quant<MP, false, QMV>(tmW, tmX, p, qp, gi, nsplit, n_tiles, nz, stream));
#define FB_GQ(MP)                                                                                                 \
  { if (qmode == Q_INT8) { FB_GQ2(MP, Q_INT8) } else if (qmode == Q_INT4G) { FB_GQ2(MP, Q_INT4G) } else if (qmode == Q_FP8) { FB_GQ2(MP, Q_FP8) } else if (qmode == Q_FP4) { FB_GQ2(MP, Q_FP4) } else return -1; }
  switch (mpad) {
    case 16: FB_GQ(16)
    case 32: FB_GQ(32)
    case 64: FB_GQ(64)
    default: FB_GQ(128)
  }
#undef FB_GQ
#undef FB_GQ2
}
