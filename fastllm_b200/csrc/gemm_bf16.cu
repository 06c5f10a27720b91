// Dense 16-bit GEMM family for sm_100a:  Y[M,N] = X[M,K] * W[N,K]^T  (+ bias, + residual, SwiGLU)
//
// Role in the framework: every Linear / LinearAdd / LinearSwiglu with fp16 or bf16 weights.  The reference
// runs these as one-CTA-per-output-row GEMV for < 8 tokens and convert + cublasGemmEx otherwise
// (reference: src/devices/cuda/linear/fastllm-linear-fp16.cu:561-650, fastllm-linear-bf16.cu:332-648).
//
// Two kernels, both tcgen05 (UMMA) with fp32 accumulators in TMEM, operands staged by TMA into
// 128-byte-swizzled shared memory through an mbarrier ring:
//
//  * small-M ("decode") kernel: swap-AB.  The weight tile [128 out-features x 64 k] is the UMMA A operand,
//    the token tile [MPAD tokens x 64 k] the B operand, so the 128-row MMA is always full no matter how
//    few tokens there are.  K is split across a thread-block cluster (1/2/4/8 CTAs); the partial tiles
//    are reduced through distributed shared memory in a fixed order (deterministic), each CTA reducing
//    and writing a slice of the tile with the epilogue applied.  No global scratch.
//  * large-M ("prefill") kernel: 128 tokens x 256 out-features tile per CTA, K pipelined, epilogue straight
//    from TMEM to global.
//
// SwiGLU epilogue expects the gate/up weight rows interleaved per 128-row tile: rows [0,64) of tile t are
// gate rows 64t..64t+63 and rows [64,128) are the matching up rows; output column = 64t + i.
#include "ptx.cuh"
#include "launch.h"
#include "tmap.h"

FB_DEFINE_ERROR_API(gemm)

#include "gemm_smallm.cuh"
#include "gemm_largem.cuh"

namespace fb {

template <int MPAD, bool BF16, int OCC>
__global__ void __launch_bounds__(192, OCC)
gemm_smallm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams p) {
  uint32_t tmem_base;
  gemm_smallm_device<MPAD, BF16, OCC>(tmW, tmX, p, tmem_base, KID_GEMM_SMALLM_PLAIN);
  if ((threadIdx.x >> 5) == 1) tmem_dealloc(tmem_base, SmallMCfg<MPAD, OCC>::TMEM_COLS);
}

// QKV projection with the per-head post-processing (norm, RoPE, cache append) as its epilogue
template <int MPAD, bool BF16, int OCC = 1>
__global__ void __launch_bounds__(192, OCC)
gemm_qkv_post_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams p,
                     const QkvEpilogueParams qp) {
  uint32_t tmem_base;
  QkvEpilogue<BF16> epi{qp};
  gemm_smallm_device<MPAD, BF16, OCC, QkvEpilogue<BF16>>(tmW, tmX, p, tmem_base, KID_GEMM_SMALLM_PLAIN, epi);
  if ((threadIdx.x >> 5) == 1) tmem_dealloc(tmem_base, SmallMCfg<MPAD, OCC>::TMEM_COLS);
}

template <int BN, bool BF16>
__global__ void __launch_bounds__(192, 1)
gemm_largem_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW, const GemmParams p,
                   int tiles_m, int tiles_n) {
  gemm_largem_device<BN, BF16, LargeMPlainHook>(tmX, tmW, p, tiles_m, tiles_n, LargeMPlainHook{});
}

// ---------------------------------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------------------------------
template <int MPAD, bool BF16, int OCC>
static cudaError_t launch_smallm(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, int nsplit, int n_tiles,
                                 cudaStream_t stream, int batch = 1) {
  using Cfg = SmallMCfg<MPAD, OCC>;
  auto kern = gemm_smallm_kernel<MPAD, BF16, OCC>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, n_tiles, batch);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nsplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attr(attr, 1);
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p);
}

// Router projection of a mixture-of-experts layer with the expert selection as its epilogue (up to 128 experts = one weight
// tile): the k-split partial tiles are reduced by token rows, a warp owns a token and a lane four consecutive experts, then
// scores (softmax or sigmoid), selection bias, top-k with ties to the lower index, optional renormalisation -- what the
// separate launch after the router GEMM does (route_topk_kernel), on the fp32 logits before they ever reach memory.
struct RouteEpilogueParams {
  int* out_idx; float* out_w; const float* sel_bias;
  int E, topk, score_mode /*0 softmax 1 sigmoid 2 none*/, renorm;
  float route_scale;
};

template <bool BF16>
struct RouteEpilogue {
  RouteEpilogueParams r;
  __device__ __forceinline__ void operator()(const GemmParams& p, uint8_t* smem, int split, int nsplit, int n_tile) const {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const uint32_t P_addr = smem_u32(smem);
    const int rows_per = (p.M + nsplit - 1) / nsplit;
    const int r0 = split * rows_per;
    int r1 = r0 + rows_per; if (r1 > p.M) r1 = p.M;
    const int e0 = lane * 4;
    for (int j = r0 + warp; j < r1; j += nwarps) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < nsplit; ++s) {
        const float4 v = ld_dsmem_f4(mapa_u32(P_addr + (uint32_t)(j * 128 + e0) * 4u, (uint32_t)s));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      float sc[4] = {acc.x, acc.y, acc.z, acc.w}, sel[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) if (e0 + i >= r.E) sc[i] = -INFINITY;
      if (r.score_mode == 0) {
        float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) { sc[i] = e0 + i < r.E ? __expf(sc[i] - mx) : 0.f; sum += sc[i]; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[i] /= sum;
      } else if (r.score_mode == 1) {
#pragma unroll
        for (int i = 0; i < 4; ++i) sc[i] = 1.f / (1.f + __expf(-sc[i]));
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) sel[i] = e0 + i < r.E ? sc[i] + (r.sel_bias ? r.sel_bias[e0 + i] : 0.f) : -INFINITY;
      float wsum = 0.f, my_w = 0.f;
      int my_i = 0;
      for (int k = 0; k < r.topk; ++k) {
        float bv = -INFINITY, bs = 0.f;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (e0 + i < r.E && (sel[i] > bv || (sel[i] == bv && e0 + i < bi))) { bv = sel[i]; bi = e0 + i; bs = sc[i]; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, o), os = __shfl_xor_sync(0xffffffffu, bs, o);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = os; }
        }
        if ((bi >> 2) == lane) {
#pragma unroll
          for (int i = 0; i < 4; ++i) if ((bi & 3) == i) sel[i] = -INFINITY;      // out of the later rounds
        }
        wsum += bs;
        if (lane == k) { my_w = bs; my_i = bi; }
      }
      if (lane < r.topk) {
        float w = my_w;
        if (r.renorm) w = w / (wsum + 1e-20f);
        r.out_idx[(size_t)j * r.topk + lane] = my_i;
        r.out_w[(size_t)j * r.topk + lane] = w * r.route_scale;
      }
    }
  }
};

template <int MPAD, bool BF16>
__global__ void __launch_bounds__(192, 1)
gemm_route_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams p,
                  const RouteEpilogueParams rp) {
  uint32_t tmem_base;
  RouteEpilogue<BF16> epi{rp};
  gemm_smallm_device<MPAD, BF16, 1, RouteEpilogue<BF16>>(tmW, tmX, p, tmem_base, KID_GEMM_SMALLM_PLAIN, epi);
  if ((threadIdx.x >> 5) == 1) tmem_dealloc(tmem_base, SmallMCfg<MPAD, 1>::TMEM_COLS);
}
template <int MPAD, bool BF16>
static cudaError_t launch_route(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const RouteEpilogueParams& rp,
                                int nsplit, cudaStream_t stream) {
  using Cfg = SmallMCfg<MPAD, 1>;
  auto kern = gemm_route_kernel<MPAD, BF16>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nsplit, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nsplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attr(attr, 1);
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, rp);
}

template <int MPAD, bool BF16, int OCC = 1>
static cudaError_t launch_qkv_post(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const QkvEpilogueParams& qp,
                                   int nsplit, int n_tiles, cudaStream_t stream) {
  using Cfg = SmallMCfg<MPAD, OCC>;
  auto kern = gemm_qkv_post_kernel<MPAD, BF16, OCC>;
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
  attr[0].val.clusterDim.x = nsplit;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = add_pdl_attr(attr, 1);
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, qp);
}

template <int BN, bool BF16>
static cudaError_t launch_largem(const CUtensorMap& tmX, const CUtensorMap& tmW, const GemmParams& p, cudaStream_t stream) {
  using Cfg = LargeMCfg<BN>;
  auto kern = gemm_largem_kernel<BN, BF16>;
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return e;
  }
  const int tiles_n = (p.N + BN - 1) / BN, tiles_m = (p.M + 127) / 128;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long tiles = (long long)tiles_n * tiles_m;
  const int grid = (int)(tiles < sm_count ? tiles : sm_count);
  kern<<<grid, 192, Cfg::SMEM_BYTES, stream>>>(tmX, tmW, p, tiles_m, tiles_n);
  return cudaGetLastError();
}

}  // namespace fb

// Heuristic used by the launcher: how many cluster ranks split K so that about one CTA lands on each SM.
extern "C" int fb_gemm_pick_split(int M, int N, int K, int slots) {
  // Largest power-of-two split whose CTAs are all resident at once (slots = SMs x CTAs per SM) and that leaves
  // at least 8 k-blocks per rank.
  const int n_tiles = (N + 127) / 128;
  const int kb = K / 64;
  int best = 1;
  for (int s = 2; s <= 8; s *= 2) {
    if (n_tiles * s > slots) break;
    if (kb / s < 8) break;
    const int per = (kb + s - 1) / s;
    if ((s - 1) * per >= kb) break;             // every rank must own at least one block
    best = s;
  }
  return best;
}

// Y = X W^T.  dtype: 0 = fp16, 1 = bf16.  X: [M, K] row stride ldx; W: [N, K] row stride ldw (elements).
// nsplit <= 0 picks automatically.  Returns 0 on success, a cudaError_t, or -1 for unsupported shapes.
extern "C" int fb_gemm_16bit_wait(const void* X, const void* W, void* out, const void* bias, const void* residual, int M, int N,
                                  int K, int ldx, int ldw, int ld_out, int ld_res, int dtype, int flags, int nsplit,
                                  const void* wait_cnt, const void* wait_expect, void* stream_);

// Router GEMM + expert selection in one launch: X [M, K] 16-bit, W [E, K] 16-bit (E <= 128), M <= 128.
extern "C" int fb_gemm_route(const void* X, const void* W, int M, int E, int K, int ldx, int ldw, int dtype, const float* sel_bias,
                             int* out_idx, float* out_w, int topk, int score_mode, int renorm, float route_scale, void* stream_) {
  using namespace fb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0) return 0;
  if (M > 128 || E <= 0 || E > 128 || K % 64 != 0 || (dtype != 0 && dtype != 1) || topk <= 0 || topk > 32 || topk > E) return -1;
  GemmParams p;
  p.out = nullptr; p.bias = nullptr; p.residual = nullptr;
  p.M = M; p.N = E; p.K = K; p.ld_out = 0; p.ld_res = 0;
  p.kb_total = K / 64;
  p.flags = 0;
  p.scatter_tp = 0; p.scatter_rows = 1; p.scatter_rank = 0; p.w_row0 = 0; p.x_row0 = 0;
  for (int i = 0; i < 8; ++i) p.scatter_out[i] = nullptr;
  const bool bf16 = dtype == 1;
  const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
  int nsplit = 8;
  while (nsplit > 1 && p.kb_total / nsplit < 2) nsplit >>= 1;          // at least two k blocks per CTA
  p.kb_per_split = (p.kb_total + nsplit - 1) / nsplit;
  p.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, mpad);
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, W, E, K, ldw, 128, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmX, X, M, K, ldx, mpad, 64, 2, 3)) return -2;
  RouteEpilogueParams rp{out_idx, out_w, sel_bias, E, topk, score_mode, renorm, route_scale};
#define FB_RT(MP) return (int)(bf16 ? launch_route<MP, true>(tmW, tmX, p, rp, nsplit, stream) : launch_route<MP, false>(tmW, tmX, p, rp, nsplit, stream));
  switch (mpad) {
    case 16: FB_RT(16)
    case 32: FB_RT(32)
    case 64: FB_RT(64)
    default: FB_RT(128)
  }
#undef FB_RT
}

extern "C" int fb_gemm_16bit(const void* X, const void* W, void* out, const void* bias, const void* residual, int M, int N,
                             int K, int ldx, int ldw, int ld_out, int ld_res, int dtype, int flags, int nsplit, void* stream_) {
  return fb_gemm_16bit_wait(X, W, out, bias, residual, M, N, K, ldx, ldw, ld_out, ld_res, dtype, flags, nsplit, nullptr, nullptr, stream_);
}

// Same, for activations that a fused collective broadcast without waiting for its peers (small-M path only): the kernel
// itself waits until the arrival counter *wait_cnt has reached *wait_expect before it reads X.  Returns -3 when a wait
// is requested for a shape that the small-M kernel does not cover.
extern "C" int fb_gemm_16bit_wait(const void* X, const void* W, void* out, const void* bias, const void* residual, int M, int N,
                                  int K, int ldx, int ldw, int ld_out, int ld_res, int dtype, int flags, int nsplit,
                                  const void* wait_cnt, const void* wait_expect, void* stream_) {
  using namespace fb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (K % 64 != 0 || N % 8 != 0 || (dtype != 0 && dtype != 1)) return -1;
  if ((flags & GEMM_SWIGLU) && (N % 128 != 0)) return -1;
  GemmParams p;
  p.out = out; p.bias = bias; p.residual = residual;
  p.M = M; p.N = N; p.K = K; p.ld_out = ld_out; p.ld_res = ld_res;
  p.kb_total = K / 64;
  p.flags = flags;
  p.scatter_tp = 0; p.scatter_rows = 1; p.scatter_rank = 0; p.w_row0 = 0; p.x_row0 = 0;
  for (int i = 0; i < 8; ++i) p.scatter_out[i] = nullptr;
  p.wait_cnt = reinterpret_cast<const uint32_t*>(wait_cnt);
  p.wait_expect = reinterpret_cast<const uint32_t*>(wait_expect);
  if (wait_cnt != nullptr && M > 256) return -3;
  const bool bf16 = dtype == 1;
  if (M <= 256) {
    const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    static int sm_count = 0;
    if (sm_count == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    }
    // nsplit argument: low 4 bits = k split (0 = auto), bits 4.. = CTAs per SM (0 = auto)
    int occ = nsplit > 0 ? (nsplit >> 4) : 0;
    nsplit = nsplit > 0 ? (nsplit & 15) : 0;
    // two CTAs per SM pay off once there are more weight tiles than SMs (no k split): one CTA streams while the
    // other is in its prologue / epilogue
    if (occ == 0) occ = (mpad <= 128 && (N + 127) / 128 > sm_count) ? 2 : 1;
    if (mpad > 128) occ = 1;
    if (nsplit <= 0) nsplit = fb_gemm_pick_split(M, N, K, sm_count * occ);
    if (nsplit != 1 && nsplit != 2 && nsplit != 4 && nsplit != 8) return -1;
    p.kb_per_split = (p.kb_total + nsplit - 1) / nsplit;
    p.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, mpad);
    CUtensorMap tmW, tmX;
    if (!make_tmap_2d(&tmW, W, N, K, ldw, 128, 64, 2, 3)) return -2;
    if (!make_tmap_2d(&tmX, X, M, K, ldx, mpad, 64, 2, 3)) return -2;
    const int n_tiles = (N + 127) / 128;
#define FB_SM(MP)                                                                                        \
  if (occ == 2)                                                                                          \
    return (int)(bf16 ? launch_smallm<MP, true, 2>(tmW, tmX, p, nsplit, n_tiles, stream)                 \
                      : launch_smallm<MP, false, 2>(tmW, tmX, p, nsplit, n_tiles, stream));              \
  return (int)(bf16 ? launch_smallm<MP, true, 1>(tmW, tmX, p, nsplit, n_tiles, stream)                   \
                    : launch_smallm<MP, false, 1>(tmW, tmX, p, nsplit, n_tiles, stream));
    switch (mpad) {
      case 16: FB_SM(16)
      case 32: FB_SM(32)
      case 64: FB_SM(64)
      case 128: FB_SM(128)
      default:
        return (int)(bf16 ? launch_smallm<256, true, 1>(tmW, tmX, p, nsplit, n_tiles, stream)
                          : launch_smallm<256, false, 1>(tmW, tmX, p, nsplit, n_tiles, stream));
    }
#undef FB_SM
  }
  if (N % 32 != 0) return -1;
  p.kb_per_split = p.kb_total;
  int bn = (N >= 256 && N % 256 == 0) || N > 2048 ? 256 : 128;
  {
    // too few 128 x 256 tiles to occupy the SMs (a few hundred tokens): halve the tile width to double the CTA count
    int sms = 0, dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const long long t256 = (long long)((N + 255) / 256) * ((M + 127) / 128);
    if (bn == 256 && t256 < sms && !(flags & GEMM_SWIGLU && N % 256 != 0)) bn = 128;
  }
  p.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, bn);
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmX, X, M, K, ldx, 128, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmW, W, N, K, ldw, bn, 64, 2, 3)) return -2;
  if (bn == 256)
    return (int)(bf16 ? launch_largem<256, true>(tmX, tmW, p, stream) : launch_largem<256, false>(tmX, tmW, p, stream));
  return (int)(bf16 ? launch_largem<128, true>(tmX, tmW, p, stream) : launch_largem<128, false>(tmX, tmW, p, stream));
}

// QKV projection (head_dim 128, M <= 256, N = (Hq + 2 Hkv) * 128) with split / per-head RMSNorm / RoPE / paged-cache append in
// the epilogue: Q rows go to q_out, K and V rows to their cache slots (slots[j] < 0: not cached).  wait_cnt / wait_expect as in
// fb_gemm_16bit_wait.  rope_mode 0 none, 1 neox, 2 interleaved; rot must be a multiple of 8.  Returns -1 for other shapes.
extern "C" int fb_gemm_qkv_post(const void* X, const void* W, const void* bias, int M, int N, int K, int ldx, int ldw, int dtype,
                                const void* wait_cnt, const void* wait_expect, void* q_out, int ld_q, void* k_pool, void* v_pool,
                                const int* positions, const int* slots, const void* q_norm_w, const void* k_norm_w,
                                const float* cos_tab, const float* sin_tab, int Hq, int Hkv, int rot, int rope_mode, float eps,
                                float norm_unit_offset, void* stream_) {
  using namespace fb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0) return 0;
  if (M > 256 || K % 64 != 0 || N != (Hq + 2 * Hkv) * 128 || (dtype != 0 && dtype != 1) || rot % 8 != 0 || rot > 128 || rot < 0) return -1;
  GemmParams p;
  p.out = nullptr; p.bias = bias; p.residual = nullptr;
  p.M = M; p.N = N; p.K = K; p.ld_out = 0; p.ld_res = 0;
  p.kb_total = K / 64;
  p.flags = bias ? GEMM_BIAS : 0;
  p.scatter_tp = 0; p.scatter_rows = 1; p.scatter_rank = 0; p.w_row0 = 0; p.x_row0 = 0;
  for (int i = 0; i < 8; ++i) p.scatter_out[i] = nullptr;
  p.wait_cnt = reinterpret_cast<const uint32_t*>(wait_cnt);
  p.wait_expect = reinterpret_cast<const uint32_t*>(wait_expect);
  const bool bf16 = dtype == 1;
  const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const int n_tiles = N / 128;
  if (n_tiles > sm_count) return -1;
  // Power-of-two cluster sizes only: clusters of 3 or 6 CTAs measured 35-50 % slower on this part (they fit the GPCs badly
  // and fewer of them are resident at once), although 48 heads x 3 would cover 144 of the 148 SMs.
  // decode-sized batches: two CTAs per SM (half the pipeline depth each), so that a deeper k-split still has every CTA resident
  // -- 48 head tiles x 4 = 192 CTAs on 148 SMs instead of 96 on 96
  static const bool occ2_ok = [] { const char* e = getenv("FB_QKV_POST_OCC2"); return !(e && e[0] == '0'); }();
  const bool occ2 = mpad <= 64 && occ2_ok;
  const int nsplit = fb_gemm_pick_split(M, N, K, occ2 ? 2 * sm_count : sm_count);
  p.kb_per_split = (p.kb_total + nsplit - 1) / nsplit;
  p.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, mpad);
  QkvEpilogueParams qp;
  qp.q_out = (uint16_t*)q_out; qp.ld_q = ld_q; qp.k_pool = (uint16_t*)k_pool; qp.v_pool = (uint16_t*)v_pool;
  qp.positions = positions; qp.slots = slots; qp.q_norm_w = (const uint16_t*)q_norm_w; qp.k_norm_w = (const uint16_t*)k_norm_w;
  qp.cos_tab = cos_tab; qp.sin_tab = sin_tab; qp.Hq = Hq; qp.Hkv = Hkv; qp.rot = rot; qp.rope_mode = rope_mode;
  qp.eps = eps; qp.norm_unit_offset = norm_unit_offset;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, W, N, K, ldw, 128, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmX, X, M, K, ldx, mpad, 64, 2, 3)) return -2;
#define FB_QP(MP)                                                                                     \
  return (int)(bf16 ? launch_qkv_post<MP, true>(tmW, tmX, p, qp, nsplit, n_tiles, stream)              \
                    : launch_qkv_post<MP, false>(tmW, tmX, p, qp, nsplit, n_tiles, stream));
#define FB_QP2(MP)                                                                                    \
  if (occ2)                                                                                           \
    return (int)(bf16 ? launch_qkv_post<MP, true, 2>(tmW, tmX, p, qp, nsplit, n_tiles, stream)         \
                      : launch_qkv_post<MP, false, 2>(tmW, tmX, p, qp, nsplit, n_tiles, stream));      \
  FB_QP(MP)
  switch (mpad) {
    case 16: FB_QP2(16)
    case 32: FB_QP2(32)
    case 64: FB_QP2(64)
    case 128: FB_QP(128)
    default: FB_QP(256)
  }
#undef FB_QP2
#undef FB_QP
}

// Batched small-M GEMM, one launch for `batch` independent products that share the token rows:
//   out[m, z * out_cols + n] = sum_k X[m, z * x_cols + k] * W[z * N + n, k]      (z < batch, n < N, k < K)
// X: [M, >= batch * x_cols] (row stride ldx), W: [batch * N, K] (row stride ldw), out row stride ld_out; 16-bit in and out.
// Used for the absorbed multi-head-latent-attention projections (one small matrix per head).  M <= 256, K % 64 == 0,
// N % 8 == 0, x_cols % 8 == 0, out_cols % 4 == 0.
extern "C" int fb_gemm_16bit_batched(const void* X, const void* W, void* out, int M, int N, int K, int batch, int ldx, int ldw, int ld_out,
                                     int x_cols, int out_cols, int dtype, void* stream_) {
  using namespace fb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || batch <= 0) return 0;
  if (M > 256 || K % 64 != 0 || N % 8 != 0 || x_cols % 8 != 0 || out_cols % 4 != 0 || batch > 65535 || (dtype != 0 && dtype != 1)) return -1;
  GemmParams p;
  p.out = out; p.bias = nullptr; p.residual = nullptr;
  p.M = M; p.N = N; p.K = K; p.ld_out = ld_out; p.ld_res = 0;
  p.kb_total = K / 64; p.kb_per_split = p.kb_total;
  p.flags = 0;
  p.scatter_tp = 0; p.scatter_rows = 1; p.scatter_rank = 0; p.w_row0 = 0; p.x_row0 = 0;
  for (int i = 0; i < 8; ++i) p.scatter_out[i] = nullptr;
  p.batch_w_rows = N; p.batch_x_cols = x_cols; p.batch_out_cols = out_cols;
  const bool bf16 = dtype == 1;
  const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  p.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, mpad);
  CUtensorMap tmW, tmX;
  // the weight map spans all batches' rows; a tile that overhangs one head's N rows reads the next head's rows, whose
  // products land in columns >= N of the tile and are dropped by the epilogue's n < N test
  if (!make_tmap_2d(&tmW, W, (uint64_t)batch * N, K, ldw, 128, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmX, X, M, (uint64_t)(batch - 1) * x_cols + K, ldx, mpad, 64, 2, 3)) return -2;
  const int n_tiles = (N + 127) / 128;
#define FB_BT(MP)                                                                                        \
  return (int)(bf16 ? launch_smallm<MP, true, 2>(tmW, tmX, p, 1, n_tiles, stream, batch)                 \
                    : launch_smallm<MP, false, 2>(tmW, tmX, p, 1, n_tiles, stream, batch));
  switch (mpad) {
    case 16: FB_BT(16)
    case 32: FB_BT(32)
    case 64: FB_BT(64)
    case 128: FB_BT(128)
    default:
      return (int)(bf16 ? launch_smallm<256, true, 1>(tmW, tmX, p, 1, n_tiles, stream, batch)
                        : launch_smallm<256, false, 1>(tmW, tmX, p, 1, n_tiles, stream, batch));
  }
#undef FB_BT
}
