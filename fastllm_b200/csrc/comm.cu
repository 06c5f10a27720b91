// Tensor-parallel communication kernels over NVLink peer memory (sm_100a): no NCCL call on these paths.
//
//  * fb_gemm_ar_norm: row-parallel small-M GEMM (tcgen05, swap-AB, cluster split-K) FUSED with
//    reduce-scatter -> (+residual) -> RMSNorm -> all-gather in ONE kernel:
//       phase 1  rank r owns token rows [r*M/tp, (r+1)*M/tp).  The GEMM epilogue PUSHES each fp32 partial row
//                straight into its owner's arena (slot = source rank) with peer stores: the reduce-scatter
//                costs one NVLink traversal, no pull round trip
//       sync 1   one aggregated arrival per rank on a counter in every rank (multimem.red through NVSwitch,
//                or P2P red)
//       phase 2  the owner sums the tp slots of its rows in rank order (local reads, deterministic), adds
//                the residual row, writes the new residual-stream row and its RMSNorm'd version to EVERY
//                rank (multimem.st through NVSwitch multicast, or P2P stores)
//       sync 2   second counter; the kernel ends only when every rank's rows have landed here, so the
//                next kernel on the stream can read the full hidden state without further waits.
//  * fb_ar_norm: phases 2.. alone for partials produced elsewhere (MoE output, embeddings).
//  * fb_argmax_merge: all-gather of per-rank (max, arg-max) candidates + merge (vocab-sharded greedy).
//
// The reference's counterpart is a separate custom all-reduce launch after the GEMM, with unbounded
// spins (src/devices/multicuda/fastllm-custom-allreduce.cu:242-368, fused add at :638); here every wait
// is bounded in time and reports through the error word.
//
// Counters only grow; the expected value is carried in a local word, so no reset races exist.  All CTAs
// of a launch must be co-resident (they wait for each other across ranks): launchers check the grid
// against the SM count.
#include "gemm_smallm.cuh"
#include "launch.h"
#include "tmap.h"
#include "comm.cuh"

FB_DEFINE_ERROR_API(comm)

namespace fb {

template <int MPAD, bool BF16>
__global__ void __launch_bounds__(192, 1)
gemm_ar_norm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams g,
                    const ArNormParams p) {
  const uint64_t t_start = p.trace ? globaltimer_ns() : 0;
  uint32_t tmem_base;
  gemm_smallm_device<MPAD, BF16>(tmW, tmX, g, tmem_base, KID_GEMM_AR);
  // every thread has passed the dependency wait inside the GEMM: the expect word written by the previous collective is final
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(p.c.local + OFF_EXPECT);
  if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) reinterpret_cast<uint64_t*>(p.c.local + OFF_TRACE)[0] = t_start;
  if ((threadIdx.x >> 5) == 1) tmem_dealloc(tmem_base, SmallMCfg<MPAD>::TMEM_COLS);
  // cluster = the gridDim.x k-split CTAs of one weight tile
  ar_norm_tail<BF16>(p, base, blockIdx.y, gridDim.y, blockIdx.x, gridDim.x, KID_GEMM_AR);
}

template <bool BF16>
__global__ void __launch_bounds__(192, 1) ar_norm_kernel(const ArNormParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(p.c.local + OFF_EXPECT);
  if (p.trace && blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<uint64_t*>(p.c.local + OFF_TRACE)[0] = globaltimer_ns();
  // phase 1: push this rank's partial rows to their owners (slot = this rank)
  const CommCtx& c = p.c;
  const int rows_per = (p.M + c.tp - 1) / c.tp;
  const int chunks = p.N >> 3;
  const long long total = (long long)p.M * chunks;
  for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(it / chunks), ch = (int)(it - (long long)row * chunks);
    float4 a, b;
    if (p.moe_ys != nullptr) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int k = 0; k < p.moe_topk; ++k) {
        const int r = p.moe_pos[row * p.moe_topk + k];
        if (r < 0) continue;
        const float wk = p.moe_w[row * p.moe_topk + k];
        const uint4 v = *reinterpret_cast<const uint4*>(p.moe_ys + (size_t)r * p.N + (size_t)ch * 8);
        const float2 v0 = unpack_16<BF16>(v.x), v1 = unpack_16<BF16>(v.y), v2 = unpack_16<BF16>(v.z), v3 = unpack_16<BF16>(v.w);
        acc[0] += wk * v0.x; acc[1] += wk * v0.y; acc[2] += wk * v1.x; acc[3] += wk * v1.y;
        acc[4] += wk * v2.x; acc[5] += wk * v2.y; acc[6] += wk * v3.x; acc[7] += wk * v3.y;
      }
      if (p.moe_add != nullptr) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.moe_add + (size_t)row * p.N + (size_t)ch * 8);
        const float2 v0 = unpack_16<BF16>(v.x), v1 = unpack_16<BF16>(v.y), v2 = unpack_16<BF16>(v.z), v3 = unpack_16<BF16>(v.w);
        acc[0] += v0.x; acc[1] += v0.y; acc[2] += v1.x; acc[3] += v1.y; acc[4] += v2.x; acc[5] += v2.y; acc[6] += v3.x; acc[7] += v3.y;
      }
      a = make_float4(acc[0], acc[1], acc[2], acc[3]); b = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else if (p.src_f32) {
      const float4* sp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.src) + (size_t)row * p.N + (size_t)ch * 8);
      a = sp[0]; b = sp[1];
    } else {
      const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.src) + (size_t)row * p.N + (size_t)ch * 8);
      const float2 v0 = unpack_16<BF16>(v.x), v1 = unpack_16<BF16>(v.y), v2 = unpack_16<BF16>(v.z), v3 = unpack_16<BF16>(v.w);
      a = make_float4(v0.x, v0.y, v1.x, v1.y); b = make_float4(v2.x, v2.y, v3.x, v3.y);
    }
    float4* dst = reinterpret_cast<float4*>(c.peer[row / rows_per] + p.off_part + (((size_t)c.rank * p.M + row) * p.N + (size_t)ch * 8) * 4);
    dst[0] = a; dst[1] = b;
  }
  const int cs = (int)cluster_nctarank();
  ar_norm_tail<BF16>(p, base, blockIdx.x / cs, gridDim.x / cs, (int)cluster_ctarank(), cs, KID_AR_NORM);
}

// ---- vocab-sharded greedy merge: every rank publishes (max value, arg-max id) per row, then picks the best ----
struct ArgmaxMergeParams {
  CommCtx c;
  uint64_t off_buf;          // [tp][B][2] 32-bit words (value as float bits, id)
  const float* vals; const int* ids; int* out; int B;
};
__global__ void argmax_merge_kernel(const ArgmaxMergeParams p) {
  __shared__ int sh_ok;
  const CommCtx& c = p.c;
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t base = *reinterpret_cast<volatile uint32_t*>(c.local + OFF_EXPECT);
  const uint32_t target = base + (uint32_t)c.tp;
  const int tid = threadIdx.x;
  for (int b = tid; b < p.B; b += blockDim.x) {
    const uint2 v = make_uint2(__float_as_uint(p.vals[b]), (uint32_t)p.ids[b]);
    const uint64_t off = p.off_buf + ((uint64_t)(c.rank * p.B + b)) * 8;
    if (c.mc) {
      asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};\n" ::"l"(c.mc + off), "f"(__uint_as_float(v.x)),
                   "f"(__uint_as_float(v.y)) : "memory");
    } else {
      for (int r = 0; r < c.tp; ++r) *reinterpret_cast<uint2*>(c.peer[r] + off) = v;
    }
  }
  __syncthreads();
  if (tid == 0) {
    signal_all(c, OFF_CNT1);
    sh_ok = wait_counter(c, OFF_CNT1, target, KID_ARGMAX_MERGE, 1) ? 1 : 0;
  }
  __syncthreads();
  if (sh_ok) {
    for (int b = tid; b < p.B; b += blockDim.x) {
      float best = -INFINITY; int bi = 0;
      for (int r = 0; r < c.tp; ++r) {
        const volatile uint32_t* src = reinterpret_cast<const volatile uint32_t*>(c.local + p.off_buf + ((uint64_t)(r * p.B + b)) * 8);
        const float f = __uint_as_float(src[0]);
        if (f > best) { best = f; bi = (int)src[1]; }      // strict: ties keep the lower rank = lower token id
      }
      p.out[b] = bi;
    }
  }
  __syncthreads();
  if (tid == 0) {
    // second counter keeps the buffer from being overwritten by a rank that is one launch ahead
    signal_all(c, OFF_CNT2);
    wait_counter(c, OFF_CNT2, target, KID_ARGMAX_MERGE, 2);
    *reinterpret_cast<volatile uint32_t*>(c.local + OFF_EXPECT) = target;
    __threadfence();
  }
}

template <int MPAD, bool BF16>
static cudaError_t launch_gemm_ar(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& g, const ArNormParams& p,
                                  int nsplit, int n_tiles, cudaStream_t stream) {
  using Cfg = SmallMCfg<MPAD>;
  auto kern = gemm_ar_norm_kernel<MPAD, BF16>;
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
  if (cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg) == cudaSuccess && max_clusters > 0 && n_tiles > max_clusters)
    return cudaErrorLaunchOutOfResources;
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, g, p);
}

}  // namespace fb

using namespace fb;

extern "C" int fb_gemm_pick_split(int M, int N, int K, int sm_count);

// Arena header must be zeroed (and all ranks synchronised) once before the first launch.
// X: [M, K_local] activations of this rank; W: [N, K_local] this rank's weight shard; bias only on one rank.
// off_part / off_h / off_x: symmetric offsets inside the arena.  has_residual: h += sum (else h = sum).
// ln_w == nullptr skips the norm.  Returns cudaErrorLaunchOutOfResources if the grid cannot be co-resident.
extern "C" int fb_gemm_ar_norm(const void* X, const void* W, const void* bias, int M, int N, int K, int ldx, int ldw,
                               void* arena_local, void* arena_mc, void* const* peers, int rank, int tp, unsigned long long off_part,
                               unsigned long long off_h, unsigned long long off_x, const void* ln_w, int has_residual, float eps,
                               float unit_offset, int dtype, int nsplit, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || M > 256 || K % 64 != 0 || N % 8 != 0 || N > 18432 || tp > MAX_TP) return -1;
  const bool bf16 = dtype == 1;
  const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
  const int n_tiles = (N + 127) / 128;
  if (nsplit <= 0) nsplit = fb_gemm_pick_split(M, N, K, sm_count());
  while (nsplit > 1 && n_tiles * nsplit > sm_count()) nsplit >>= 1;
  if (n_tiles * nsplit > sm_count()) return (int)cudaErrorLaunchOutOfResources;
  GemmParams g;
  g.out = (uint8_t*)arena_local + off_part; g.bias = bias; g.residual = nullptr;
  g.M = M; g.N = N; g.K = K; g.ld_out = N; g.ld_res = 0;
  g.scatter_tp = tp; g.scatter_rows = (M + tp - 1) / tp; g.scatter_rank = rank; g.w_row0 = 0; g.x_row0 = 0;
  for (int i = 0; i < 8; ++i) g.scatter_out[i] = i < tp ? reinterpret_cast<float*>((uint8_t*)peers[i] + off_part) : nullptr;
  g.kb_total = K / 64; g.kb_per_split = (g.kb_total + nsplit - 1) / nsplit;
  g.flags = GEMM_OUT_F32 | (bias ? GEMM_BIAS : 0);
  g.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, mpad);
  ArNormParams p;
  fill_ctx(p.c, arena_local, arena_mc, peers, rank, tp);
  p.off_part = off_part; p.off_h = off_h; p.off_x = off_x; p.ln_w = (const uint16_t*)ln_w; p.M = M; p.N = N;
  p.has_residual = has_residual & 1; p.trace = (has_residual >> 1) & 1; p.defer_sync2 = (has_residual >> 2) & 1; p.eps = eps; p.unit_offset = unit_offset;
  p.src = nullptr; p.src_f32 = 0; p.moe_ys = nullptr; p.moe_pos = nullptr; p.moe_w = nullptr; p.moe_add = nullptr; p.moe_topk = 0;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, W, N, K, ldw, 128, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmX, X, M, K, ldx, mpad, 64, 2, 3)) return -2;
#define FB_GA(MP)                                                                                       \
  return (int)(bf16 ? launch_gemm_ar<MP, true>(tmW, tmX, g, p, nsplit, n_tiles, stream)                  \
                    : launch_gemm_ar<MP, false>(tmW, tmX, g, p, nsplit, n_tiles, stream));
  switch (mpad) {
    case 16: FB_GA(16)
    case 32: FB_GA(32)
    case 64: FB_GA(64)
    case 128: FB_GA(128)
    default: FB_GA(256)
  }
#undef FB_GA
}

static int launch_ar_norm(ArNormParams& p, int M, int N, int tp, int dtype, cudaStream_t stream) {
  int rows_per = (M + tp - 1) / tp;
  const int cs = N >= 4096 ? 4 : (N >= 2048 ? 2 : 1);     // CTAs per row
  int groups = rows_per < 1 ? 1 : rows_per;
  if (groups * cs > sm_count()) groups = sm_count() / cs;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(groups * cs, 1, 1);
  cfg.blockDim = dim3(192, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = add_pdl_attr(attr, 1);
  if (dtype == 1) return (int)cudaLaunchKernelEx(&cfg, ar_norm_kernel<true>, p);
  return (int)cudaLaunchKernelEx(&cfg, ar_norm_kernel<false>, p);
}

// All-reduce (+residual, +RMSNorm) of this rank's partial `src` [M, N] (fp32 if src_f32 else the 16-bit dtype).
extern "C" int fb_ar_norm(const void* src, int src_f32, int M, int N, void* arena_local, void* arena_mc, void* const* peers, int rank,
                          int tp, unsigned long long off_part, unsigned long long off_h, unsigned long long off_x, const void* ln_w,
                          int has_residual, float eps, float unit_offset, int dtype, void* stream_) {
  if (M <= 0 || N % 8 != 0 || N > 18432 || tp > MAX_TP) return -1;
  ArNormParams p;
  fill_ctx(p.c, arena_local, arena_mc, peers, rank, tp);
  p.off_part = off_part; p.off_h = off_h; p.off_x = off_x; p.ln_w = (const uint16_t*)ln_w; p.M = M; p.N = N;
  p.has_residual = has_residual & 1; p.trace = (has_residual >> 1) & 1; p.defer_sync2 = (has_residual >> 2) & 1; p.eps = eps; p.unit_offset = unit_offset;
  p.src = src; p.src_f32 = src_f32; p.moe_ys = nullptr; p.moe_pos = nullptr; p.moe_w = nullptr; p.moe_add = nullptr; p.moe_topk = 0;
  return launch_ar_norm(p, M, N, tp, dtype, reinterpret_cast<cudaStream_t>(stream_));
}

// Expert-parallel combine fused with the cross-rank reduction: this rank's weighted sum over its local experts' outputs
// (ys rows addressed by pos, -1 = expert on another rank; `add` = e.g. the shared expert's partial) is formed on the fly,
// pushed to the row owners, reduced, joined with the residual, normalised and broadcast.
extern "C" int fb_moe_combine_ar_norm(const void* ys, const int* pos, const float* w, const void* add, int topk, int M, int N,
                                      void* arena_local, void* arena_mc, void* const* peers, int rank, int tp,
                                      unsigned long long off_part, unsigned long long off_h, unsigned long long off_x, const void* ln_w,
                                      int has_residual, float eps, float unit_offset, int dtype, void* stream_) {
  if (M <= 0 || N % 8 != 0 || N > 18432 || tp > MAX_TP) return -1;
  ArNormParams p;
  fill_ctx(p.c, arena_local, arena_mc, peers, rank, tp);
  p.off_part = off_part; p.off_h = off_h; p.off_x = off_x; p.ln_w = (const uint16_t*)ln_w; p.M = M; p.N = N;
  p.has_residual = has_residual & 1; p.trace = (has_residual >> 1) & 1; p.defer_sync2 = (has_residual >> 2) & 1; p.eps = eps; p.unit_offset = unit_offset;
  p.src = nullptr; p.src_f32 = 0;
  p.moe_ys = (const uint16_t*)ys; p.moe_pos = pos; p.moe_w = w; p.moe_add = (const uint16_t*)add; p.moe_topk = topk;
  return launch_ar_norm(p, M, N, tp, dtype, reinterpret_cast<cudaStream_t>(stream_));
}

// One-thread kernel that ends once the deferred all-gather of the previous fused collective has landed on this rank
// (CNT2 >= EXPECT); for consumers that cannot wait themselves.
__global__ void comm_wait_kernel(const uint8_t* local) {
  pdl_launch_dependents();
  pdl_wait();
  const uint32_t target = *reinterpret_cast<const volatile uint32_t*>(local + fb::OFF_EXPECT);
  fb::wait_counter_ge(reinterpret_cast<const uint32_t*>(local + fb::OFF_CNT2), target, fb::KID_AR_NORM, 3);
}
extern "C" int fb_comm_wait(const void* arena_local, void* stream_) {
  launch_k(comm_wait_kernel, dim3(1), dim3(1), 0, reinterpret_cast<cudaStream_t>(stream_), 0, reinterpret_cast<const uint8_t*>(arena_local));
  return (int)cudaGetLastError();
}
extern "C" void fb_comm_header_offsets(unsigned* cnt2, unsigned* expect) { *cnt2 = fb::OFF_CNT2; *expect = fb::OFF_EXPECT; }

extern "C" int fb_argmax_merge(const float* vals, const int* ids, int* out, int B, void* arena_local, void* arena_mc,
                               void* const* peers, int rank, int tp, unsigned long long off_buf, void* stream_) {
  if (B <= 0 || tp > MAX_TP) return -1;
  ArgmaxMergeParams p;
  fill_ctx(p.c, arena_local, arena_mc, peers, rank, tp);
  p.off_buf = off_buf; p.vals = vals; p.ids = ids; p.out = out; p.B = B;
  launch_k(argmax_merge_kernel, dim3(1), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream_), 0, p);
  return (int)cudaGetLastError();
}
