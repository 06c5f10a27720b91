// Mixture-of-experts execution for sm_100a: routing plan, token gather, grouped expert GEMMs, weighted combine.
//
//   moe_plan     one CTA: per-local-expert token counts, segment offsets padded to 16 rows, and for every (token, k)
//                pair its row in the expert-sorted buffer (-1 if the expert lives on another rank).  Deterministic:
//                rows inside a segment follow (token, k) order.
//   moe_gather   copies each routed token row into its sorted position
//   grouped GEMM the swap-AB tcgen05 decode GEMM run once per (expert, 128/256-token chunk) through blockIdx.z; the
//                weight tile coordinate is offset into the stacked expert matrix, the activation tile into the sorted
//                buffer; experts without tokens exit at once.  gate/up uses the SwiGLU epilogue.
//   moe_combine  out[t] = sum_k w[t,k] * y_sorted[pos[t,k]]   in fixed k order (deterministic)
//
// Role of the reference's MergeMOE / FusedMOE (src/devices/cuda/cudadevice.cpp:8279-8562) and of its routed-row
// kernels ("Grouped...Indexed", src/devices/cuda/moe/fastllm-moe-fp8.cu; route count/offset/scatter in
// fastllm-moe-vllm-marlin.cu:405-528), which run the expert FFNs as CUDA-core GEMVs or Marlin mma.sync.
#include "gemm_smallm.cuh"
#include "launch.h"
#include "tmap.h"

FB_DEFINE_ERROR_API(moe)

namespace fb {

constexpr int KID_MOE_GROUPED = 40;

struct MoeGroupInfo {
  const int* counts;       // [E_local] routed rows per expert
  const int* offsets;      // [E_local] first row of the expert's segment in the sorted buffer
  int rows_per_chunk;      // MPAD
  int chunks;              // blockIdx.z = expert * chunks + chunk
  int n_rows_w;            // weight rows per expert in the stacked matrix
  long long out_stride_e;  // unused (outputs follow the sorted rows)
  int ld_bias_e;           // bias elements per expert (0: no per-expert stride)
  int n_local, compact;    // compact: grid.z enumerates existing (expert, chunk) pairs (moe_find_item)
};

// counts/offsets/pos for the experts in [first, first + n_local)
__global__ void moe_plan_kernel(const int* __restrict__ idx, int T, int topk, int first, int n_local, int* __restrict__ counts,
                                int* __restrict__ offsets, int* __restrict__ pos, int* __restrict__ total_rows, int pad) {
  __shared__ int s_cnt[1024];
  __shared__ int s_off[1025];
  const int e = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int pairs = T * topk;
  int c = 0;
  if (e < n_local) {
    for (int i = 0; i < pairs; ++i) c += (idx[i] == first + e);
  }
  s_cnt[e] = e < n_local ? c : 0;
  __syncthreads();
  if (e == 0) {
    int acc = 0;
    for (int i = 0; i < n_local; ++i) { s_off[i] = acc; acc += (s_cnt[i] + pad - 1) / pad * pad; }
    s_off[n_local] = acc;
    *total_rows = acc;
  }
  __syncthreads();
  if (e < n_local) {
    counts[e] = s_cnt[e];
    offsets[e] = s_off[e];
    int r = s_off[e];
    for (int i = 0; i < pairs; ++i)
      if (idx[i] == first + e) pos[i] = r++;
  }
  // pairs whose expert is not local
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int x = idx[i];
    if (x < first || x >= first + n_local) pos[i] = -1;
  }
}

// Small problems (pairs <= 4096): one thread per (token, k) pair; rank inside the expert segment = number of earlier pairs
// routed to the same expert, so the order is deterministic without any sorting pass.
__global__ void moe_plan_small_kernel(const int* __restrict__ idx, int pairs, int first, int n_local, int* __restrict__ counts,
                                      int* __restrict__ offsets, int* __restrict__ pos, int* __restrict__ total_rows, int pad) {
  __shared__ int s_idx[4096];
  __shared__ int s_cnt[1024];
  __shared__ int s_off[1024];
  pdl_launch_dependents();
  pdl_wait();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = idx[i] - first;
    s_idx[i] = (e >= 0 && e < n_local) ? e : -1;
  }
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) s_cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x)
    if (s_idx[i] >= 0) atomicAdd(&s_cnt[s_idx[i]], 1);
  __syncthreads();
  if (threadIdx.x < 32) {
    // warp-level exclusive scan of the padded counts, 32 experts at a time
    int carry = 0;
    for (int base = 0; base < n_local; base += 32) {
      const int e = base + threadIdx.x;
      const int c = e < n_local ? (s_cnt[e] + pad - 1) / pad * pad : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if ((int)threadIdx.x >= o) incl += v;
      }
      if (e < n_local) s_off[e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (threadIdx.x == 0) *total_rows = carry;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) { counts[e] = s_cnt[e]; offsets[e] = s_off[e]; }
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = s_idx[i];
    if (e < 0) { pos[i] = -1; continue; }
    int rank = 0;
    for (int j = 0; j < i; ++j) rank += (s_idx[j] == e);
    pos[i] = s_off[e] + rank;
  }
}

// The same plan with warp votes: pairs are taken in chunks of 32; a chunk's lanes learn by `match.any` how many earlier lanes
// go to the same expert, one lane per (chunk, expert) records the chunk's count, a scan over the chunks per expert turns the
// counts into bases, and rank = base of the chunk + earlier lanes of the chunk.  Same (deterministic) order as above at
// O(chunks) instead of O(pairs) work per thread.  Needs chunks * n_local <= 8192 (16-bit counts in shared memory).
__global__ void __launch_bounds__(1024)
moe_plan_warp_kernel(const int* __restrict__ idx, int pairs, int first, int n_local, int* __restrict__ counts,
                     int* __restrict__ offsets, int* __restrict__ pos, int* __restrict__ total_rows, int pad) {
  __shared__ int s_idx[4096];
  __shared__ uint16_t s_w[8192];
  __shared__ int s_cnt[1024];
  __shared__ int s_off[1024];
  pdl_launch_dependents();
  pdl_wait();
  const int chunks = (pairs + 31) >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const uint32_t lt_mask = (1u << lane) - 1u;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = idx[i] - first;
    s_idx[i] = (e >= 0 && e < n_local) ? e : -1;
  }
  for (int i = threadIdx.x; i < chunks * n_local; i += blockDim.x) s_w[i] = 0;
  __syncthreads();
  for (int c = warp; c < chunks; c += nwarps) {
    const int i = (c << 5) + lane;
    const int e = i < pairs ? s_idx[i] : -1;
    const uint32_t same = __match_any_sync(0xffffffffu, e);
    if (e >= 0 && (same & lt_mask) == 0) s_w[c * n_local + e] = (uint16_t)__popc(same);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) {
    int run = 0;
    for (int c = 0; c < chunks; ++c) {
      const int v = s_w[c * n_local + e];
      s_w[c * n_local + e] = (uint16_t)run;
      run += v;
    }
    s_cnt[e] = run;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    int carry = 0;
    for (int base = 0; base < n_local; base += 32) {
      const int e = base + threadIdx.x;
      const int c = e < n_local ? (s_cnt[e] + pad - 1) / pad * pad : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if ((int)threadIdx.x >= o) incl += v;
      }
      if (e < n_local) s_off[e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (threadIdx.x == 0) *total_rows = carry;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < n_local; e += blockDim.x) { counts[e] = s_cnt[e]; offsets[e] = s_off[e]; }
  for (int c = warp; c < chunks; c += nwarps) {
    const int i = (c << 5) + lane;
    const int e = i < pairs ? s_idx[i] : -1;
    const uint32_t same = __match_any_sync(0xffffffffu, e);
    if (i < pairs) pos[i] = e < 0 ? -1 : s_off[e] + (int)s_w[c * n_local + e] + __popc(same & lt_mask);
  }
}

__global__ void moe_gather_kernel(const uint16_t* __restrict__ x, const int* __restrict__ pos, uint16_t* __restrict__ xs, int T,
                                  int topk, int H) {
  const int pair = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  const int r = pos[pair];
  if (r < 0) return;
  const int t = pair / topk;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)t * H);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)r * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

template <bool BF16>
__global__ void moe_combine_kernel(const uint16_t* __restrict__ ys, const int* __restrict__ pos, const float* __restrict__ w,
                                   const uint16_t* __restrict__ add, uint16_t* __restrict__ out, int topk, int H) {
  const int t = blockIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < topk; ++k) {
      const int r = pos[t * topk + k];
      if (r < 0) continue;
      const float wk = w[t * topk + k];
      const uint4 v = *reinterpret_cast<const uint4*>(ys + (size_t)r * H + c * 8);
      const float2 a = unpack_16<BF16>(v.x), b = unpack_16<BF16>(v.y), cc = unpack_16<BF16>(v.z), d = unpack_16<BF16>(v.w);
      acc[0] += wk * a.x; acc[1] += wk * a.y; acc[2] += wk * b.x; acc[3] += wk * b.y;
      acc[4] += wk * cc.x; acc[5] += wk * cc.y; acc[6] += wk * d.x; acc[7] += wk * d.y;
    }
    if (add != nullptr) {
      const uint4 v = *reinterpret_cast<const uint4*>(add + (size_t)t * H + c * 8);
      const float2 a = unpack_16<BF16>(v.x), b = unpack_16<BF16>(v.y), cc = unpack_16<BF16>(v.z), d = unpack_16<BF16>(v.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_16<BF16>(acc[0], acc[1]); o.y = pack_16<BF16>(acc[2], acc[3]);
    o.z = pack_16<BF16>(acc[4], acc[5]); o.w = pack_16<BF16>(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + (size_t)t * H + c * 8) = o;
  }
}

// grouped dense GEMM: one (expert, chunk) per blockIdx.z
template <int MPAD, bool BF16>
__global__ void __launch_bounds__(192, 1)
moe_grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const GemmParams base,
                        const MoeGroupInfo gi) {
  int e = blockIdx.z / gi.chunks, chunk = blockIdx.z - e * gi.chunks;
  pdl_launch_dependents();
  pdl_wait();   // counts / offsets come from the plan kernel
  if (gi.compact && !moe_find_item(gi.counts, gi.n_local, gi.rows_per_chunk, (int)blockIdx.z, e, chunk)) return;
  const int cnt = gi.counts[e];
  const int row0 = chunk * gi.rows_per_chunk;
  if (row0 >= cnt) return;                          // uniform over the cluster (same blockIdx.z)
  GemmParams p = base;
  const int seg = gi.offsets[e] + row0;
  p.M = cnt - row0 < gi.rows_per_chunk ? cnt - row0 : gi.rows_per_chunk;
  p.x_row0 = seg;
  p.w_row0 = e * gi.n_rows_w;
  const int out_cols = (p.flags & GEMM_SWIGLU) ? (p.N >> 1) : p.N;
  (void)out_cols;
  p.out = reinterpret_cast<uint16_t*>(base.out) + (size_t)seg * base.ld_out;
  if (base.bias != nullptr) p.bias = reinterpret_cast<const uint16_t*>(base.bias) + (size_t)e * gi.ld_bias_e;
  uint32_t tmem_base;
  gemm_smallm_device<MPAD, BF16, 1>(tmW, tmX, p, tmem_base, KID_MOE_GROUPED);
  if ((threadIdx.x >> 5) == 1) tmem_dealloc(tmem_base, SmallMCfg<MPAD, 1>::TMEM_COLS);
}

template <int MPAD, bool BF16>
static cudaError_t launch_grouped(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p, const MoeGroupInfo& gi,
                                  int nsplit, int n_tiles, int nz, cudaStream_t stream) {
  using Cfg = SmallMCfg<MPAD, 1>;
  auto kern = moe_grouped_gemm_kernel<MPAD, BF16>;
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
  return cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p, gi);
}

}  // namespace fb

using namespace fb;

extern "C" int fb_moe_plan(const int* idx, int T, int topk, int first, int n_local, int* counts, int* offsets, int* pos,
                           int* total_rows, int pad, void* stream) {
  if (n_local <= 0 || n_local > 1024 || T <= 0) return -1;
  static const bool warp_plan = [] { const char* e = getenv("FB_MOE_PLAN_WARP"); return !(e && e[0] == '0'); }();
  if (warp_plan && T * topk <= 4096 && ((T * topk + 31) / 32) * n_local <= 8192) {
    launch_k(moe_plan_warp_kernel, dim3(1), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream), 0, idx, T * topk, first, n_local, counts, offsets, pos, total_rows, pad);
    return (int)cudaGetLastError();
  }
  if (T * topk <= 4096) {
    launch_k(moe_plan_small_kernel, dim3(1), dim3(1024), 0, reinterpret_cast<cudaStream_t>(stream), 0, idx, T * topk, first, n_local, counts, offsets, pos, total_rows, pad);
    return (int)cudaGetLastError();
  }
  int threads = 32;
  while (threads < n_local) threads <<= 1;
  if (threads < 256) threads = 256;
  launch_k(moe_plan_kernel, dim3(1), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream), 0, idx, T, topk, first, n_local, counts, offsets, pos, total_rows, pad);
  return (int)cudaGetLastError();
}

extern "C" int fb_moe_gather(const void* x, const int* pos, void* xs, int T, int topk, int H, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  launch_k(moe_gather_kernel, dim3(T * topk), dim3(128), 0, reinterpret_cast<cudaStream_t>(stream), 0, (const uint16_t*)x, pos, (uint16_t*)xs, T, topk, H);
  return (int)cudaGetLastError();
}

extern "C" int fb_moe_combine(const void* ys, const int* pos, const float* w, const void* add, void* out, int T, int topk, int H,
                              int dtype, void* stream) {
  if (T <= 0) return 0;
  if (H % 8 != 0) return -1;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) launch_k(moe_combine_kernel<true>, dim3(T), dim3(256), 0, s, 0, (const uint16_t*)ys, pos, w, (const uint16_t*)add, (uint16_t*)out, topk, H);
  else launch_k(moe_combine_kernel<false>, dim3(T), dim3(256), 0, s, 0, (const uint16_t*)ys, pos, w, (const uint16_t*)add, (uint16_t*)out, topk, H);
  return (int)cudaGetLastError();
}

// Grouped Y_e = X_e W_e^T over the sorted buffer.  Xs: [rows_cap, K] sorted rows; W: stacked [E_local * N, K]; out: [rows_cap, N or N/2].
// max_rows_per_expert bounds the chunk count (T for decode: every token could pick the same expert).
extern "C" int fb_moe_grouped_gemm(const void* Xs, const void* W, void* out, const void* bias, const int* counts, const int* offsets,
                                   int rows_cap, int E_local, int N, int K, int ld_out, int max_rows_per_expert, int dtype, int flags,
                                   int total_rows, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (E_local <= 0 || rows_cap <= 0) return 0;
  if (K % 64 != 0 || N % 128 != 0 || (dtype != 0 && dtype != 1)) return -1;
  const bool bf16 = dtype == 1;
  // rows per chunk: low 16 bits of max_rows_per_expert = most rows an expert can get, high 16 bits = chunk size hint (0: auto)
  const int hint = max_rows_per_expert >> 16;
  max_rows_per_expert &= 0xFFFF;
  int mpad = max_rows_per_expert <= 16 ? 16 : max_rows_per_expert <= 32 ? 32 : max_rows_per_expert <= 64 ? 64 : 128;
  if (hint == 16 || hint == 32 || hint == 64 || hint == 128) mpad = hint < mpad ? hint : mpad;
  const int chunks = (max_rows_per_expert + mpad - 1) / mpad;
  GemmParams p;
  p.out = out; p.bias = bias; p.residual = nullptr;
  p.M = 0; p.N = N; p.K = K; p.ld_out = ld_out; p.ld_res = 0;
  p.kb_total = K / 64; p.flags = flags;
  p.scatter_tp = 0; p.scatter_rows = 1; p.scatter_rank = 0; p.w_row0 = 0; p.x_row0 = 0;
  for (int i = 0; i < 8; ++i) p.scatter_out[i] = nullptr;
  const int n_tiles = N / 128;
  // k split: keep clusters small, experts already provide parallelism
  int nsplit = 1;
  while (nsplit < 4 && n_tiles * E_local * nsplit < 148 && (p.kb_total / (nsplit * 2)) >= 8) nsplit *= 2;
  p.kb_per_split = (p.kb_total + nsplit - 1) / nsplit;
  p.idesc = make_idesc(bf16 ? 1 : 0, bf16 ? 1 : 0, 0, 0, 128, mpad);
  MoeGroupInfo gi;
  gi.counts = counts; gi.offsets = offsets; gi.rows_per_chunk = mpad; gi.chunks = chunks; gi.n_rows_w = N; gi.out_stride_e = 0;
  gi.ld_bias_e = N;
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, W, (uint64_t)E_local * N, K, K, 128, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmX, Xs, rows_cap, K, K, mpad, 64, 2, 3)) return -2;
  int nz = E_local * chunks;
  gi.n_local = E_local; gi.compact = 0;
  if (total_rows > 0) {               // upper bound of the routed rows: one grid slot per existing row chunk
    const int bound = E_local + (total_rows + mpad - 1) / mpad;
    if (bound < nz) { nz = bound; gi.compact = 1; }
  }
  if (nz > 65535) return -1;
#define FB_MG(MP)                                                                                              \
  return (int)(bf16 ? launch_grouped<MP, true>(tmW, tmX, p, gi, nsplit, n_tiles, nz, stream)                    \
                    : launch_grouped<MP, false>(tmW, tmX, p, gi, nsplit, n_tiles, nz, stream));
  switch (mpad) {
    case 16: FB_MG(16)
    case 32: FB_MG(32)
    case 64: FB_MG(64)
    default: FB_MG(128)
  }
#undef FB_MG
}
