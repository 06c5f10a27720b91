// Absorbed multi-head latent attention (MLA) decode for sm_100a over a paged latent cache.
//
// Cache entry per token: 512 compressed-KV dims followed by 64 rotary key dims (576 x 16 bit); page length 128.
// Query per head: q_nope already multiplied by W_UK (512 dims) followed by the rotated q_pe (64 dims).
//     S^T[128 tokens x N heads] = Lat_page[128 x 576] * Q^T            9 column tiles of 64, K-major, SW128
//     O^T[512 dims   x N heads] = Lat_page[:, :512]^T * P^T             4 row blocks of 128 dims, A read MN-major
// The latent page is both K and V: it is loaded ONCE into nine 16 KB tiles, each with its own full/empty barrier, so the
// next page streams in tile by tile while the current page's softmax and PV products still run (one CTA per SM, 144 KB of
// page + 36 KB of queries).  A work item is a run of consecutive pages of one request and one group of <= 32 heads; the
// running softmax keeps (max, sum) per head across the run and rescales the TMEM accumulator when a maximum moves, so the
// un-normalised partial output is written once per item.  A combine kernel merges the items of a request.
//
// Reference: MergeMLAPaged / FastllmCudaMLAPaged -> FlashInfer BatchMLAPagedAttention<512, 64>, one request per call
// (src/devices/cuda/attention/fastllm-attention.cu:3619-3727); the absorb GEMMs stay outside (src/models/deepseekv2.cpp:283-697).
#include "ptx.cuh"
#include "launch.h"
#include "tmap.h"

FB_DEFINE_ERROR_API(attn_mla)

namespace fb {

constexpr int KID_MLA = 12;
constexpr int ML_PAGE = 128;
constexpr int ML_LORA = 512;
constexpr int ML_DQK = 576;
constexpr int ML_TILES = 9;                       // 64-column tiles of the latent page
constexpr int ML_N = 32;                          // MMA N: heads per item (padded)
constexpr int ML_TILE_BYTES = ML_PAGE * 64 * 2;   // 16 KB
constexpr int ML_QTILE_BYTES = ML_N * 64 * 2;     // 4 KB
constexpr int ML_P_BYTES = ML_N * ML_PAGE * 2;    // 8 KB
constexpr int ML_SMEM = ML_TILES * (ML_TILE_BYTES + ML_QTILE_BYTES) + ML_P_BYTES + 2048 /*barriers, reductions*/ + 1024 /*align*/;
constexpr int ML_TMEM_COLS = 256;                 // S: [0,32)  O blocks: [64 + 32*blk, +32)

struct MlaParams {
  const int* work;          // [n_work][4] = (request, first page, page count, head group)
  const int* n_work;
  const int* page_table; int max_pages;
  const int* seq_lens;
  float* part_o;            // [n_work_cap][ML_N][512]
  float* part_ml;           // [n_work_cap][ML_N][2]
  int H, B, max_items;
  float scale_log2;
  uint32_t idesc_s, idesc_o;
};

// ---- plan: one item per (request, run of pages, head group); also the per-request item ranges for the combine ----
// item_range: [B][2] = (first item, item count) of the request's head group 0; groups follow each other per run.
__global__ void mla_plan_kernel(const int* __restrict__ seq_lens, int B, int n_groups, int target_items, int* __restrict__ work,
                                int* __restrict__ n_work, int* __restrict__ item_range, int max_items) {
  __shared__ int offs[1025];
  __shared__ int s_ppi;
  pdl_launch_dependents();
  pdl_wait();
  const int t = threadIdx.x;
  int np = 0;
  if (t < B) np = (seq_lens[t] + ML_PAGE - 1) / ML_PAGE;
  offs[t + 1] = np;
  if (t == 0) offs[0] = 0;
  __syncthreads();
  for (int d = 1; d < blockDim.x; d <<= 1) {
    int v = 0;
    if (t >= d) v = offs[t + 1 - d];
    __syncthreads();
    if (t >= d) offs[t + 1] += v;
    __syncthreads();
  }
  if (t == 0) {
    const int total_pages = offs[blockDim.x];
    int ppi = (total_pages * n_groups + target_items - 1) / target_items;      // pages per item
    s_ppi = ppi < 1 ? 1 : ppi;
  }
  __syncthreads();
  const int ppi = s_ppi;
  // runs per request, exclusive scan over requests (reuse offs)
  const int runs = t < B ? (np + ppi - 1) / ppi : 0;
  __syncthreads();
  offs[t + 1] = runs;
  if (t == 0) offs[0] = 0;
  __syncthreads();
  for (int d = 1; d < blockDim.x; d <<= 1) {
    int v = 0;
    if (t >= d) v = offs[t + 1 - d];
    __syncthreads();
    if (t >= d) offs[t + 1] += v;
    __syncthreads();
  }
  if (t < B) {
    const int first = offs[t] * n_groups;
    item_range[2 * t] = first;
    item_range[2 * t + 1] = runs;
    for (int r = 0; r < runs; ++r)
      for (int g = 0; g < n_groups; ++g) {
        const int it = first + r * n_groups + g;
        if (it < max_items) {
          work[4 * it] = t;
          work[4 * it + 1] = r * ppi;
          work[4 * it + 2] = (np - r * ppi) < ppi ? (np - r * ppi) : ppi;
          work[4 * it + 3] = g;
        }
      }
  }
  if (t == 0) { const int total = offs[blockDim.x] * n_groups; *n_work = total < max_items ? total : max_items; }
}

// Reads and validates one work item; every warp role uses this, so a rejected item is rejected by all of them alike.
__device__ __forceinline__ bool mla_item(const MlaParams& p, int w, int& b, int& p0, int& cnt, int& hg) {
  b = p.work[4 * w]; p0 = p.work[4 * w + 1]; cnt = p.work[4 * w + 2]; hg = p.work[4 * w + 3];
  if ((unsigned)b >= (unsigned)p.B || p0 < 0 || cnt < 0 || p0 + cnt > p.max_pages || hg < 0 || hg * ML_N >= p.H) {
    b = 0; p0 = 0; cnt = 0; hg = 0;
    return false;
  }
  return true;
}

template <bool BF16, int GP>
__global__ void __launch_bounds__(192, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmLat, const __grid_constant__ CUtensorMap tmQ, const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* lat = smem;                                         // 9 tiles [128 tokens x 64 cols]
  uint8_t* qs = lat + ML_TILES * ML_TILE_BYTES;                // 9 tiles [32 heads x 64 cols]
  uint8_t* p_smem = qs + ML_TILES * ML_QTILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + ML_P_BYTES);
  uint64_t* full = bars;                   // [9] tile landed
  uint64_t* empty = bars + ML_TILES;       // [9] tile consumed by its last MMA
  uint64_t* q_full = bars + 2 * ML_TILES;
  uint64_t* q_empty = q_full + 1;
  uint64_t* s_full = q_full + 2;
  uint64_t* p_ready = q_full + 3;
  uint64_t* o_full = q_full + 4;
  uint64_t* o_read = q_full + 5;           // epilogue has read O of the finished item
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 6);
  float* red_max = reinterpret_cast<float*>(tmem_slot + 4);    // [4 warps][32]
  float* red_sum = red_max + 128;                                // [4 warps][32]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bool dead = false;
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int j = 0; j < ML_TILES; ++j) { mbar_init(&full[j], 1); mbar_init(&empty[j], 1); }
    mbar_init(q_full, 1); mbar_init(q_empty, 1); mbar_init(s_full, 1); mbar_init(p_ready, 128); mbar_init(o_full, 1);
    mbar_init(o_read, 128);
    mbar_init_fence();
    tma_prefetch_desc(&tmLat); tma_prefetch_desc(&tmQ);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, ML_TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_s = *tmem_slot;
  const uint32_t tmem_o = tmem_s + 64;
  pdl_wait();
  int n_items = *p.n_work;
  if (n_items < 0) n_items = 0;
  if (n_items > p.max_items) n_items = p.max_items;

  if (warp == 0) {
    if (elect_one()) {
      int pi = 0, ii = 0;                  // CTA-local page and item counters (barrier phases)
      for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++ii) {
        int b, p0, cnt, hg;
        if (!mla_item(p, w, b, p0, cnt, hg)) report_error(ERR_BAD_ARG, KID_MLA, 20);
        if (!mbar_wait(q_empty, ((uint32_t)ii & 1u) ^ 1u, dead, KID_MLA, 1)) break;
        mbar_expect_tx(q_full, ML_TILES * ML_QTILE_BYTES);
        for (int j = 0; j < ML_TILES; ++j) tma_load_2d(qs + j * ML_QTILE_BYTES, &tmQ, q_full, j * 64, b * p.H + hg * ML_N);
        for (int i = 0; i < cnt; ++i, ++pi) {
          const int page = p.page_table[(size_t)b * p.max_pages + p0 + i];
          for (int j = 0; j < ML_TILES; ++j) {
            if (!mbar_wait(&empty[j], ((uint32_t)pi & 1u) ^ 1u, dead, KID_MLA, 2)) break;
            mbar_expect_tx(&full[j], ML_TILE_BYTES);
            tma_load_2d(lat + j * ML_TILE_BYTES, &tmLat, &full[j], j * 64, page * ML_PAGE);
          }
          if (dead) break;
        }
        if (dead) break;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      int pi = 0, ii = 0;
      for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++ii) {
        int b, p0, cnt, hg;
        mla_item(p, w, b, p0, cnt, hg);
        if (!mbar_wait(q_full, (uint32_t)ii & 1u, dead, KID_MLA, 3)) break;
        if (cnt == 0) umma_commit(q_empty);                  // rejected item: hand the query buffer straight back
        for (int i = 0; i < cnt; ++i, ++pi) {
          const uint32_t ph = (uint32_t)pi & 1u;
          // ---- S^T = Lat * Q^T over 9 column tiles ----
          for (int j = 0; j < ML_TILES; ++j) {
            if (!mbar_wait(&full[j], ph, dead, KID_MLA, 4)) break;
            tc_fence_after_sync();
            const uint32_t a0 = smem_u32(lat + j * ML_TILE_BYTES), b0 = smem_u32(qs + j * ML_QTILE_BYTES);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16(tmem_s, make_smem_desc(a0 + k * 32, 16, 1024, SWZ_128B), make_smem_desc(b0 + k * 32, 16, 1024, SWZ_128B),
                       p.idesc_s, (j | k) != 0 ? 1u : 0u);
          }
          if (dead) break;
          umma_commit(s_full);
          umma_commit(&empty[ML_TILES - 1]);                 // the rotary tile is not part of V
          if (i == cnt - 1) umma_commit(q_empty);            // queries are free once the item's last S product is done
          if (!mbar_wait(p_ready, ph, dead, KID_MLA, 5)) break;
          if (i == 0 && ii > 0 && !mbar_wait(o_read, ((uint32_t)ii & 1u) ^ 1u, dead, KID_MLA, 6)) break;
          tc_fence_after_sync();
          // ---- O^T[blk] (+)= V_blk^T * P^T, V_blk = latent columns [128 blk, +128) = tiles 2 blk, 2 blk + 1 ----
          for (int blk = 0; blk < 4; ++blk) {
            const uint32_t vb = smem_u32(lat + 2 * blk * ML_TILE_BYTES);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_f16(tmem_o + blk * ML_N, make_smem_desc(vb + k * 2048, ML_TILE_BYTES, 1024, SWZ_128B),
                       make_smem_desc(smem_u32(p_smem) + k * 1024, 512, 128, SWZ_NONE), p.idesc_o, (i | k) != 0 ? 1u : 0u);
            umma_commit(&empty[2 * blk]);
            umma_commit(&empty[2 * blk + 1]);
          }
          umma_commit(o_full);
        }
        if (dead) break;
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    const int t = q * 32 + lane;                   // token within the page (softmax) / dim within a 128-block (epilogue)
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    int pi = 0, ii = 0;
    for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++ii) {
      int b, p0, cnt, hg;
      mla_item(p, w, b, p0, cnt, hg);
      const int seq = p.seq_lens[b];
      const int nh = min(GP, p.H - hg * ML_N);     // real heads in this group
      float m_run[GP], l_part[GP];
#pragma unroll
      for (int h = 0; h < GP; ++h) { m_run[h] = -INFINITY; l_part[h] = 0.f; }
      for (int i = 0; i < cnt; ++i, ++pi) {
        const uint32_t ph = (uint32_t)pi & 1u;
        const bool valid = (p0 + i) * ML_PAGE + t < seq;
        mbar_wait(s_full, ph, dead, KID_MLA, 7);
        tc_fence_after_sync();
        uint32_t r[32];
        tmem_ld_32x32b_x32(tmem_s + lane_off, r);
        tmem_ld_wait();
        float sv[GP];
#pragma unroll
        for (int h = 0; h < GP; ++h) sv[h] = (valid && h < nh) ? __uint_as_float(r[h]) * p.scale_log2 : -INFINITY;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          float m = sv[h];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
          if (lane == 0) red_max[q * 32 + h] = m;
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        float fac[GP];
        bool moved = false;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          const float pm = fmaxf(fmaxf(red_max[h], red_max[32 + h]), fmaxf(red_max[64 + h], red_max[96 + h]));
          const float mn = fmaxf(m_run[h], pm);
          fac[h] = (m_run[h] == -INFINITY) ? 0.f : exp2f(m_run[h] - mn);
          moved = moved || (mn != m_run[h] && m_run[h] != -INFINITY);
          m_run[h] = mn;
        }
        if (i > 0) {
          // the previous page's PV products must be complete before O is rescaled or P overwritten
          mbar_wait(o_full, ph ^ 1u, dead, KID_MLA, 8);
          tc_fence_after_sync();
          if (moved) {                                   // same decision in every thread: the maxima are CTA-wide
#pragma unroll 1
            for (int blk = 0; blk < 4; ++blk) {
              uint32_t o[32];
              tmem_ld_32x32b_x32(tmem_o + blk * ML_N + lane_off, o);
              tmem_ld_wait();
#pragma unroll
              for (int h = 0; h < GP; ++h) o[h] = __float_as_uint(__uint_as_float(o[h]) * fac[h]);
              tmem_st_32x32b_x32(tmem_o + blk * ML_N + lane_off, o);
            }
            tmem_st_wait();
          }
        }
        // P^T[n][t], K-major core matrices: ((t/8) * (N/8) + n/8) * 128 + (n%8) * 16 + (t%8) * 2 bytes
        uint8_t* pb = p_smem + (t >> 3) * (ML_N / 8) * 128 + (t & 7) * 2;
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          float pv = 0.f;
          if (h < nh && valid) pv = exp2f(sv[h] - m_run[h]);
          const uint16_t bits = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(pv)) : __half_as_ushort(__float2half_rn(pv));
          *reinterpret_cast<uint16_t*>(pb + (h >> 3) * 128 + (h & 7) * 16) = bits;
          const float seen = BF16 ? __bfloat162float(__ushort_as_bfloat16(bits)) : __half2float(__ushort_as_half(bits));
          l_part[h] = l_part[h] * fac[h] + seen;
        }
        if (GP < ML_N) {
#pragma unroll
          for (int h = GP; h < ML_N; ++h) *reinterpret_cast<uint16_t*>(pb + (h >> 3) * 128 + (h & 7) * 16) = 0;
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        mbar_arrive(p_ready);
      }
      // ---- item epilogue ----
      if (cnt > 0) {
        mbar_wait(o_full, (uint32_t)(pi - 1) & 1u, dead, KID_MLA, 9);
        tc_fence_after_sync();
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          float s = l_part[h];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
          if (lane == 0) red_sum[q * 32 + h] = s;
        }
        float* po = p.part_o + (size_t)w * ML_N * ML_LORA;
#pragma unroll 1
        for (int blk = 0; blk < 4; ++blk) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_o + blk * ML_N + lane_off, o);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < GP; ++h)
            if (h < nh) po[(size_t)h * ML_LORA + blk * 128 + t] = __uint_as_float(o[h]);
        }
        tc_fence_before_sync();
        mbar_arrive(o_read);
        asm volatile("bar.sync 1, 128;\n" ::: "memory");     // every thread is past its last read of red_max
      } else {
        mbar_arrive(o_read);
      }
      // running maxima live in registers indexed at compile time: publish them through shared memory
#pragma unroll
      for (int h = 0; h < GP; ++h)
        if (t == h) red_max[h] = m_run[h];
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      if (cnt > 0 && t < nh) {
        p.part_ml[((size_t)w * ML_N + t) * 2] = red_max[t];
        p.part_ml[((size_t)w * ML_N + t) * 2 + 1] = red_sum[t] + red_sum[32 + t] + red_sum[64 + t] + red_sum[96 + t];
      }
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_s, ML_TMEM_COLS);
}

// one CTA per (request, head): merges the request's items of that head's group; 128 threads x 4 dims
template <bool BF16>
__global__ void mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ item_range,
                                   uint16_t* __restrict__ out, int H, int n_groups) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x, h = blockIdx.y, t = threadIdx.x;
  const int g = h / ML_N, hl = h - g * ML_N;
  const int first = item_range[2 * b], runs = item_range[2 * b + 1];
  float M = -INFINITY;
  for (int r = 0; r < runs; ++r) M = fmaxf(M, part_ml[((size_t)(first + r * n_groups + g) * ML_N + hl) * 2]);
  float L = 0.f;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int r = 0; r < runs; ++r) {
    const size_t it = (size_t)(first + r * n_groups + g);
    const float wgt = exp2f(part_ml[(it * ML_N + hl) * 2] - M);
    L += part_ml[(it * ML_N + hl) * 2 + 1] * wgt;
    const float4 o = *reinterpret_cast<const float4*>(&part_o[(it * ML_N + hl) * ML_LORA + t * 4]);
    acc.x += o.x * wgt; acc.y += o.y * wgt; acc.z += o.z * wgt; acc.w += o.w * wgt;
  }
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  uint2 pk;
  pk.x = pack_16<BF16>(acc.x * inv, acc.y * inv);
  pk.y = pack_16<BF16>(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(&out[((size_t)b * H + h) * ML_LORA + t * 4]) = pk;
}

}  // namespace fb

using namespace fb;

// q: [B, H, 576] (q_lat | q_pe), lat_pool: [num_slots, 576], out: [B, H, 512]; all 16-bit (dtype 0 = fp16, 1 = bf16).
// Scratch: work [4 * max_items] ints, n_work [1], item_range [2 * B], part_o [max_items * 32 * 512] floats,
// part_ml [max_items * 32 * 2] floats, with max_items >= (B * max_pages) * ceil(H / 32) (one page per item, worst case).
extern "C" int fb_mla_decode(const void* q, const void* lat_pool, void* out, const int* page_table, const int* seq_lens, int* work,
                             int* n_work, int* item_range, float* part_o, float* part_ml, int B, int H, long long num_slots,
                             int max_pages, int max_items, float scale, int dtype, void* stream_) {
  if (B <= 0) return 0;
  if (B > 1024 || H <= 0 || max_pages <= 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const int n_groups = (H + ML_N - 1) / ML_N;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap tmLat, tmQ;
  if (!make_tmap_2d(&tmLat, lat_pool, (uint64_t)num_slots, ML_DQK, ML_DQK, ML_PAGE, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmQ, q, (uint64_t)B * H, ML_DQK, ML_DQK, ML_N, 64, 2, 3)) return -2;
  int threads = 32;
  while (threads < B) threads <<= 1;
  launch_k(mla_plan_kernel, dim3(1), dim3(threads), 0, stream, 0, seq_lens, B, n_groups, 2 * sm_count, work, n_work, item_range, max_items);
  MlaParams p;
  p.work = work; p.n_work = n_work; p.page_table = page_table; p.max_pages = max_pages; p.seq_lens = seq_lens;
  p.part_o = part_o; p.part_ml = part_ml; p.H = H; p.B = B; p.max_items = max_items;
  p.scale_log2 = scale * 1.4426950408889634f;
  const uint32_t f = dtype == 1 ? 1u : 0u;
  p.idesc_s = make_idesc(f, f, 0, 0, 128, ML_N);
  p.idesc_o = make_idesc(f, f, 1, 0, 128, ML_N);
  const int gp = (H <= 16) ? 16 : 32;
#define FB_MLA_LAUNCH(BF, GPV)                                                                                          \
  {                                                                                                                     \
    static DeviceOnce cfg;                                                                                            \
    if (cfg.need()) { cudaFuncSetAttribute(mla_decode_kernel<BF, GPV>, cudaFuncAttributeMaxDynamicSharedMemorySize, ML_SMEM); } \
    launch_k<PDL_ATTN>(mla_decode_kernel<BF, GPV>, dim3(sm_count), dim3(192), ML_SMEM, stream, 0, tmLat, tmQ, p);        \
    launch_k<PDL_COMBINE>(mla_combine_kernel<BF>, dim3(B, H), dim3(128), 0, stream, 0, part_o, part_ml, item_range, (uint16_t*)out, H, n_groups); \
  }
  if (dtype == 1) { if (gp == 16) FB_MLA_LAUNCH(true, 16) else FB_MLA_LAUNCH(true, 32) }
  else { if (gp == 16) FB_MLA_LAUNCH(false, 16) else FB_MLA_LAUNCH(false, 32) }
#undef FB_MLA_LAUNCH
  return (int)cudaGetLastError();
}
