// Paged GQA decode attention for sm_100a (head_dim 128, page length 128, up to 16 query heads per KV head).
//
// One KV page (128 tokens of one KV head) is exactly one UMMA tile:
//     S^T[128 tokens x G] = K_page[128 x 128] * Q^T        (A = K page, K-major, straight from the page pool by TMA)
//     O^T[128 dims   x G] = V_page^T[128 x 128] * P^T      (A = V page read MN-major, B = P^T written by the softmax warps)
// so the tensor core runs full 128-row MMAs although only G (<= 16) query rows exist.  Work items are
// (request, page) pairs listed by a tiny plan kernel; CTAs stride over items x KV heads with a 3-stage
// TMA ring, write un-normalised partial outputs + (max, sum) per item to scratch, and a combine kernel
// merges the partials.  This is the split-KV structure of the reference's native paged fallback
// (src/devices/cuda/attention/paged/fastllm-paged-attention-native.cu:1050-1562) mapped onto tcgen05;
// the reference's main path is FlashInfer's mma.sync prefill kernel (fastllm-attention.cu:3032-3600).
//
// Page pools must be zero-initialised: the unused tail of a request's last page is multiplied by P = 0.
#include "ptx.cuh"
#include "launch.h"
#include "tmap.h"

FB_DEFINE_ERROR_API(attn_decode)

namespace fb {

constexpr int KID_ATTN_DECODE = 10;
constexpr int AD_D = 128;
constexpr int AD_PAGE = 128;
constexpr int AD_NPAD = 16;
constexpr int AD_K_BYTES = AD_PAGE * AD_D * 2;     // 32 KB
constexpr int AD_Q_BYTES = AD_NPAD * AD_D * 2;     // 4 KB
constexpr int AD_STAGE_BYTES = 2 * AD_K_BYTES + AD_Q_BYTES;   // K, V, Q
constexpr int AD_P_BYTES = AD_NPAD * AD_PAGE * 2;  // 4 KB
constexpr int ad_smem_bytes(int stages) { return stages * AD_STAGE_BYTES + AD_P_BYTES + 1024 /*barriers+red*/ + 1024 /*align*/; }

struct AttnDecodeParams {
  const int* work;        // [n_work][2] = (request, page index within the request)
  const int* n_work;      // device scalar
  const int* page_table;  // [B, max_pages]
  const int* seq_lens;    // [B]
  float* part_o;          // [B, Hkv, max_splits, G, D]
  float* part_ml;         // [B, Hkv, max_splits, G, 2]
  int max_pages, max_splits, Hq, Hkv, G;
  int B, max_items;       // bounds for validating work items read from device memory
  float scale_log2;       // softmax scale * log2(e)
  uint32_t idesc_s, idesc_o;
  // fused combine: the CTA that finishes the last split of a (request, KV head) merges the partials and writes `out`.
  // counters: [B * Hkv] ints, zero before the first launch; the merging CTA sets its counter back to zero.
  int* counters;          // null: partials only (a separate combine kernel follows)
  uint16_t* out; int ld_out;
  int clip;               // 1: the last page of a request is loaded in 32-token boxes, only as far as it is filled
  // attention variants (reference: include/models/qwen3_cuda_common.h:1262-1263, src/models/gpt_oss.cpp)
  int window;             // > 0: sliding window, the query at position seq-1 sees keys at positions >= seq - window
  float softcap;          // > 0: logits become softcap * tanh(logit / softcap) before the softmax (Gemma-2)
  float scale;            // plain softmax scale (scale_log2 / log2(e)), used with softcap
};

// ---- plan: flatten (request, page) pairs ---------------------------------------------------------
__global__ void attn_decode_plan_kernel(const int* __restrict__ seq_lens, int B, int* __restrict__ work, int* __restrict__ n_work,
                                        int max_items, int window = 0) {
  __shared__ int offs[1025];
  pdl_launch_dependents();
  pdl_wait();
  // single CTA; B <= 1024
  const int t = threadIdx.x;
  int np = 0, first = 0;
  if (t < B) {
    const int seq = seq_lens[t];
    np = (seq + AD_PAGE - 1) / AD_PAGE;
    if (window > 0 && seq > window) first = (seq - window) / AD_PAGE;     // pages wholly before the window are not listed
    np -= first;
  }
  offs[t + 1] = np;
  if (t == 0) offs[0] = 0;
  __syncthreads();
  // inclusive scan (Hillis-Steele) over blockDim entries
  for (int d = 1; d < blockDim.x; d <<= 1) {
    int v = 0;
    if (t >= d) v = offs[t + 1 - d];
    __syncthreads();
    if (t >= d) offs[t + 1] += v;
    __syncthreads();
  }
  if (t < B) {
    const int base = offs[t];
    for (int i = 0; i < np; ++i)
      if (base + i < max_items) { work[2 * (base + i)] = t; work[2 * (base + i) + 1] = first + i; }
  }
  if (t == 0) { const int total = offs[B]; *n_work = total < max_items ? total : max_items; }
}

// One raw page (128 tokens x 128 e4m3 bytes, row-major) -> the fp16 operand tile: two half tiles of 64 dims (16 KB each), a row
// of a half tile is 128 bytes and its 16-byte chunk j sits at chunk position j ^ (row & 7) (the 128-byte swizzle TMA applies).
// 128 threads; eight consecutive threads read one raw row, so the loads are conflict-free.
__device__ __forceinline__ void kv8_convert_page(const uint8_t* __restrict__ raw, uint8_t* __restrict__ tile, int ctid) {
  uint4 r[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) r[i] = *reinterpret_cast<const uint4*>(raw + (size_t)(ctid + i * 128) * 16);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = ctid + i * 128, row = idx >> 3, c16 = idx & 7;       // c16: 16 dims of the row
    const uint32_t w[4] = {r[i].x, r[i].y, r[i].z, r[i].w};
    uint32_t h[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h[2 * j]) : "h"((unsigned short)(w[j] & 0xFFFFu)));
      asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h[2 * j + 1]) : "h"((unsigned short)(w[j] >> 16)));
    }
    uint8_t* dst = tile + (c16 >> 2) * (AD_K_BYTES / 2) + row * 128;
    const int cc = (c16 & 3) * 2, sw = row & 7;
    *reinterpret_cast<uint4*>(dst + ((cc ^ sw) << 4)) = make_uint4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<uint4*>(dst + (((cc + 1) ^ sw) << 4)) = make_uint4(h[4], h[5], h[6], h[7]);
  }
}

// GP = query heads per KV head rounded up to a power of two: the softmax warps only touch GP of the 16 MMA columns.
//
// KV8: the page pools hold unscaled e4m3 bytes (half the cache traffic).  TMA brings a raw page (128 tokens x 128 bytes) into
// a staging buffer, four extra warps turn it into the 16-bit operand tile -- written in exactly the 128-byte-swizzled layout
// the 16-bit TMA load would have produced, so the MMA descriptors, the softmax and the epilogue are the same code -- and the
// next raw page is already in flight while the current one is converted and multiplied.  e4m3 converts exactly to fp16
// (`cvt.rn.f16x2.e4m3x2`), so this mode computes in fp16: the caller passes fp16 queries.
//
// KV8 == 2: the e4m3 pages go to the tensor core as they are (`kind::f8f6f4`): K page = A operand K-major, V page = A operand
// read MN-major, no conversion and no 16-bit operand tiles (a stage is 36 KB).  The other operand of each product must be
// 8-bit too; to keep 16-bit-class accuracy it is split in two e4m3 terms, x = hi + lo / 16: the queries by a small kernel
// beforehand (Qa, Qb), the probabilities (scaled by 256 so that small ones stay representable) by the softmax warps
// (Pa, Pb).  Each product runs once per term into its own TMEM accumulator: S = Sa + Sb / 16, O = (Oa + Ob / 16) / 256.
template <bool BF16, int AD_STAGES, int GP, int KV8 = 0>
__global__ void __launch_bounds__(KV8 == 1 ? 320 : 192, KV8 == 1 ? 2 : (KV8 == 2 ? 4 : (AD_STAGES == 1 ? 3 : 1)))
attn_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK32,
                   const __grid_constant__ CUtensorMap tmV32, const AttnDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int K8_BYTES = AD_PAGE * AD_D;                           // one e4m3 page
  constexpr int Q8_BYTES = AD_NPAD * AD_D;                           // one e4m3 query tile (16 heads x 128)
  constexpr int STAGE_B = KV8 == 2 ? 2 * K8_BYTES + 2 * Q8_BYTES : AD_STAGE_BYTES;      // KV8 == 2: K8, V8, Qa, Qb
  uint8_t* p_smem = smem + AD_STAGES * STAGE_B;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + AD_P_BYTES);
  uint64_t* full_k = bars;                  // [STAGES]  K + Q landed
  uint64_t* full_v = bars + AD_STAGES;      // [STAGES]
  uint64_t* empty_k = bars + 2 * AD_STAGES;   // [STAGES]  K + Q consumed (S MMA done)
  uint64_t* empty_v = bars + 3 * AD_STAGES;   // [STAGES]  V consumed (PV MMA done)
  uint64_t* s_full = bars + 4 * AD_STAGES;
  uint64_t* p_ready = s_full + 1;
  uint64_t* o_full = s_full + 2;
  uint64_t* o_empty = s_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(s_full + 4);
  float* red_max = reinterpret_cast<float*>(tmem_slot + 4);      // [4 warps][16]
  float* red_sum = red_max + 64;                                  // [2 parity][4 warps][16]
  int* sh_flag = reinterpret_cast<int*>(red_sum + 128);
  // KV8: raw page staging (K then V, 16 KB each) behind the barrier block, and its four barriers
  uint64_t* raw_full_k = reinterpret_cast<uint64_t*>(sh_flag + 2);
  uint64_t* raw_full_v = raw_full_k + 1;
  uint64_t* raw_empty_k = raw_full_k + 2;
  uint64_t* raw_empty_v = raw_full_k + 3;
  uint8_t* raw_k = p_smem + AD_P_BYTES + 1024;
  uint8_t* raw_v = raw_k + AD_PAGE * AD_D;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bool dead = false;
  pdl_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < AD_STAGES; ++s) {
      // KV8: the operand tiles are completed by the 128 converter threads (plus the producer's arrival for the Q tile)
      mbar_init(&full_k[s], KV8 == 1 ? 129 : 1); mbar_init(&full_v[s], KV8 == 1 ? 128 : 1); mbar_init(&empty_k[s], 1); mbar_init(&empty_v[s], 1);
    }
    if (KV8 == 1) { mbar_init(raw_full_k, 1); mbar_init(raw_full_v, 1); mbar_init(raw_empty_k, 128); mbar_init(raw_empty_v, 128); }
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_full, 1);
    mbar_init(o_empty, 128);
    mbar_init_fence();
    tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmQ);
    if (p.clip) { tma_prefetch_desc(&tmK32); tma_prefetch_desc(&tmV32); }
  }
  if (p.clip) {
    // rows of a clipped page that are never loaded still enter the PV product with P = 0: they must be finite
    for (int s = 0; s < AD_STAGES; ++s) {
      uint4* vz = reinterpret_cast<uint4*>(smem + s * AD_STAGE_BYTES + AD_K_BYTES);
      for (int i = threadIdx.x; i < AD_K_BYTES / 16; i += blockDim.x) vz[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();
  }
  constexpr uint32_t TMEM_COLS = KV8 == 2 ? 64 : 32;
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_s = *tmem_slot;        // columns [0,16): S^T, [16,32): O^T   (KV8 == 2: Sa, Sb, Oa, Ob of 16 columns each)
  const uint32_t tmem_o = tmem_s + (KV8 == 2 ? 32 : 16);
  pdl_wait();   // everything above touches only this CTA's shared memory and TMEM
  int n_items = *p.n_work;
  if (n_items < 0) n_items = 0;
  if (n_items > p.max_items) n_items = p.max_items;   // never trust a count read from memory beyond the list's capacity
  const int total = n_items * p.Hkv;

  if (warp == 0) {
    if (elect_one()) {
      int it = 0;
      for (int w = blockIdx.x; w < total; w += gridDim.x, ++it) {
        const int item = w / p.Hkv, kvh = w - item * p.Hkv;
        int b = p.work[2 * item], pg = p.work[2 * item + 1];
        if ((unsigned)b >= (unsigned)p.B || (unsigned)pg >= (unsigned)p.max_splits || pg >= p.max_pages) {
          report_error(ERR_BAD_ARG, KID_ATTN_DECODE, 20);
          b = 0; pg = 0;
        }
        const int page = p.page_table[(size_t)b * p.max_pages + pg];
        const int s = it % AD_STAGES;
        const uint32_t ph = (uint32_t)(it / AD_STAGES) & 1u;
        if (KV8 == 2) {
          if (!mbar_wait(&empty_k[s], ph ^ 1u, dead, KID_ATTN_DECODE, 1)) break;
          uint8_t* k8 = smem + s * STAGE_B;
          mbar_expect_tx(&full_k[s], K8_BYTES + 2 * Q8_BYTES);
          tma_load_2d(k8, &tmK, &full_k[s], kvh * AD_D, page * AD_PAGE);
          tma_load_2d(k8 + 2 * K8_BYTES, &tmQ, &full_k[s], 0, b * p.Hq + kvh * p.G);                 // Qa
          tma_load_2d(k8 + 2 * K8_BYTES + Q8_BYTES, &tmK32, &full_k[s], 0, b * p.Hq + kvh * p.G);    // Qb (its map rides in the tmK32 slot)
          if (!mbar_wait(&empty_v[s], ph ^ 1u, dead, KID_ATTN_DECODE, 8)) break;
          mbar_expect_tx(&full_v[s], K8_BYTES);
          tma_load_2d(k8 + K8_BYTES, &tmV, &full_v[s], kvh * AD_D, page * AD_PAGE);
          continue;
        }
        if (KV8 == 1) {
          // raw pages first (their staging buffers free up long before the operand tiles do), then Q into the operand stage
          if (!mbar_wait(raw_empty_k, ph ^ 1u, dead, KID_ATTN_DECODE, 11)) break;
          mbar_expect_tx(raw_full_k, AD_PAGE * AD_D);
          tma_load_2d(raw_k, &tmK, raw_full_k, kvh * AD_D, page * AD_PAGE);
          if (!mbar_wait(raw_empty_v, ph ^ 1u, dead, KID_ATTN_DECODE, 12)) break;
          mbar_expect_tx(raw_full_v, AD_PAGE * AD_D);
          tma_load_2d(raw_v, &tmV, raw_full_v, kvh * AD_D, page * AD_PAGE);
          if (!mbar_wait(&empty_k[s], ph ^ 1u, dead, KID_ATTN_DECODE, 1)) break;
          uint8_t* qb8 = smem + s * AD_STAGE_BYTES + 2 * AD_K_BYTES;
          mbar_expect_tx(&full_k[s], AD_Q_BYTES);
          tma_load_2d(qb8, &tmQ, &full_k[s], 0, b * p.Hq + kvh * p.G);
          tma_load_2d(qb8 + AD_Q_BYTES / 2, &tmQ, &full_k[s], 64, b * p.Hq + kvh * p.G);
          continue;
        }
        if (!mbar_wait(&empty_k[s], ph ^ 1u, dead, KID_ATTN_DECODE, 1)) break;
        uint8_t* kb = smem + s * AD_STAGE_BYTES;
        uint8_t* vb = kb + AD_K_BYTES;
        uint8_t* qb = vb + AD_K_BYTES;
        int rows = p.seq_lens[b] - pg * AD_PAGE;
        const int nbox = (p.clip && rows < AD_PAGE) ? (rows <= 0 ? 1 : (rows + 31) >> 5) : 0;     // 0: whole page in one box
        if (nbox == 0) {
          mbar_expect_tx(&full_k[s], AD_K_BYTES + AD_Q_BYTES);
          tma_load_2d(kb, &tmK, &full_k[s], kvh * AD_D, page * AD_PAGE);
          tma_load_2d(kb + AD_K_BYTES / 2, &tmK, &full_k[s], kvh * AD_D + 64, page * AD_PAGE);
        } else {
          mbar_expect_tx(&full_k[s], nbox * 2 * 4096 + AD_Q_BYTES);
          for (int j = 0; j < nbox; ++j) {
            tma_load_2d(kb + j * 4096, &tmK32, &full_k[s], kvh * AD_D, page * AD_PAGE + j * 32);
            tma_load_2d(kb + AD_K_BYTES / 2 + j * 4096, &tmK32, &full_k[s], kvh * AD_D + 64, page * AD_PAGE + j * 32);
          }
        }
        tma_load_2d(qb, &tmQ, &full_k[s], 0, b * p.Hq + kvh * p.G);
        tma_load_2d(qb + AD_Q_BYTES / 2, &tmQ, &full_k[s], 64, b * p.Hq + kvh * p.G);
        if (!mbar_wait(&empty_v[s], ph ^ 1u, dead, KID_ATTN_DECODE, 8)) break;
        if (nbox == 0) {
          mbar_expect_tx(&full_v[s], AD_K_BYTES);
          tma_load_2d(vb, &tmV, &full_v[s], kvh * AD_D, page * AD_PAGE);
          tma_load_2d(vb + AD_K_BYTES / 2, &tmV, &full_v[s], kvh * AD_D + 64, page * AD_PAGE);
        } else {
          mbar_expect_tx(&full_v[s], nbox * 2 * 4096);
          for (int j = 0; j < nbox; ++j) {
            tma_load_2d(vb + j * 4096, &tmV32, &full_v[s], kvh * AD_D, page * AD_PAGE + j * 32);
            tma_load_2d(vb + AD_K_BYTES / 2 + j * 4096, &tmV32, &full_v[s], kvh * AD_D + 64, page * AD_PAGE + j * 32);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      int it = 0;
      for (int w = blockIdx.x; w < total; w += gridDim.x, ++it) {
        const int s = it % AD_STAGES;
        const uint32_t ph = (uint32_t)(it / AD_STAGES) & 1u;
        const uint32_t iph = (uint32_t)it & 1u;
        const uint32_t kb = smem_u32(smem + s * AD_STAGE_BYTES);
        const uint32_t vb = kb + AD_K_BYTES, qb = vb + AD_K_BYTES;
        if (KV8 == 2) {
          const uint32_t k8 = smem_u32(smem + s * STAGE_B), v8 = k8 + K8_BYTES, qa = v8 + K8_BYTES, qb8 = qa + Q8_BYTES;
          if (!mbar_wait(&full_k[s], ph, dead, KID_ATTN_DECODE, 2)) break;
          tc_fence_after_sync();
          // Sa = K8 * Qa^T, Sb = K8 * Qb^T: rows of 128 bytes, 128-byte swizzle, 32 dims per instruction
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8(tmem_s, make_smem_desc(k8 + k * 32, 16, 1024, SWZ_128B), make_smem_desc(qa + k * 32, 16, 1024, SWZ_128B), p.idesc_s, k != 0 ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8(tmem_s + 16, make_smem_desc(k8 + k * 32, 16, 1024, SWZ_128B), make_smem_desc(qb8 + k * 32, 16, 1024, SWZ_128B), p.idesc_s, k != 0 ? 1u : 0u);
          umma_commit(s_full);
          umma_commit(&empty_k[s]);
          if (!mbar_wait(p_ready, iph, dead, KID_ATTN_DECODE, 3)) break;
          if (!mbar_wait(&full_v[s], ph, dead, KID_ATTN_DECODE, 4)) break;
          if (it > 0 && !mbar_wait(o_empty, iph ^ 1u, dead, KID_ATTN_DECODE, 5)) break;
          tc_fence_after_sync();
          // Oa = V8^T * Pa^T, Ob = V8^T * Pb^T: the V page read MN-major (dims contiguous, one 128-byte atom wide), 32 tokens per
          // instruction; P^T [16 x 128 tokens] bytes in the un-swizzled core-matrix layout (8 heads x 16 tokens per core matrix)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8(tmem_o, make_smem_desc(v8 + k * 4096, 16, 1024, SWZ_128B), make_smem_desc(smem_u32(p_smem) + k * 512, 256, 128, SWZ_NONE), p.idesc_o, k != 0 ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f8(tmem_o + 16, make_smem_desc(v8 + k * 4096, 16, 1024, SWZ_128B), make_smem_desc(smem_u32(p_smem) + 2048 + k * 512, 256, 128, SWZ_NONE), p.idesc_o, k != 0 ? 1u : 0u);
          umma_commit(o_full);
          umma_commit(&empty_v[s]);
          continue;
        }
        if (!mbar_wait(&full_k[s], ph, dead, KID_ATTN_DECODE, 2)) break;
        tc_fence_after_sync();
        // S^T = K * Q^T : K-major operands, 128-byte swizzle; d 0..63 in the first half tile, 64..127 in the second
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t da = make_smem_desc(kb + (k >> 2) * (AD_K_BYTES / 2) + (k & 3) * 32, 16, 1024, SWZ_128B);
          const uint64_t db = make_smem_desc(qb + (k >> 2) * (AD_Q_BYTES / 2) + (k & 3) * 32, 16, 1024, SWZ_128B);
          umma_f16(tmem_s, da, db, p.idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        umma_commit(&empty_k[s]);
        if (!mbar_wait(p_ready, iph, dead, KID_ATTN_DECODE, 3)) break;
        if (!mbar_wait(&full_v[s], ph, dead, KID_ATTN_DECODE, 4)) break;
        if (it > 0 && !mbar_wait(o_empty, iph ^ 1u, dead, KID_ATTN_DECODE, 5)) break;
        tc_fence_after_sync();
        // O^T = V^T * P^T : A = V page read MN-major (dims contiguous), 16 tokens per MMA;
        // B = P^T [16 x 128 tokens] in the un-swizzled core-matrix layout written by the softmax warps.
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t da = make_smem_desc(vb + k * 2048, AD_K_BYTES / 2, 1024, SWZ_128B);
          const uint64_t db = make_smem_desc(smem_u32(p_smem) + k * 512, 256, 128, SWZ_NONE);
          umma_f16(tmem_o, da, db, p.idesc_o, k != 0 ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(&empty_v[s]);
      }
    }
    __syncwarp();
  } else if (KV8 == 1 && warp >= 6) {
    // ---- converter warps: raw e4m3 page -> fp16 operand tile in the swizzled layout of the 16-bit TMA load ----
    const int ctid = (int)threadIdx.x - 192;
    int it = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++it) {
      const int s = it % AD_STAGES;
      const uint32_t ph = (uint32_t)(it / AD_STAGES) & 1u;
      uint8_t* kb = smem + s * AD_STAGE_BYTES;
      if (!mbar_wait(raw_full_k, ph, dead, KID_ATTN_DECODE, 13)) break;
      if (!mbar_wait(&empty_k[s], ph ^ 1u, dead, KID_ATTN_DECODE, 14)) break;       // the previous S MMA is done with the K tile
      kv8_convert_page(raw_k, kb, ctid);
      fence_proxy_async_smem();
      mbar_arrive(&full_k[s]);
      mbar_arrive(raw_empty_k);
      if (!mbar_wait(raw_full_v, ph, dead, KID_ATTN_DECODE, 15)) break;
      if (!mbar_wait(&empty_v[s], ph ^ 1u, dead, KID_ATTN_DECODE, 16)) break;       // the previous PV MMA is done with the V tile
      kv8_convert_page(raw_v, kb + AD_K_BYTES, ctid);
      fence_proxy_async_smem();
      mbar_arrive(&full_v[s]);
      mbar_arrive(raw_empty_v);
    }
  } else {
    const int q = warp & 3;                // TMEM lane quarter
    const int t = q * 32 + lane;           // token within page (softmax) / head dim (epilogue)
    const int G = p.G;
    int it = 0;
    for (int w = blockIdx.x; w < total; w += gridDim.x, ++it) {
      const int item = w / p.Hkv, kvh = w - item * p.Hkv;
      int b = p.work[2 * item], pg = p.work[2 * item + 1];
      if ((unsigned)b >= (unsigned)p.B || (unsigned)pg >= (unsigned)p.max_splits || pg >= p.max_pages) { b = 0; pg = 0; }
      const int seq = p.seq_lens[b];
      const uint32_t iph = (uint32_t)it & 1u;
      const int kpos = pg * AD_PAGE + t;
      const bool valid = kpos < seq && (p.window <= 0 || kpos >= seq - p.window);
      mbar_wait(s_full, iph, dead, KID_ATTN_DECODE, 6);
      tc_fence_after_sync();
      uint32_t r[16];
      tmem_ld_32x32b_x16(tmem_s + ((uint32_t)(q * 32) << 16), r);
      tmem_ld_wait();
      if (KV8 == 2) {                      // S = Sa + Sb / 16
        uint32_t r2[16];
        tmem_ld_32x32b_x16(tmem_s + 16 + ((uint32_t)(q * 32) << 16), r2);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 16; ++h) r[h] = __float_as_uint(fmaf(__uint_as_float(r2[h]), 0.0625f, __uint_as_float(r[h])));
      }
      float sv[GP];
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        float x = __uint_as_float(r[h]) * p.scale_log2;
        if (p.softcap > 0.f) x = p.softcap * tanhf(__uint_as_float(r[h]) * p.scale / p.softcap) * 1.4426950408889634f;
        sv[h] = (valid && h < G) ? x : -INFINITY;
      }
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        float m = sv[h];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) red_max[q * 16 + h] = m;
      }
      asm volatile("bar.sync 1, 128;\n" ::: "memory");
      float mx[GP];
#pragma unroll
      for (int h = 0; h < GP; ++h)
        mx[h] = fmaxf(fmaxf(red_max[h], red_max[16 + h]), fmaxf(red_max[32 + h], red_max[48 + h]));
      // P^T[n][t] in the K-major core-matrix layout: ((t/8)*2 + n/8)*128 + (n%8)*16 + (t%8)*2 bytes
      uint8_t* pb = p_smem + (t >> 3) * 256 + (t & 7) * 2;
      float* rs = red_sum + iph * 64;
      if (KV8 == 2) {
        // two e4m3 terms of 256 p: Pa = fl8(256 p), Pb = fl8(16 (256 p - Pa)); bytes at ((t / 16) * 2 + h / 8) * 128 + (h % 8) * 16 + t % 16
        uint8_t* pa8 = p_smem + (t >> 4) * 256 + (t & 15);
#pragma unroll
        for (int h = 0; h < GP; ++h) {
          float pv = 0.f;
          if (h < G && valid) pv = exp2f(sv[h] - mx[h]) * 256.0f;
          unsigned short a8, b8;
          asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(a8) : "f"(0.f), "f"(pv));
          uint32_t ah;
          asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(ah) : "h"(a8));
          const float af = __half2float(__ushort_as_half((unsigned short)(ah & 0xFFFFu)));
          asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(b8) : "f"(0.f), "f"((pv - af) * 16.0f));
          uint32_t bh;
          asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(bh) : "h"(b8));
          const float bf = __half2float(__ushort_as_half((unsigned short)(bh & 0xFFFFu)));
          const int off = (h >> 3) * 128 + (h & 7) * 16;
          pa8[off] = (uint8_t)(a8 & 0xFF);
          pa8[2048 + off] = (uint8_t)(b8 & 0xFF);
          float pr = fmaf(bf, 0.0625f, af) * (1.0f / 256.0f);          // what the tensor core will see
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) pr += __shfl_xor_sync(0xffffffffu, pr, o);
          if (lane == 0) rs[q * 16 + h] = pr;
        }
      } else {
#pragma unroll
      for (int h = 0; h < GP; ++h) {
        float pv = 0.f;
        if (h < G && valid) pv = exp2f(sv[h] - mx[h]);
        const uint16_t bits = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(pv)) : __half_as_ushort(__float2half_rn(pv));
        *reinterpret_cast<uint16_t*>(pb + (h >> 3) * 128 + (h & 7) * 16) = bits;
        // sum what the tensor core will actually see
        float pr = BF16 ? __bfloat162float(__ushort_as_bfloat16(bits)) : __half2float(__ushort_as_half(bits));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pr += __shfl_xor_sync(0xffffffffu, pr, o);
        if (lane == 0) rs[q * 16 + h] = pr;
      }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_ready);
      // ---- epilogue: O^T lanes = head dims ----
      mbar_wait(o_full, iph, dead, KID_ATTN_DECODE, 7);
      tc_fence_after_sync();
      tmem_ld_32x32b_x16(tmem_o + ((uint32_t)(q * 32) << 16), r);
      tmem_ld_wait();
      if (KV8 == 2) {                      // O = (Oa + Ob / 16) / 256
        uint32_t r2[16];
        tmem_ld_32x32b_x16(tmem_o + 16 + ((uint32_t)(q * 32) << 16), r2);
        tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 16; ++h)
          r[h] = __float_as_uint(fmaf(__uint_as_float(r2[h]), 0.0625f, __uint_as_float(r[h])) * (1.0f / 256.0f));
      }
      tc_fence_before_sync();
      mbar_arrive(o_empty);
      const size_t slot = ((size_t)(b * p.Hkv + kvh) * p.max_splits + pg) * G;
      float* po = p.part_o + slot * AD_D + t;
#pragma unroll
      for (int h = 0; h < GP; ++h)
        if (h < G) po[(size_t)h * AD_D] = __uint_as_float(r[h]);
      if (t < G) {
        const float l = rs[t] + rs[16 + t] + rs[32 + t] + rs[48 + t];
        // (read back from shared memory: indexing the register copy mx[] with t would force it into local memory)
        p.part_ml[(slot + t) * 2] = fmaxf(fmaxf(red_max[t], red_max[16 + t]), fmaxf(red_max[32 + t], red_max[48 + t]));
        p.part_ml[(slot + t) * 2 + 1] = l;
      }
      if (p.counters != nullptr) {
        // ---- fused combine: the last split of this (request, KV head) to arrive merges all of them.
        // Release: CTA barrier, then one thread fences and counts (fences are cumulative over the barrier).
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        if (t == 0) {
          __threadfence();
          const int old = atomicAdd(&p.counters[b * p.Hkv + kvh], 1);
          __threadfence();
          *sh_flag = old;
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        int ns = (seq + AD_PAGE - 1) / AD_PAGE;
        if (ns > p.max_splits) {      // a length beyond the page table: merge only the slots this (request, head) owns
          ns = p.max_splits;
          if (t == 0) report_error(ERR_BAD_ARG, KID_ATTN_DECODE, 21);
        }
        if (*sh_flag == ns - 1) {
          // warp q merges heads q, q+4, ...; a lane owns four consecutive dims; eight splits are in flight per pass
          const size_t base = (size_t)(b * p.Hkv + kvh) * p.max_splits * G;
          for (int g = q; g < G; g += 4) {
            float M = -INFINITY, L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int sp0 = 0; sp0 < ns; sp0 += 8) {
              float m8[8], l8[8];
              float4 o8[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int sp = sp0 + j < ns ? sp0 + j : ns - 1;        // clamped: the duplicate gets weight zero below
                const size_t sl = base + (size_t)sp * G + g;
                m8[j] = __ldcg(&p.part_ml[sl * 2]);
                l8[j] = __ldcg(&p.part_ml[sl * 2 + 1]);
                o8[j] = __ldcg(reinterpret_cast<const float4*>(&p.part_o[sl * AD_D + lane * 4]));
              }
              float cm = M;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (sp0 + j < ns) cm = fmaxf(cm, m8[j]);
              const float resc = M == -INFINITY ? 0.f : exp2f(M - cm);
              L *= resc; acc.x *= resc; acc.y *= resc; acc.z *= resc; acc.w *= resc;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float wgt = sp0 + j < ns ? exp2f(m8[j] - cm) : 0.f;
                L += l8[j] * wgt;
                acc.x += o8[j].x * wgt; acc.y += o8[j].y * wgt; acc.z += o8[j].z * wgt; acc.w += o8[j].w * wgt;
              }
              M = cm;
            }
            const float inv = L > 0.f ? 1.0f / L : 0.f;
            uint2 pk;
            pk.x = pack_16<BF16>(acc.x * inv, acc.y * inv);
            pk.y = pack_16<BF16>(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(&p.out[(size_t)b * p.ld_out + (size_t)(kvh * G + g) * AD_D + lane * 4]) = pk;
          }
          if (t == 0) p.counters[b * p.Hkv + kvh] = 0;
        }
      }
      asm volatile("bar.sync 1, 128;\n" ::: "memory");     // red_max / sh_flag are rewritten by the next item
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_s, TMEM_COLS);
}

// Optional second output of the combine: its row quantised for the 8-bit-activation output projection.  One (request, head)
// row of 128 values is exactly one 128-wide k block of that projection (QMODE 1: int8 + scale + block sum, 2: e4m3 + scale;
// tables [Hq, ld_a]), computed from the 16-bit-rounded output so it equals what the stand-alone quantiser would produce.
struct CombineQuant {
  uint8_t* xq; int ldq;
  float* scales; float* sums;
  int ld_a;
};

// ---- combine: one CTA per (request, query head), 128 threads = head dims --------------------------
template <bool BF16, int QMODE = 0>
__global__ void attn_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                           const int* __restrict__ seq_lens, uint16_t* __restrict__ out, int ld_out, int Hq,
                                           int Hkv, int G, int max_splits, CombineQuant cq = {}, int window = 0,
                                           const float* __restrict__ sinks = nullptr) {
  const int b = blockIdx.x, hq = blockIdx.y, d = threadIdx.x;
  const int kvh = hq / G, g = hq - kvh * G;
  pdl_launch_dependents();
  pdl_wait();
  const int seq = seq_lens[b];
  int ns = (seq + AD_PAGE - 1) / AD_PAGE;
  if (ns > max_splits) {          // a length beyond the page table: merge only the slots this (request, head) owns
    ns = max_splits;
    if (d == 0) report_error(ERR_BAD_ARG, KID_ATTN_DECODE, 22);
  }
  const size_t base = (size_t)(b * Hkv + kvh) * max_splits;
  const int s0 = (window > 0 && seq > window) ? (seq - window) / AD_PAGE : 0;      // first page the plan listed
  // attention sink: a per-head logit that takes part in the softmax normalisation only
  const float sink = sinks != nullptr ? sinks[hq] * 1.4426950408889634f : -INFINITY;
  // one pass, eight splits at a time: the (max, sum, output) loads of a group are all independent, the merge is the running
  // form of the softmax combination (the running maximum replaces a separate pass over the maxima)
  float M = sink, acc = 0.f, L = sinks != nullptr ? 1.f : 0.f;
  for (int s = s0; s < ns; s += 8) {
    float m8[8], l8[8], o8[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s + j < ns) {
        const size_t sl = (base + s + j) * G + g;
        m8[j] = part_ml[sl * 2];
        l8[j] = part_ml[sl * 2 + 1];
        o8[j] = part_o[sl * AD_D + d];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (s + j < ns) {
        const float nm = fmaxf(M, m8[j]);
        if (nm > -INFINITY) {
          const float a = exp2f(M - nm), bw = exp2f(m8[j] - nm);
          acc = acc * a + o8[j] * bw;
          L = L * a + l8[j] * bw;
          M = nm;
        }
      }
    }
  }
  const float o = (ns > 0 && L > 0.f) ? acc / L : 0.f;
  uint16_t bits = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(o)) : __half_as_ushort(__float2half_rn(o));
  out[(size_t)b * ld_out + (size_t)hq * AD_D + d] = bits;
  if (QMODE != 0) {
    __shared__ float red[8];
    const float v = BF16 ? __bfloat162float(__ushort_as_bfloat16(bits)) : __half2float(__ushort_as_half(bits));
    float amax = fabsf(v);
#pragma unroll
    for (int sft = 16; sft > 0; sft >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, sft));
    if ((d & 31) == 0) red[d >> 5] = amax;
    __syncthreads();
    amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    if (QMODE == 1) {
      const float scale = fmaxf(amax, 1e-12f) / 127.0f, iv = 1.0f / scale;
      const int q = __float2int_rn(v * iv);
      cq.xq[(size_t)b * cq.ldq + (size_t)hq * AD_D + d] = (uint8_t)(q & 0xFF);
      int sm = q;
#pragma unroll
      for (int sft = 16; sft > 0; sft >>= 1) sm += __shfl_xor_sync(0xffffffffu, sm, sft);
      if ((d & 31) == 0) red[4 + (d >> 5)] = (float)sm;
      __syncthreads();
      if (d == 0) {
        cq.scales[(size_t)hq * cq.ld_a + b] = scale;
        cq.sums[(size_t)hq * cq.ld_a + b] = red[4] + red[5] + red[6] + red[7];
      }
    } else {
      const float scale = fmaxf(amax, 1e-12f) / 448.0f, iv = 1.0f / scale;
      cq.xq[(size_t)b * cq.ldq + (size_t)hq * AD_D + d] = (uint8_t)(pack_e4m3x4(v * iv, 0.f, 0.f, 0.f) & 0xFFu);
      if (d == 0) cq.scales[(size_t)hq * cq.ld_a + b] = scale;
    }
  }
}

}  // namespace fb

using namespace fb;

extern "C" int fb_attn_decode_plan_window(const int* seq_lens, int B, int* work, int* n_work, int max_items, int window, void* stream) {
  if (B <= 0 || B > 1024) return -1;
  int threads = 32;
  while (threads < B) threads <<= 1;
  launch_k(attn_decode_plan_kernel, dim3(1), dim3(threads), 0, reinterpret_cast<cudaStream_t>(stream), 0, seq_lens, B, work, n_work, max_items, window);
  return (int)cudaGetLastError();
}
extern "C" int fb_attn_decode_plan(const int* seq_lens, int B, int* work, int* n_work, int max_items, void* stream) {
  return fb_attn_decode_plan_window(seq_lens, B, work, n_work, max_items, 0, stream);
}

// Scratch sizes (floats): part_o = B*Hkv*max_splits*G*128, part_ml = B*Hkv*max_splits*G*2.
// q: [B, Hq, 128] with row stride ld_q elements between requests' heads packed (ld_q == Hq*128 required).
// k_pool/v_pool: [num_slots, Hkv, 128].  dtype: 0 = fp16, 1 = bf16; 2 / 3 = e4m3 pages with fp16 q and fp16 / bf16 out (fb_attn_decode_opts).
// counters: [B * Hkv] ints, zero on first use (the kernel leaves them zero); null keeps the separate combine kernel.
extern "C" int fb_attn_decode_opts(const void* q, const void* k_pool, const void* v_pool, void* out, int ld_out, const int* work,
                                   const int* n_work, const int* page_table, const int* seq_lens, float* part_o, float* part_ml,
                                   int B, int Hq, int Hkv, int D, long long num_slots, int max_pages, int max_splits, int max_items,
                                   float scale, int dtype, int grid_ctas, int* counters, int qmode, void* xq, int ldq, float* q_scales,
                                   float* q_sums, int ld_a, int window, float softcap, const float* sinks, void* stream_);

extern "C" int fb_attn_decode(const void* q, const void* k_pool, const void* v_pool, void* out, int ld_out, const int* work,
                              const int* n_work, const int* page_table, const int* seq_lens, float* part_o, float* part_ml,
                              int B, int Hq, int Hkv, int D, long long num_slots, int max_pages, int max_splits, int max_items,
                              float scale, int dtype, int grid_ctas, int* counters, int qmode, void* xq, int ldq, float* q_scales,
                              float* q_sums, int ld_a, void* stream_) {
  return fb_attn_decode_opts(q, k_pool, v_pool, out, ld_out, work, n_work, page_table, seq_lens, part_o, part_ml, B, Hq, Hkv, D, num_slots,
                             max_pages, max_splits, max_items, scale, dtype, grid_ctas, counters, qmode, xq, ldq, q_scales, q_sums, ld_a,
                             0, 0.f, nullptr, stream_);
}

// window > 0: sliding-window attention (the work list must come from fb_attn_decode_plan_window with the same window);
// softcap > 0: tanh soft-capping of the logits; sinks: fp32 [Hq] per-head sink logits (null: none).  The variants use the
// separate combine kernel (counters must be null).
extern "C" int fb_attn_decode_opts(const void* q, const void* k_pool, const void* v_pool, void* out, int ld_out, const int* work,
                                   const int* n_work, const int* page_table, const int* seq_lens, float* part_o, float* part_ml,
                                   int B, int Hq, int Hkv, int D, long long num_slots, int max_pages, int max_splits, int max_items,
                                   float scale, int dtype, int grid_ctas, int* counters, int qmode, void* xq, int ldq, float* q_scales,
                                   float* q_sums, int ld_a, int window, float softcap, const float* sinks, void* stream_) {
  if ((window > 0 || sinks != nullptr) && counters != nullptr) return -1;
  // qmode 1 / 2: the combine also writes the output quantised to int8 / e4m3 per (request, head) for the output projection
  // (xq [B, Hq * 128] bytes, q_scales / q_sums [Hq, ld_a]); needs the separate combine kernel (counters == null)
  if (B <= 0) return 0;
  if (qmode != 0 && (counters != nullptr || (qmode != 1 && qmode != 2))) return -1;
  CombineQuant cq;
  cq.xq = (uint8_t*)xq; cq.ldq = ldq; cq.scales = q_scales; cq.sums = q_sums; cq.ld_a = ld_a;
  if (D != AD_D || Hq % Hkv != 0) return -1;
  const int G = Hq / Hkv;
  if (G > AD_NPAD) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  // dtype 2 / 3: e4m3 pages, fp16 queries, fp16 / bf16 output (pages converted to fp16 operand tiles in shared memory).
  // dtype 4 / 5: e4m3 pages on the fp8 tensor-core path, fp16 / bf16 output; `q` = Qa and `xq` = Qb, the two e4m3 terms of the
  // queries ([B * Hq, 128] bytes each, from fb_quant_q_e4m3x2).
  const bool kv8tc = dtype == 4 || dtype == 5;
  const bool kv8 = dtype == 2 || dtype == 3 || kv8tc;
  const bool kv8_out_bf16 = dtype == 3 || dtype == 5;
  const void* q_b = kv8tc ? xq : nullptr;
  if (kv8tc) { xq = nullptr; qmode = 0; }
  if (kv8) dtype = 0;
  if (kv8 && qmode != 0) return -1;
  if (kv8tc && q_b == nullptr) return -1;
  CUtensorMap tmK, tmV, tmQ;
  CUtensorMap tmK32, tmV32;
  if (kv8tc) {
    // pages and query terms as tensor-core operands: rows of 128 bytes, 128-byte swizzle
    if (!make_tmap_2d(&tmK, k_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AD_PAGE, 128, 1, 3)) return -2;
    if (!make_tmap_2d(&tmV, v_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AD_PAGE, 128, 1, 3)) return -2;
    if (!make_tmap_2d(&tmQ, q, (uint64_t)B * Hq, D, D, AD_NPAD, 128, 1, 3)) return -2;
    if (!make_tmap_2d(&tmK32, q_b, (uint64_t)B * Hq, D, D, AD_NPAD, 128, 1, 3)) return -2;
    tmV32 = tmV;
  } else if (kv8) {
    // raw pages: one box of 128 tokens x 128 bytes, no swizzle (the converter warps build the operand layout)
    if (!make_tmap_2d(&tmK, k_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AD_PAGE, 128, 1, 0)) return -2;
    if (!make_tmap_2d(&tmV, v_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AD_PAGE, 128, 1, 0)) return -2;
    tmK32 = tmK; tmV32 = tmV;
  } else {
    if (!make_tmap_2d(&tmK, k_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AD_PAGE, 64, 2, 3)) return -2;
    if (!make_tmap_2d(&tmV, v_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AD_PAGE, 64, 2, 3)) return -2;
    if (!make_tmap_2d(&tmK32, k_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, 32, 64, 2, 3)) return -2;
    if (!make_tmap_2d(&tmV32, v_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, 32, 64, 2, 3)) return -2;
  }
  if (!kv8tc && !make_tmap_2d(&tmQ, q, (uint64_t)B * Hq, D, D, AD_NPAD, 64, 2, 3)) return -2;
  AttnDecodeParams p;
  p.work = work; p.n_work = n_work; p.page_table = page_table; p.seq_lens = seq_lens; p.part_o = part_o; p.part_ml = part_ml;
  p.max_pages = max_pages; p.max_splits = max_splits; p.Hq = Hq; p.Hkv = Hkv; p.G = G;
  p.B = B; p.max_items = max_items;
  p.counters = counters; p.out = reinterpret_cast<uint16_t*>(out); p.ld_out = ld_out; p.clip = kv8 ? 0 : 1;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window; p.softcap = softcap; p.scale = scale;
  const uint32_t f = dtype == 1 ? 1u : 0u;
  p.idesc_s = make_idesc(f, f, 0, 0, 128, AD_NPAD);            // kind::f8f6f4: format 0 = e4m3
  p.idesc_o = make_idesc(f, f, 1, 0, 128, AD_NPAD);
  // stages: 1 -> 3 resident CTAs per SM hide each other's load latency; 3 -> one CTA per SM with a deep ring
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  }
  const bool deep = grid_ctas < 0;
  if (grid_ctas < 0) grid_ctas = -grid_ctas;
  if (grid_ctas == 0) grid_ctas = deep ? sm_count : 2 * sm_count;
#define FB_AD_LAUNCH(BF, ST, GPV)                                                                                       \
  {                                                                                                                     \
    static DeviceOnce cfg;                                                                                            \
    if (cfg.need()) { cudaFuncSetAttribute(attn_decode_kernel<BF, ST, GPV>, cudaFuncAttributeMaxDynamicSharedMemorySize, ad_smem_bytes(ST)); } \
    launch_k<PDL_ATTN>(attn_decode_kernel<BF, ST, GPV>, dim3(grid_ctas), dim3(192), ad_smem_bytes(ST), stream, 0, tmK, tmV, tmQ, tmK32, tmV32, p); \
    if (counters == nullptr && qmode == 0)                                                                              \
      launch_k<PDL_COMBINE>(attn_decode_combine_kernel<BF, 0>, dim3(B, Hq), dim3(AD_D), 0, stream, 0, part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_splits, cq, window, sinks); \
    else if (counters == nullptr && qmode == 1)                                                                         \
      launch_k<PDL_COMBINE>(attn_decode_combine_kernel<BF, 1>, dim3(B, Hq), dim3(AD_D), 0, stream, 0, part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_splits, cq, window, sinks); \
    else if (counters == nullptr)                                                                                       \
      launch_k<PDL_COMBINE>(attn_decode_combine_kernel<BF, 2>, dim3(B, Hq), dim3(AD_D), 0, stream, 0, part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_splits, cq, window, sinks); \
  }
#define FB_AD_GP(BF)                                                                                                    \
  {                                                                                                                     \
    if (deep) FB_AD_LAUNCH(BF, 3, 16)                                                                                   \
    else if (G <= 1) FB_AD_LAUNCH(BF, 1, 1)                                                                             \
    else if (G <= 2) FB_AD_LAUNCH(BF, 1, 2)                                                                             \
    else if (G <= 4) FB_AD_LAUNCH(BF, 1, 4)                                                                             \
    else if (G <= 8) FB_AD_LAUNCH(BF, 1, 8)                                                                             \
    else FB_AD_LAUNCH(BF, 1, 16)                                                                                        \
  }
#define FB_AD_LAUNCH8(GPV)                                                                                               \
  {                                                                                                                     \
    static DeviceOnce cfg8;                                                                                           \
    if (cfg8.need()) { cudaFuncSetAttribute(attn_decode_kernel<false, 1, GPV, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, ad_smem_bytes(1) + 2 * AD_PAGE * AD_D); } \
    launch_k<PDL_ATTN>(attn_decode_kernel<false, 1, GPV, 1>, dim3(grid_ctas), dim3(320), ad_smem_bytes(1) + 2 * AD_PAGE * AD_D, stream, 0, tmK, tmV, tmQ, tmK32, tmV32, p); \
    if (counters == nullptr && kv8_out_bf16)                                                                            \
      launch_k<PDL_COMBINE>(attn_decode_combine_kernel<true, 0>, dim3(B, Hq), dim3(AD_D), 0, stream, 0, part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_splits, cq, window, sinks); \
    else if (counters == nullptr)                                                                                       \
      launch_k<PDL_COMBINE>(attn_decode_combine_kernel<false, 0>, dim3(B, Hq), dim3(AD_D), 0, stream, 0, part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_splits, cq, window, sinks); \
  }
#define FB_AD_LAUNCHTC(GPV)                                                                                              \
  {                                                                                                                     \
    constexpr int smem_tc = 2 * AD_PAGE * AD_D + 2 * AD_NPAD * AD_D + AD_P_BYTES + 2048;                              \
    static DeviceOnce cfgtc;                                                                                          \
    if (cfgtc.need()) { cudaFuncSetAttribute(attn_decode_kernel<false, 1, GPV, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_tc); } \
    launch_k<PDL_ATTN>(attn_decode_kernel<false, 1, GPV, 2>, dim3(grid_ctas), dim3(192), smem_tc, stream, 0, tmK, tmV, tmQ, tmK32, tmV32, p); \
    if (kv8_out_bf16)                                                                                                   \
      launch_k<PDL_COMBINE>(attn_decode_combine_kernel<true, 0>, dim3(B, Hq), dim3(AD_D), 0, stream, 0, part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_splits, cq, window, sinks); \
    else                                                                                                                \
      launch_k<PDL_COMBINE>(attn_decode_combine_kernel<false, 0>, dim3(B, Hq), dim3(AD_D), 0, stream, 0, part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_splits, cq, window, sinks); \
  }
  if (kv8tc) {
    if (counters != nullptr) return -1;
    if (grid_ctas == 2 * sm_count) grid_ctas = 4 * sm_count;       // 43 KB and 80 registers per thread: four CTAs per SM
    if (G <= 1) FB_AD_LAUNCHTC(1)
    else if (G <= 2) FB_AD_LAUNCHTC(2)
    else if (G <= 4) FB_AD_LAUNCHTC(4)
    else if (G <= 8) FB_AD_LAUNCHTC(8)
    else FB_AD_LAUNCHTC(16)
  } else if (kv8) {
    if (G <= 1) FB_AD_LAUNCH8(1)
    else if (G <= 2) FB_AD_LAUNCH8(2)
    else if (G <= 4) FB_AD_LAUNCH8(4)
    else if (G <= 8) FB_AD_LAUNCH8(8)
    else FB_AD_LAUNCH8(16)
  } else if (dtype == 1) FB_AD_GP(true) else FB_AD_GP(false)
#undef FB_AD_LAUNCH8
#undef FB_AD_LAUNCHTC
#undef FB_AD_GP
#undef FB_AD_LAUNCH
  return (int)cudaGetLastError();
}

// Two-term e4m3 form of the queries for the fp8 tensor-core mode: q = Qa + Qb / 16 (Qa = fl8(q), Qb = fl8(16 (q - Qa))).
template <bool BF16>
__global__ void quant_q_e4m3x2_kernel(const uint16_t* __restrict__ q, uint8_t* __restrict__ qa, uint8_t* __restrict__ qb, long long n8) {
  pdl_launch_dependents();
  pdl_wait();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const uint4 x = *reinterpret_cast<const uint4*>(q + i * 8);
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
  uint32_t oa[2] = {0u, 0u}, ob[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_16<BF16>(w[j]);
    unsigned short a8, b8;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(a8) : "f"(f.y), "f"(f.x));
    uint32_t ah;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(ah) : "h"(a8));
    const float2 af = __half22float2(*reinterpret_cast<const __half2*>(&ah));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(b8) : "f"((f.y - af.y) * 16.0f), "f"((f.x - af.x) * 16.0f));
    oa[j >> 1] |= (uint32_t)a8 << ((j & 1) * 16);
    ob[j >> 1] |= (uint32_t)b8 << ((j & 1) * 16);
  }
  *reinterpret_cast<uint2*>(qa + i * 8) = make_uint2(oa[0], oa[1]);
  *reinterpret_cast<uint2*>(qb + i * 8) = make_uint2(ob[0], ob[1]);
}

extern "C" int fb_quant_q_e4m3x2(const void* q, void* qa, void* qb, long long n, int dtype, void* stream) {
  if (n <= 0) return 0;
  if (n % 8 != 0 || (dtype != 0 && dtype != 1)) return -1;
  const long long n8 = n / 8;
  const int blocks = (int)((n8 + 255) / 256);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) launch_k(quant_q_e4m3x2_kernel<true>, dim3(blocks), dim3(256), 0, s, 0, (const uint16_t*)q, (uint8_t*)qa, (uint8_t*)qb, n8);
  else launch_k(quant_q_e4m3x2_kernel<false>, dim3(blocks), dim3(256), 0, s, 0, (const uint16_t*)q, (uint8_t*)qa, (uint8_t*)qb, n8);
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------------
// Allocation-free entry point (declared and documented in attn_decode_static.h)
// ---------------------------------------------------------------------------------------------------
#include "attn_decode_static.h"

namespace fb {

// layout of the static scratch (floats / ints):  [work: 2*MAX_ITEMS ints][n_work: 64 ints (one used)]
//                                                [part_ml: 2*MAX_SLOTS floats][part_o: 128*MAX_SLOTS floats]
constexpr size_t ST_WORK_WORDS = 2 * (size_t)FB_STATIC_MAX_ITEMS;
constexpr size_t ST_NWORK_WORDS = 64;
constexpr size_t ST_ML_WORDS = 2 * (size_t)FB_STATIC_MAX_SLOTS;
constexpr size_t ST_O_WORDS = (size_t)AD_D * FB_STATIC_MAX_SLOTS;
constexpr size_t ST_TOTAL_WORDS = ST_WORK_WORDS + ST_NWORK_WORDS + ST_ML_WORDS + ST_O_WORDS;

// In host code this name is only a handle for cudaGetSymbolAddress, never a device pointer.
static __device__ __align__(256) uint32_t g_static_scratch[ST_TOTAL_WORDS];

constexpr int ST_MAX_DEVICES = 64;
static uint32_t* g_static_ptr[ST_MAX_DEVICES];        // device address of the array, per device (0 = not set up)
static std::mutex g_static_mu;

// Encodes one 2-D tensor map without touching the shared descriptor cache (no host allocation either).
static bool encode_tmap_2d_direct(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                                  uint32_t box_rows, uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) || ((ld * 2) & 15)) return false;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace fb

extern "C" int fb_attn_decode_static(const void* q, const void* k_pool, const void* v_pool, void* out, int ld_out,
                                     const int* page_table, const int* seq_lens, int B, int Hq, int Hkv, int D,
                                     long long num_slots, int max_pages, float scale, int dtype, void* stream_) {
  using namespace fb;
  if (B <= 0) return 0;
  if (D != AD_D || Hkv <= 0 || Hq % Hkv != 0 || B > 1024 || max_pages <= 0 || (dtype != 0 && dtype != 1)) return -1;
  const int G = Hq / Hkv;
  if (G > AD_NPAD) return -1;
  const long long items = (long long)B * max_pages;
  const long long slots = items * Hkv * G;
  if (items > FB_STATIC_MAX_ITEMS || slots > FB_STATIC_MAX_SLOTS) return FB_STATIC_TOO_LARGE;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= ST_MAX_DEVICES) return -1;
  uint32_t* base = nullptr;
  {
    std::lock_guard<std::mutex> g(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
      // once per device, with that device current: resolve the device address of the file-scope array
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess) return (int)e;
      e = cudaFuncSetAttribute(attn_decode_kernel<true, 1, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, ad_smem_bytes(1));
      if (e != cudaSuccess) return (int)e;
      e = cudaFuncSetAttribute(attn_decode_kernel<false, 1, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, ad_smem_bytes(1));
      if (e != cudaSuccess) return (int)e;
      g_static_ptr[dev] = reinterpret_cast<uint32_t*>(p);
    }
    base = g_static_ptr[dev];
  }
  int* work = reinterpret_cast<int*>(base);
  int* n_work = reinterpret_cast<int*>(base + ST_WORK_WORDS);
  float* part_ml = reinterpret_cast<float*>(base + ST_WORK_WORDS + ST_NWORK_WORDS);
  float* part_o = reinterpret_cast<float*>(base + ST_WORK_WORDS + ST_NWORK_WORDS + ST_ML_WORDS);
  CUtensorMap tmK, tmV, tmQ;
  if (!encode_tmap_2d_direct(&tmK, k_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AD_PAGE, 64)) return -2;
  if (!encode_tmap_2d_direct(&tmV, v_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AD_PAGE, 64)) return -2;
  if (!encode_tmap_2d_direct(&tmQ, q, (uint64_t)B * Hq, D, D, AD_NPAD, 64)) return -2;
  int threads = 32;
  while (threads < B) threads <<= 1;
  attn_decode_plan_kernel<<<1, threads, 0, stream>>>(seq_lens, B, work, n_work, (int)items);
  AttnDecodeParams p;
  p.work = work; p.n_work = n_work; p.page_table = page_table; p.seq_lens = seq_lens; p.part_o = part_o; p.part_ml = part_ml;
  p.max_pages = max_pages; p.max_splits = max_pages; p.Hq = Hq; p.Hkv = Hkv; p.G = G;
  p.B = B; p.max_items = (int)items;
  p.counters = nullptr; p.out = nullptr; p.ld_out = 0; p.clip = 0;      // whole-page loads, separate combine kernel
  p.window = 0; p.softcap = 0.f; p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  const uint32_t f = dtype == 1 ? 1u : 0u;
  p.idesc_s = make_idesc(f, f, 0, 0, 128, AD_NPAD);
  p.idesc_o = make_idesc(f, f, 1, 0, 128, AD_NPAD);
  int sms = 0;
  e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
  const int grid = 2 * sms;
  if (dtype == 1) {
    attn_decode_kernel<true, 1, 16><<<grid, 192, ad_smem_bytes(1), stream>>>(tmK, tmV, tmQ, tmK, tmV, p);
    attn_decode_combine_kernel<true, 0><<<dim3(B, Hq), AD_D, 0, stream>>>(part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_pages, CombineQuant{});
  } else {
    attn_decode_kernel<false, 1, 16><<<grid, 192, ad_smem_bytes(1), stream>>>(tmK, tmV, tmQ, tmK, tmV, p);
    attn_decode_combine_kernel<false, 0><<<dim3(B, Hq), AD_D, 0, stream>>>(part_o, part_ml, seq_lens, (uint16_t*)out, ld_out, Hq, Hkv, G, max_pages, CombineQuant{});
  }
  return (int)cudaGetLastError();
}
