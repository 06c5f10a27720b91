// Paged causal GQA prefill attention for sm_100a (head_dim 128, page length 128), tcgen05 + TMEM.
//
// One CTA owns 128 consecutive new tokens of one request for one query head and walks the request's KV
// pages (prefix-cache pages and chunked-prefill history included) up to the causal frontier:
//     S[128 q x 128 kv] = Q * K_page^T          accumulators in TMEM columns [0,128)
//     online softmax: one thread per query row reads its S row from TMEM (no cross-thread reductions)
//     O[128 q x 128 d] += P * V_page            accumulators in TMEM columns [128,256), rescaled in place
//                                               through tcgen05.ld/st only when a row maximum moved
// K and V pages arrive by TMA into a 2-stage ring; P goes back to shared memory in the 128-byte-swizzled
// K-major layout as the A operand of the second MMA; V is consumed MN-major straight from the page layout.
// The reference routes this through FlashInfer's FA2 mma.sync kernel
// (src/devices/cuda/attention/fastllm-attention.cu:2490, 3032-3600).
#include <cstdlib>
#include "ptx.cuh"
#include "launch.h"
#include "tmap.h"

FB_DEFINE_ERROR_API(attn_prefill)

namespace fb {

constexpr int KID_ATTN_PREFILL = 11;
constexpr int AP_STAGES = 2;
constexpr int AP_D = 128;
constexpr int AP_PAGE = 128;
constexpr int AP_TILE = 128 * 128 * 2;   // 32 KB: 128 rows x 128 16-bit values (two 16 KB half tiles)
constexpr int AP_SMEM_BYTES = AP_TILE /*Q*/ + AP_STAGES * 2 * AP_TILE + AP_TILE /*P*/ + 256 + 1024;

struct AttnPrefillParams {
  const int* blocks;      // [n_blocks][2] = (request, first new-token index of the block within the request)
  const int* cu_q;        // [B+1] offsets of each request's new tokens in the packed q / out tensors
  const int* kv_lens;     // [B] tokens in the cache after the append (history + new)
  const int* page_table;  // [B, max_pages]
  uint16_t* out; int ld_out;
  int max_pages, Hq, G;
  float scale_log2;
  uint32_t idesc_s, idesc_o;
};

template <bool BF16>
__global__ void __launch_bounds__(192, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnPrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;
  uint8_t* kv_smem = smem + AP_TILE;
  uint8_t* p_smem = kv_smem + AP_STAGES * 2 * AP_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + AP_TILE);
  uint64_t* full_k = bars;
  uint64_t* full_v = bars + AP_STAGES;
  uint64_t* empty = bars + 2 * AP_STAGES;
  uint64_t* q_full = bars + 3 * AP_STAGES;
  uint64_t* s_full = q_full + 1;
  uint64_t* p_ready = q_full + 2;
  uint64_t* o_full = q_full + 3;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = p.blocks[2 * blockIdx.x], q0 = p.blocks[2 * blockIdx.x + 1];
  const int hq = blockIdx.y, kvh = hq / p.G;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int kv_len = p.kv_lens[b];
  const int pos0 = kv_len - q_len + q0;                 // absolute position of the block's first query
  int rows = q_len - q0; if (rows > 128) rows = 128;
  int kv_end = pos0 + rows;                              // causal frontier (exclusive) of the last row
  if (kv_end > kv_len) kv_end = kv_len;
  const int n_pages = (kv_end + AP_PAGE - 1) / AP_PAGE;
  bool dead = false;

  if (threadIdx.x == 0) {
    for (int s = 0; s < AP_STAGES; ++s) { mbar_init(&full_k[s], 1); mbar_init(&full_v[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(q_full, 1);
    mbar_init(s_full, 1);
    mbar_init(p_ready, 128);
    mbar_init(o_full, 1);
    mbar_init_fence();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_s = *tmem_slot;
  const uint32_t tmem_o = tmem_s + 128;

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, AP_TILE);
      tma_load_2d(q_smem, &tmQ, q_full, hq * AP_D, q_begin + q0);
      tma_load_2d(q_smem + AP_TILE / 2, &tmQ, q_full, hq * AP_D + 64, q_begin + q0);
      for (int it = 0; it < n_pages; ++it) {
        const int s = it % AP_STAGES;
        const uint32_t ph = (uint32_t)(it / AP_STAGES) & 1u;
        if (!mbar_wait(&empty[s], ph ^ 1u, dead, KID_ATTN_PREFILL, 1)) break;
        const int page = p.page_table[(size_t)b * p.max_pages + it];
        uint8_t* kb = kv_smem + s * 2 * AP_TILE;
        uint8_t* vb = kb + AP_TILE;
        mbar_expect_tx(&full_k[s], AP_TILE);
        tma_load_2d(kb, &tmK, &full_k[s], kvh * AP_D, page * AP_PAGE);
        tma_load_2d(kb + AP_TILE / 2, &tmK, &full_k[s], kvh * AP_D + 64, page * AP_PAGE);
        mbar_expect_tx(&full_v[s], AP_TILE);
        tma_load_2d(vb, &tmV, &full_v[s], kvh * AP_D, page * AP_PAGE);
        tma_load_2d(vb + AP_TILE / 2, &tmV, &full_v[s], kvh * AP_D + 64, page * AP_PAGE);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      bool ok = mbar_wait(q_full, 0, dead, KID_ATTN_PREFILL, 2);
      const uint32_t qb = smem_u32(q_smem), pb = smem_u32(p_smem);
      for (int it = 0; ok && it < n_pages; ++it) {
        const int s = it % AP_STAGES;
        const uint32_t ph = (uint32_t)(it / AP_STAGES) & 1u;
        const uint32_t iph = (uint32_t)it & 1u;
        const uint32_t kb = smem_u32(kv_smem + s * 2 * AP_TILE), vb = kb + AP_TILE;
        if (!mbar_wait(&full_k[s], ph, dead, KID_ATTN_PREFILL, 3)) break;
        tc_fence_after_sync();
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t da = make_smem_desc(qb + (k >> 2) * (AP_TILE / 2) + (k & 3) * 32, 16, 1024, SWZ_128B);
          const uint64_t db = make_smem_desc(kb + (k >> 2) * (AP_TILE / 2) + (k & 3) * 32, 16, 1024, SWZ_128B);
          umma_f16(tmem_s, da, db, p.idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        if (!mbar_wait(p_ready, iph, dead, KID_ATTN_PREFILL, 4)) break;
        if (!mbar_wait(&full_v[s], ph, dead, KID_ATTN_PREFILL, 5)) break;
        tc_fence_after_sync();
        // O += P * V : A = P (K-major, kv 0..63 in the first half tile), B = V page MN-major (16 tokens per MMA)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t da = make_smem_desc(pb + (k >> 2) * (AP_TILE / 2) + (k & 3) * 32, 16, 1024, SWZ_128B);
          const uint64_t db = make_smem_desc(vb + k * 2048, AP_TILE / 2, 1024, SWZ_128B);
          umma_f16(tmem_o, da, db, p.idesc_o, (it | k) != 0 ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(&empty[s]);
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;                 // query row within the block
    const int pos = pos0 + r;                    // absolute position (causal limit, inclusive)
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    for (int it = 0; it < n_pages; ++it) {
      const uint32_t iph = (uint32_t)it & 1u;
      mbar_wait(s_full, iph, dead, KID_ATTN_PREFILL, 6);
      tc_fence_after_sync();
      const int kv0 = it * AP_PAGE;
      // pass 1: row maximum
      float m_new = m_run;
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t sreg[32];
        tmem_ld_32x32b_x32(tmem_s + lane_off + c0, sreg);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int kv = kv0 + c0 + j;
          const float s = (kv <= pos && kv < kv_len) ? __uint_as_float(sreg[j]) * p.scale_log2 : -INFINITY;
          m_new = fmaxf(m_new, s);
        }
      }
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);          // m_run = -inf -> 0
      // The previous P*V must be complete before P is overwritten or O is rescaled.
      if (it > 0) {
        mbar_wait(o_full, iph ^ 1u, dead, KID_ATTN_PREFILL, 7);
        tc_fence_after_sync();
        // rescale O in TMEM only if some row of this warp moved its maximum
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t oreg[32];
            tmem_ld_32x32b_x32(tmem_o + lane_off + c0, oreg);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) oreg[j] = __float_as_uint(__uint_as_float(oreg[j]) * alpha);
            tmem_st_32x32b_x32(tmem_o + lane_off + c0, oreg);
          }
          tmem_st_wait();
        }
      }
      // pass 2: probabilities -> shared memory (A operand of the second MMA), running sum
      float l_add = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        uint32_t sreg[32];
        tmem_ld_32x32b_x32(tmem_s + lane_off + c0, sreg);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int kv = kv0 + c0 + j;
          const float s0 = (kv <= pos && kv < kv_len) ? __uint_as_float(sreg[j]) * p.scale_log2 : -INFINITY;
          const float s1 = (kv + 1 <= pos && kv + 1 < kv_len) ? __uint_as_float(sreg[j + 1]) * p.scale_log2 : -INFINITY;
          const float p0 = exp2f(s0 - m_use), p1 = exp2f(s1 - m_use);
          const uint32_t pk = pack_16<BF16>(p0, p1);
          packed[j >> 1] = pk;
          const float2 back = unpack_16<BF16>(pk);
          l_add += back.x + back.y;
        }
        // 32 values = 64 bytes = 4 chunks of 16 B; half tile = c0 / 64, chunk index within the 128-byte row = (c0 % 64) / 8 + g
        uint8_t* rowp = p_smem + (c0 >> 6) * (AP_TILE / 2) + r * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int chunk = ((c0 & 63) >> 3) + g;
          *reinterpret_cast<uint4*>(rowp + ((chunk ^ (r & 7)) << 4)) =
              make_uint4(packed[4 * g], packed[4 * g + 1], packed[4 * g + 2], packed[4 * g + 3]);
        }
      }
      l_run = l_run * alpha + l_add;
      m_run = m_new;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(p_ready);
    }
    // final: normalise and write
    if (n_pages > 0) {
      mbar_wait(o_full, (uint32_t)(n_pages - 1) & 1u, dead, KID_ATTN_PREFILL, 8);
      tc_fence_after_sync();
    }
    const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
    uint16_t* orow = p.out + (size_t)(q_begin + q0 + r) * p.ld_out + (size_t)hq * AP_D;
#pragma unroll 1
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t oreg[32];
      __syncwarp();
      tmem_ld_32x32b_x32(tmem_o + lane_off + c0, oreg);
      tmem_ld_wait();
      if (r < rows) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_16<BF16>(__uint_as_float(oreg[8 * g + 0]) * inv_l, __uint_as_float(oreg[8 * g + 1]) * inv_l);
          o.y = pack_16<BF16>(__uint_as_float(oreg[8 * g + 2]) * inv_l, __uint_as_float(oreg[8 * g + 3]) * inv_l);
          o.z = pack_16<BF16>(__uint_as_float(oreg[8 * g + 4]) * inv_l, __uint_as_float(oreg[8 * g + 5]) * inv_l);
          o.w = pack_16<BF16>(__uint_as_float(oreg[8 * g + 6]) * inv_l, __uint_as_float(oreg[8 * g + 7]) * inv_l);
          if (n_pages == 0) o = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(orow + c0 + 8 * g) = o;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_s, 256);
}


// ---------------------------------------------------------------------------------------------------
// Second-generation kernel: two query heads of one KV head per CTA, half-page (64-token) KV steps.
//
// Both heads read the same K / V tiles (loaded once), and their softmax runs on two separate warp groups, so the tensor
// core alternates between the heads: while head B's probabilities are being formed it computes P_A * V and the next
// Q_A * K^T, and vice versa.  TMEM holds S_A, S_B (64 columns each) and O_A, O_B (128 each).  A softmax thread owns one
// query row and keeps the step's 64 logits in registers (one TMEM read per step).
//   shared memory: Q_A, Q_B 64 KB | 3-stage ring of (K, V) half pages 96 KB | P_A, P_B 32 KB
// ---------------------------------------------------------------------------------------------------
constexpr int AP2_KV = 64;
constexpr int AP2_STAGES = 3;
constexpr int AP2_KT = AP2_KV * 128 * 2;          // 16 KB: 64 rows x 128 values, two 8 KB halves (64 dims each)
constexpr int AP2_PT = 128 * AP2_KV * 2;          // 16 KB: 128 query rows x 64 probabilities
constexpr int AP2_SMEM_BYTES = 2 * AP_TILE + AP2_STAGES * 2 * AP2_KT + 2 * AP2_PT + 256 + 1024;

template <bool BF16>
__global__ void __launch_bounds__(320, 1)
attn_prefill2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const AttnPrefillParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_smem = smem;                                   // [2 heads] x 32 KB
  uint8_t* kv_smem = smem + 2 * AP_TILE;                    // [stages] x (K 16 KB, V 16 KB)
  uint8_t* p_smem = kv_smem + AP2_STAGES * 2 * AP2_KT;      // [2 heads] x 16 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + 2 * AP2_PT);
  uint64_t* full_k = bars;
  uint64_t* full_v = bars + AP2_STAGES;
  uint64_t* empty = bars + 2 * AP2_STAGES;
  uint64_t* q_full = bars + 3 * AP2_STAGES;
  uint64_t* s_full = q_full + 1;      // [2]
  uint64_t* p_ready = q_full + 3;     // [2]
  uint64_t* o_full = q_full + 5;      // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 7);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid: x = head pair (fast), y = query block; the host lists the blocks longest-first, so CTAs are handed out heaviest
  // first and the short blocks near the start of a sequence fill the tail of the launch
  const int b = p.blocks[2 * blockIdx.y], q0 = p.blocks[2 * blockIdx.y + 1];
  const int hq0 = 2 * blockIdx.x, kvh = hq0 / p.G;
  const int q_begin = p.cu_q[b], q_len = p.cu_q[b + 1] - q_begin;
  const int kv_len = p.kv_lens[b];
  const int pos0 = kv_len - q_len + q0;
  int rows = q_len - q0; if (rows > 128) rows = 128;
  int kv_end = pos0 + rows;
  if (kv_end > kv_len) kv_end = kv_len;
  const int n_steps = (kv_end + AP2_KV - 1) / AP2_KV;
  bool dead = false;

  if (threadIdx.x == 0) {
    for (int s = 0; s < AP2_STAGES; ++s) { mbar_init(&full_k[s], 1); mbar_init(&full_v[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(q_full, 1);
    for (int h = 0; h < 2; ++h) { mbar_init(&s_full[h], 1); mbar_init(&p_ready[h], 128); mbar_init(&o_full[h], 1); }
    mbar_init_fence();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem0 = *tmem_slot;
  // columns: S_A [0,64) S_B [64,128) O_A [128,256) O_B [256,384)

  if (warp == 0) {
    if (elect_one()) {
      mbar_expect_tx(q_full, 2 * AP_TILE);
      for (int h = 0; h < 2; ++h) {
        tma_load_2d(q_smem + h * AP_TILE, &tmQ, q_full, (hq0 + h) * AP_D, q_begin + q0);
        tma_load_2d(q_smem + h * AP_TILE + AP_TILE / 2, &tmQ, q_full, (hq0 + h) * AP_D + 64, q_begin + q0);
      }
      for (int it = 0; it < n_steps; ++it) {
        const int s = it % AP2_STAGES;
        const uint32_t ph = (uint32_t)(it / AP2_STAGES) & 1u;
        if (!mbar_wait(&empty[s], ph ^ 1u, dead, KID_ATTN_PREFILL, 11)) break;
        const int page = p.page_table[(size_t)b * p.max_pages + (it >> 1)];
        const int row = page * AP_PAGE + (it & 1) * AP2_KV;
        uint8_t* kb = kv_smem + s * 2 * AP2_KT;
        uint8_t* vb = kb + AP2_KT;
        mbar_expect_tx(&full_k[s], AP2_KT);
        tma_load_2d(kb, &tmK, &full_k[s], kvh * AP_D, row);
        tma_load_2d(kb + AP2_KT / 2, &tmK, &full_k[s], kvh * AP_D + 64, row);
        mbar_expect_tx(&full_v[s], AP2_KT);
        tma_load_2d(vb, &tmV, &full_v[s], kvh * AP_D, row);
        tma_load_2d(vb + AP2_KT / 2, &tmV, &full_v[s], kvh * AP_D + 64, row);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      bool ok = n_steps > 0 && mbar_wait(q_full, 0, dead, KID_ATTN_PREFILL, 12);
      const uint32_t qb = smem_u32(q_smem), pb = smem_u32(p_smem);
      auto issue_s = [&](int h, uint32_t kb) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t da = make_smem_desc(qb + h * AP_TILE + (k >> 2) * (AP_TILE / 2) + (k & 3) * 32, 16, 1024, SWZ_128B);
          const uint64_t db = make_smem_desc(kb + (k >> 2) * (AP2_KT / 2) + (k & 3) * 32, 16, 1024, SWZ_128B);
          umma_f16(tmem0 + (uint32_t)(h * 64), da, db, p.idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[h]);
      };
      if (ok) ok = mbar_wait(&full_k[0], 0, dead, KID_ATTN_PREFILL, 13);
      if (ok) {
        tc_fence_after_sync();
        issue_s(0, smem_u32(kv_smem));
        issue_s(1, smem_u32(kv_smem));
      }
      for (int it = 0; ok && it < n_steps; ++it) {
        const int s = it % AP2_STAGES, s1 = (it + 1) % AP2_STAGES;
        const uint32_t ph = (uint32_t)(it / AP2_STAGES) & 1u, ph1 = (uint32_t)((it + 1) / AP2_STAGES) & 1u;
        const uint32_t iph = (uint32_t)it & 1u;
        const uint32_t vb = smem_u32(kv_smem + s * 2 * AP2_KT) + AP2_KT;
        const uint32_t kb1 = smem_u32(kv_smem + s1 * 2 * AP2_KT);
        const bool more = it + 1 < n_steps;
        for (int h = 0; h < 2; ++h) {
          if (!mbar_wait(&p_ready[h], iph, dead, KID_ATTN_PREFILL, 14)) { ok = false; break; }
          if (h == 0 && !mbar_wait(&full_v[s], ph, dead, KID_ATTN_PREFILL, 15)) { ok = false; break; }
          tc_fence_after_sync();
          // O_h += P_h * V : A = P_h (K-major, 64 kv), B = V half page MN-major (16 tokens per MMA)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_smem_desc(pb + h * AP2_PT + k * 32, 16, 1024, SWZ_128B);
            const uint64_t db = make_smem_desc(vb + k * 2048, AP2_KT / 2, 1024, SWZ_128B);
            umma_f16(tmem0 + 128u + (uint32_t)(h * 128), da, db, p.idesc_o, (it | k) != 0 ? 1u : 0u);
          }
          umma_commit(&o_full[h]);
          if (more) {
            if (h == 0 && !mbar_wait(&full_k[s1], ph1, dead, KID_ATTN_PREFILL, 16)) { ok = false; break; }
            tc_fence_after_sync();
            issue_s(h, kb1);
          }
        }
        if (ok) umma_commit(&empty[s]);
      }
    }
    __syncwarp();
  } else {
    const int h = (warp - 2) >> 2;               // which head this warp group serves
    const int q = warp & 3;                      // TMEM lane quarter: warps 2..5 -> 2,3,0,1 ; 6..9 -> 2,3,0,1
    const int r = q * 32 + lane;
    const int pos = pos0 + r;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const uint32_t tmem_s = tmem0 + (uint32_t)(h * 64), tmem_o = tmem0 + 128u + (uint32_t)(h * 128);
    uint8_t* prow = p_smem + h * AP2_PT + r * 128;
    float m_run = -INFINITY, l_run = 0.f;
    for (int it = 0; it < n_steps; ++it) {
      const uint32_t iph = (uint32_t)it & 1u;
      mbar_wait(&s_full[h], iph, dead, KID_ATTN_PREFILL, 17);
      tc_fence_after_sync();
      const int kv0 = it * AP2_KV;
      uint32_t sreg[64];
      tmem_ld_32x32b_x32(tmem_s + lane_off, sreg);
      tmem_ld_32x32b_x32(tmem_s + lane_off + 32, sreg + 32);
      tmem_ld_wait();
      // Raw logits stay in registers; the softmax scale is folded into the exponent's FMA.  Only steps that touch the
      // causal diagonal of this block (or the end of the cache) pay for the mask; kv0 + 63 <= pos0 means every row of
      // the block sees the whole step.
      const bool full_step = kv0 + AP2_KV - 1 <= pos0 && kv0 + AP2_KV <= kv_len;
      float m_raw = -INFINITY;
      if (full_step) {
#pragma unroll
        for (int j = 0; j < 64; ++j) m_raw = fmaxf(m_raw, __uint_as_float(sreg[j]));
      } else {
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const int kv = kv0 + j;
          const float sv = (kv <= pos && kv < kv_len) ? __uint_as_float(sreg[j]) : -INFINITY;
          sreg[j] = __float_as_uint(sv);
          m_raw = fmaxf(m_raw, sv);
        }
      }
      const float m_new = fmaxf(m_run, m_raw * p.scale_log2);          // scale > 0: the maximum commutes with it
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m_run - m_use);
      if (it > 0) {
        // the previous P * V of this head must be complete before P is overwritten or O is rescaled
        mbar_wait(&o_full[h], iph ^ 1u, dead, KID_ATTN_PREFILL, 18);
        tc_fence_after_sync();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 32) {
            uint32_t oreg[32];
            tmem_ld_32x32b_x32(tmem_o + lane_off + c0, oreg);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) oreg[j] = __float_as_uint(__uint_as_float(oreg[j]) * alpha);
            tmem_st_32x32b_x32(tmem_o + lane_off + c0, oreg);
          }
          tmem_st_wait();
        }
      }
      float l_add = 0.f;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        uint32_t pk[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float p0 = exp2f(fmaf(__uint_as_float(sreg[8 * g + 2 * j]), p.scale_log2, -m_use));
          const float p1 = exp2f(fmaf(__uint_as_float(sreg[8 * g + 2 * j + 1]), p.scale_log2, -m_use));
          pk[j] = pack_16<BF16>(p0, p1);
          l_add += p0 + p1;
        }
        *reinterpret_cast<uint4*>(prow + ((g ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l_run = l_run * alpha + l_add;
      m_run = m_new;
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&p_ready[h]);
    }
    if (n_steps > 0) {
      mbar_wait(&o_full[h], (uint32_t)(n_steps - 1) & 1u, dead, KID_ATTN_PREFILL, 19);
      tc_fence_after_sync();
    }
    const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
    uint16_t* orow = p.out + (size_t)(q_begin + q0 + r) * p.ld_out + (size_t)(hq0 + h) * AP_D;
#pragma unroll 1
    for (int c0 = 0; c0 < 128; c0 += 32) {
      uint32_t oreg[32];
      __syncwarp();
      tmem_ld_32x32b_x32(tmem_o + lane_off + c0, oreg);
      tmem_ld_wait();
      if (r < rows) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 o;
          o.x = pack_16<BF16>(__uint_as_float(oreg[8 * g + 0]) * inv_l, __uint_as_float(oreg[8 * g + 1]) * inv_l);
          o.y = pack_16<BF16>(__uint_as_float(oreg[8 * g + 2]) * inv_l, __uint_as_float(oreg[8 * g + 3]) * inv_l);
          o.z = pack_16<BF16>(__uint_as_float(oreg[8 * g + 4]) * inv_l, __uint_as_float(oreg[8 * g + 5]) * inv_l);
          o.w = pack_16<BF16>(__uint_as_float(oreg[8 * g + 6]) * inv_l, __uint_as_float(oreg[8 * g + 7]) * inv_l);
          if (n_steps == 0) o = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(orow + c0 + 8 * g) = o;
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem0, 512);
}

}  // namespace fb

using namespace fb;

// q/out: packed new tokens [T, Hq*128] (row strides ld_q / ld_out elements).  blocks: device int32 [n_blocks][2].
extern "C" int fb_attn_prefill(const void* q, int ld_q, long long T, const void* k_pool, const void* v_pool, void* out, int ld_out,
                               const int* blocks, int n_blocks, const int* cu_q, const int* kv_lens, const int* page_table,
                               int Hq, int Hkv, int D, long long num_slots, int max_pages, float scale, int dtype, void* stream_) {
  if (n_blocks <= 0) return 0;
  if (D != AP_D || Hq % Hkv != 0) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  CUtensorMap tmQ, tmK, tmV;
  if (!make_tmap_2d(&tmQ, q, (uint64_t)T, (uint64_t)Hq * D, (uint64_t)ld_q, 128, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmK, k_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AP_PAGE, 64, 2, 3)) return -2;
  if (!make_tmap_2d(&tmV, v_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AP_PAGE, 64, 2, 3)) return -2;
  AttnPrefillParams p;
  p.blocks = blocks; p.cu_q = cu_q; p.kv_lens = kv_lens; p.page_table = page_table;
  p.out = (uint16_t*)out; p.ld_out = ld_out; p.max_pages = max_pages; p.Hq = Hq; p.G = Hq / Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  const uint32_t f = dtype == 1 ? 1u : 0u;
  p.idesc_s = make_idesc(f, f, 0, 0, 128, 128);
  p.idesc_o = make_idesc(f, f, 0, 1, 128, 128);
  static const bool use_v2 = []() { const char* e = std::getenv("FB_ATTN_PREFILL_V2"); return e == nullptr || std::atoi(e) != 0; }();
  if (use_v2 && (Hq / Hkv) % 2 == 0) {
    // two heads of a KV group per CTA, 64-token KV steps
    CUtensorMap tmK64, tmV64;
    if (!make_tmap_2d(&tmK64, k_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AP2_KV, 64, 2, 3)) return -2;
    if (!make_tmap_2d(&tmV64, v_pool, (uint64_t)num_slots, (uint64_t)Hkv * D, (uint64_t)Hkv * D, AP2_KV, 64, 2, 3)) return -2;
    p.idesc_s = make_idesc(f, f, 0, 0, 128, AP2_KV);
    if (n_blocks > 65535) return -1;
    dim3 grid2(Hq / 2, n_blocks);
    if (dtype == 1) {
      static DeviceOnce cfg;
      if (cfg.need()) { cudaFuncSetAttribute(attn_prefill2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, AP2_SMEM_BYTES); }
      attn_prefill2_kernel<true><<<grid2, 320, AP2_SMEM_BYTES, stream>>>(tmQ, tmK64, tmV64, p);
    } else {
      static DeviceOnce cfg;
      if (cfg.need()) { cudaFuncSetAttribute(attn_prefill2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, AP2_SMEM_BYTES); }
      attn_prefill2_kernel<false><<<grid2, 320, AP2_SMEM_BYTES, stream>>>(tmQ, tmK64, tmV64, p);
    }
    return (int)cudaGetLastError();
  }
  dim3 grid(n_blocks, Hq);
  if (dtype == 1) {
    static DeviceOnce cfg;
    if (cfg.need()) { cudaFuncSetAttribute(attn_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, AP_SMEM_BYTES); }
    attn_prefill_kernel<true><<<grid, 192, AP_SMEM_BYTES, stream>>>(tmQ, tmK, tmV, p);
  } else {
    static DeviceOnce cfg;
    if (cfg.need()) { cudaFuncSetAttribute(attn_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, AP_SMEM_BYTES); }
    attn_prefill_kernel<false><<<grid, 192, AP_SMEM_BYTES, stream>>>(tmQ, tmK, tmV, p);
  }
  return (int)cudaGetLastError();
}
