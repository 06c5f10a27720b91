// Small-M (decode) tcgen05 GEMM body shared by the plain GEMM kernel and the fused GEMM + all-reduce kernel.
// See gemm_bf16.cu for the design notes.
#pragma once
#include "ptx.cuh"

namespace fb {

// Grouped (mixture-of-experts) launches: grid slot j -> (expert, row chunk).  The slots enumerate only the chunks that exist,
// expert by expert (sum over experts of ceil(count / rows_per_chunk)), so the grid needs E + rows / rows_per_chunk slots instead
// of E * (most rows any expert could get / rows_per_chunk), nearly all of which would be empty.  Every warp computes the same
// answer from the counts (a 32-wide scan per 32 experts); returns false for a slot past the last chunk.
__device__ __forceinline__ bool moe_find_item(const int* __restrict__ counts, int n_local, int rows_per_chunk, int j, int& e, int& chunk) {
  const int lane = threadIdx.x & 31;
  int base = 0;
  for (int e0 = 0; e0 < n_local; e0 += 32) {
    const int ee = e0 + lane;
    const int nch = ee < n_local ? (counts[ee] + rows_per_chunk - 1) / rows_per_chunk : 0;
    int incl = nch;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    const int total = __shfl_sync(0xffffffffu, incl, 31);
    if (j < base + total) {
      const int excl = base + incl - nch;
      const unsigned hit = __ballot_sync(0xffffffffu, j >= excl && j < excl + nch);
      const int src = __ffs(hit) - 1;
      e = e0 + src;
      chunk = j - __shfl_sync(0xffffffffu, excl, src);
      return true;
    }
    base += total;
  }
  return false;
}


constexpr int KID_GEMM_SMALLM_PLAIN = 1;
constexpr int KID_GEMM_LARGEM = 2;

enum GemmFlags : int {
  GEMM_BIAS = 1,       // += bias[n]
  GEMM_RESIDUAL = 2,   // += residual[m, n]
  GEMM_SWIGLU = 4,     // out[m, i] = silu(gate) * up   (N_out = N / 2)
  GEMM_OUT_F32 = 8,    // write fp32 instead of the 16-bit input dtype
  GEMM_FP4_F16W = 256, // fp4 weights, fp16 activations: the scale table lies within fp16's range (host-checked): half2 de-quantiser
};

struct GemmParams {
  void* out;
  const void* bias;
  const void* residual;
  int M, N, K;
  int ld_out, ld_res;
  int kb_per_split;   // 64-wide k blocks per cluster rank
  int kb_total;
  uint32_t idesc;
  int flags;
  // Row scatter (tensor-parallel reduce-scatter by push): with scatter_tp > 0 and GEMM_OUT_F32 the fp32 row j goes to
  // scatter_out[j / scatter_rows] (a peer's arena), at row (scatter_rank * M + j) of a [tp * M, ld_out] matrix.
  int scatter_tp, scatter_rows, scatter_rank;
  int w_row0, x_row0;        // row offsets added to the weight / activation tile coordinates (grouped GEMM)
  float* scatter_out[8];
  // Deferred all-gather wait: the activations were broadcast by a fused collective kernel that did not wait for its
  // peers' rows to land.  The producer thread waits (bounded) until *wait_cnt has reached *wait_expect after it has
  // requested the first ring of weight tiles and before it requests any activation tile.
  const uint32_t* wait_cnt = nullptr;
  const uint32_t* wait_expect = nullptr;
  // Batched mode (grid.z = batch index z): weight rows start at z * batch_w_rows, the activation's k range at column
  // z * batch_x_cols, the output at column z * batch_out_cols -- one launch for a GEMM per attention head (the absorbed
  // multi-head-latent-attention projections, where every head has its own small matrix and its own slice of the activations).
  int batch_w_rows = 0, batch_x_cols = 0, batch_out_cols = 0;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// OCC = CTAs meant to be co-resident per SM: 1 -> deep ring (~200 KB), 2 -> two CTAs share the SM so that one
// streams weights while the other is in its prologue / epilogue.
template <int MPAD, int OCC = 1>
struct SmallMCfg {
  static constexpr int A_BYTES = 128 * 128;            // 128 rows x 64 bf16
  static constexpr int B_BYTES = MPAD * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int MAX_STAGES = ((200 * 1024) / OCC) / STAGE_BYTES;
  static constexpr int STAGES = MAX_STAGES > 10 ? 10 : MAX_STAGES;
  static constexpr int RED_BYTES = MPAD * 128 * 4;     // fp32 partial tile [MPAD][128]
  static constexpr int PIPE_BYTES = STAGES * STAGE_BYTES;
  static constexpr int BODY_BYTES = PIPE_BYTES > RED_BYTES ? PIPE_BYTES : RED_BYTES;
  static constexpr int SMEM_BYTES = BODY_BYTES + 256 + 1024;   // + barriers + alignment slack
  static constexpr int TMEM_COLS = MPAD < 32 ? 32 : MPAD;
};

// Cross-CTA reduction over the k splits + epilogue.  Every CTA of the cluster holds its fp32 partial tile P[token][n]
// at `smem`; this CTA reduces and stores its own column slice (bias -> SwiGLU -> residual -> store / scatter).
template <bool BF16>
__device__ __forceinline__ void smallm_reduce_store(const GemmParams& p, uint8_t* smem, int split, int nsplit, int n_tile) {
  {
    const bool swiglu = (p.flags & GEMM_SWIGLU) != 0;
    const int outw = swiglu ? 64 : 128;
    const int per = outw / nsplit;           // columns owned by this CTA (>= 8)
    const int vec_per_row = per >> 2;
    const int items = p.M * vec_per_row;
    const uint32_t P_addr = smem_u32(smem);
    for (int it = threadIdx.x; it < items; it += blockDim.x) {
      const int j = it / vec_per_row;
      const int c = split * per + (it - j * vec_per_row) * 4;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f), acc2 = acc;
      for (int s = 0; s < nsplit; ++s) {
        const uint32_t ra = mapa_u32(P_addr + (uint32_t)(j * 128 + c) * 4u, (uint32_t)s);
        float4 v = ld_dsmem_f4(ra);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        if (swiglu) {
          float4 u = ld_dsmem_f4(ra + 64 * 4);
          acc2.x += u.x; acc2.y += u.y; acc2.z += u.z; acc2.w += u.w;
        }
      }
      int n_out;
      if (swiglu) {
        n_out = n_tile * 64 + c;
        if (p.flags & GEMM_BIAS) {
          const uint32_t* bg = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.bias) + n_tile * 128 + c);
          float2 b0 = unpack_16<BF16>(bg[0]), b1 = unpack_16<BF16>(bg[1]);
          float2 u0 = unpack_16<BF16>(bg[32]), u1 = unpack_16<BF16>(bg[33]);
          acc.x += b0.x; acc.y += b0.y; acc.z += b1.x; acc.w += b1.y;
          acc2.x += u0.x; acc2.y += u0.y; acc2.z += u1.x; acc2.w += u1.y;
        }
        acc.x = silu_f(acc.x) * acc2.x; acc.y = silu_f(acc.y) * acc2.y;
        acc.z = silu_f(acc.z) * acc2.z; acc.w = silu_f(acc.w) * acc2.w;
        if (n_out >= (p.N >> 1)) continue;
      } else {
        n_out = n_tile * 128 + c;
        if (n_out >= p.N) continue;
        if (p.flags & GEMM_BIAS) {
          const uint32_t* bp = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.bias) + n_out);
          float2 b0 = unpack_16<BF16>(bp[0]), b1 = unpack_16<BF16>(bp[1]);
          acc.x += b0.x; acc.y += b0.y; acc.z += b1.x; acc.w += b1.y;
        }
      }
      if (p.flags & GEMM_RESIDUAL) {
        const uint2 rv = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(p.residual) + (size_t)j * p.ld_res + n_out);
        float2 r0 = unpack_16<BF16>(rv.x), r1 = unpack_16<BF16>(rv.y);
        acc.x += r0.x; acc.y += r0.y; acc.z += r1.x; acc.w += r1.y;
      }
      const size_t zo = (size_t)blockIdx.z * (size_t)p.batch_out_cols;
      if (p.scatter_tp > 0) {
        float* dst = p.scatter_out[j / p.scatter_rows] + ((size_t)p.scatter_rank * p.M + j) * p.ld_out + n_out;
        *reinterpret_cast<float4*>(dst) = acc;
      } else if (p.flags & GEMM_OUT_F32) {
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + (size_t)j * p.ld_out + zo + n_out) = acc;
      } else {
        uint2 o;
        o.x = pack_16<BF16>(acc.x, acc.y);
        o.y = pack_16<BF16>(acc.z, acc.w);
        *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(p.out) + (size_t)j * p.ld_out + zo + n_out) = o;
      }
    }
  }
}

// Default epilogue: column slices, bias -> SwiGLU -> residual -> store / scatter.
template <bool BF16>
struct StoreEpilogue {
  __device__ __forceinline__ void operator()(const GemmParams& p, uint8_t* smem, int split, int nsplit, int n_tile) const {
    smallm_reduce_store<BF16>(p, smem, split, nsplit, n_tile);
  }
};

// Epilogue of the QKV projection for head_dim 128: one 128-wide output tile is exactly one head, so everything the reference
// does in a separate launch after the projection (split, per-head RMSNorm of Q and K, RoPE, K/V rows into their cache pages,
// Q to its buffer: QKVRMSNormRopeSplitAppendPagedCache, src/devices/cuda/fastllm-cuda.cu:12190) happens here on the fp32 tile.
// The k-split reduction is by token rows (a warp owns a row, a lane four consecutive dims), so a head's 128 values of one
// token are in one warp.  Values are rounded to the 16-bit dtype at the points where the unfused sequence stores them
// (projection output, norm output), which keeps the two paths bit-compatible.
struct QkvEpilogueParams {
  uint16_t* q_out; int ld_q;
  uint16_t* k_pool; uint16_t* v_pool;
  const int* positions; const int* slots;
  const uint16_t* q_norm_w; const uint16_t* k_norm_w;
  const float* cos_tab; const float* sin_tab;
  int Hq, Hkv, rot, rope_mode;         // rope_mode: 0 none, 1 neox (i pairs with i + rot/2), 2 interleaved (2i, 2i+1)
  float eps, norm_unit_offset;
};

template <bool BF16>
struct QkvEpilogue {
  QkvEpilogueParams q;
  __device__ __forceinline__ void operator()(const GemmParams& p, uint8_t* smem, int split, int nsplit, int n_tile) const {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const uint32_t P_addr = smem_u32(smem);
    const int rows_per = (p.M + nsplit - 1) / nsplit;
    const int r0 = split * rows_per;
    int r1 = r0 + rows_per; if (r1 > p.M) r1 = p.M;
    const int head = n_tile;
    const bool is_q = head < q.Hq, is_k = !is_q && head < q.Hq + q.Hkv;
    const uint16_t* nw = is_q ? q.q_norm_w : (is_k ? q.k_norm_w : nullptr);
    const int half = q.rot >> 1;
    const int e0 = lane * 4;
    for (int j = r0 + warp; j < r1; j += nwarps) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < nsplit; ++s) {
        const float4 v = ld_dsmem_f4(mapa_u32(P_addr + (uint32_t)(j * 128 + e0) * 4u, (uint32_t)s));
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      if (p.flags & GEMM_BIAS) {
        const uint32_t* bp = reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint16_t*>(p.bias) + n_tile * 128 + e0);
        const float2 b0 = unpack_16<BF16>(bp[0]), b1 = unpack_16<BF16>(bp[1]);
        acc.x += b0.x; acc.y += b0.y; acc.z += b1.x; acc.w += b1.y;
      }
      // the projection's output as it would have been stored
      float2 t0 = unpack_16<BF16>(pack_16<BF16>(acc.x, acc.y)), t1 = unpack_16<BF16>(pack_16<BF16>(acc.z, acc.w));
      float v[4] = {t0.x, t0.y, t1.x, t1.y};
      if (nw != nullptr) {
        float ss = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = rsqrtf(ss / 128.0f + q.eps);
        const uint32_t* wp = reinterpret_cast<const uint32_t*>(nw + e0);
        const float2 w0 = unpack_16<BF16>(wp[0]), w1 = unpack_16<BF16>(wp[1]);
        t0 = unpack_16<BF16>(pack_16<BF16>(v[0] * inv * (w0.x + q.norm_unit_offset), v[1] * inv * (w0.y + q.norm_unit_offset)));
        t1 = unpack_16<BF16>(pack_16<BF16>(v[2] * inv * (w1.x + q.norm_unit_offset), v[3] * inv * (w1.y + q.norm_unit_offset)));
        v[0] = t0.x; v[1] = t0.y; v[2] = t1.x; v[3] = t1.y;
      }
      if ((is_q || is_k) && q.rope_mode != 0) {
        const int pos = q.positions[j];
        const float* ct = q.cos_tab + (size_t)pos * half;
        const float* st = q.sin_tab + (size_t)pos * half;
        if (q.rope_mode == 2) {
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const int i = lane * 2 + k;          // pair index
            if (i < half) {
              const float c = ct[i], sn = st[i], a = v[2 * k], b = v[2 * k + 1];
              v[2 * k] = a * c - b * sn;
              v[2 * k + 1] = a * sn + b * c;
            }
          }
        } else {
          // neox; rot is a multiple of 8, so a lane's four dims lie on one side and its partner lane holds the other side
          const int hl = half >> 2;              // lanes per half
          const bool first = e0 < half, in_rot = e0 < q.rot;
          const int partner = first ? lane + hl : lane - hl;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float other = __shfl_sync(0xffffffffu, v[k], in_rot ? (partner & 31) : lane);
            if (in_rot) {
              const int f = (first ? e0 : e0 - half) + k;
              const float c = ct[f], sn = st[f];
              v[k] = first ? v[k] * c - other * sn : v[k] * c + other * sn;
            }
          }
        }
      }
      uint16_t* dst;
      if (is_q) {
        dst = q.q_out + (size_t)j * q.ld_q + (size_t)head * 128;
      } else {
        const int slot = q.slots[j];
        if (slot < 0) continue;                  // warp-uniform: the whole warp works on row j
        const int kvh = is_k ? head - q.Hq : head - q.Hq - q.Hkv;
        dst = (is_k ? q.k_pool : q.v_pool) + ((size_t)slot * q.Hkv + kvh) * 128;
      }
      uint2 o;
      o.x = pack_16<BF16>(v[0], v[1]);
      o.y = pack_16<BF16>(v[2], v[3]);
      *reinterpret_cast<uint2*>(dst + e0) = o;
    }
  }
};

// Body of the small-M kernel.  Returns with the output tile written and every cluster peer done reading this
// CTA's shared memory; the caller still owns TMEM (returned in tmem_base_out) and must release it from warp 1.
template <int MPAD, bool BF16, int OCC = 1, class Epi = StoreEpilogue<BF16>>
__device__ __forceinline__ void gemm_smallm_device(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p,
                                                   uint32_t& tmem_base_out, int kernel_id, const Epi& epi = Epi()) {
  using Cfg = SmallMCfg<MPAD, OCC>;
  const int KID_GEMM_SMALLM = kernel_id;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + Cfg::BODY_BYTES);
  uint64_t* empty_bar = full_bar + Cfg::STAGES;
  uint64_t* accum_bar = empty_bar + Cfg::STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);

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
    for (int s = 0; s < Cfg::STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
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
      const int w_row = p.w_row0 + (int)blockIdx.z * p.batch_w_rows + n_tile * 128;
      const int x_col0 = (int)blockIdx.z * p.batch_x_cols;     // a multiple of 8 elements (16 bytes), checked by the launcher
      // Weights do not depend on the kernel before this one: the first ring of weight tiles is requested before the
      // dependency wait, so the weight stream starts while that kernel drains.  Activations follow the wait.
      const int pre = kb_cnt < Cfg::STAGES ? kb_cnt : Cfg::STAGES;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(&full_bar[i], Cfg::STAGE_BYTES);
        tma_load_2d_hint(smem + i * Cfg::STAGE_BYTES, &tmW, &full_bar[i], (kb0 + i) * 64, w_row, pol_w);
      }
      pdl_wait();
      if (p.wait_cnt != nullptr) {
        // the expect word was written by the kernel before this one and is final after the dependency wait
        const uint32_t target = *reinterpret_cast<const volatile uint32_t*>(p.wait_expect);
        wait_counter_ge(p.wait_cnt, target, KID_GEMM_SMALLM, 9);      // on expiry: reported; the tile is computed from what is there
        fence_proxy_async_global();
      }
      for (int i = 0; i < pre; ++i)
        tma_load_2d_hint(smem + i * Cfg::STAGE_BYTES + Cfg::A_BYTES, &tmX, &full_bar[i], x_col0 + (kb0 + i) * 64, p.x_row0, pol_x);
      for (int i = pre; i < kb_cnt; ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u;
        if (!mbar_wait(&empty_bar[s], ph ^ 1u, dead, KID_GEMM_SMALLM, 1)) break;
        uint8_t* a = smem + s * Cfg::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], Cfg::STAGE_BYTES);
        tma_load_2d_hint(a, &tmW, &full_bar[s], (kb0 + i) * 64, w_row, pol_w);
        tma_load_2d_hint(a + Cfg::A_BYTES, &tmX, &full_bar[s], x_col0 + (kb0 + i) * 64, p.x_row0, pol_x);
      }
    }
    __syncwarp();
    pdl_wait();
  } else if (warp == 1) {
    pdl_wait();
    if (elect_one()) {
      for (int i = 0; i < kb_cnt; ++i) {
        const int s = i % Cfg::STAGES;
        const uint32_t ph = (uint32_t)(i / Cfg::STAGES) & 1u;
        if (!mbar_wait(&full_bar[s], ph, dead, KID_GEMM_SMALLM, 2)) break;
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(smem + s * Cfg::STAGE_BYTES);
        const uint64_t da = make_smem_desc(a_addr, 16, 1024, SWZ_128B);
        const uint64_t db = make_smem_desc(a_addr + Cfg::A_BYTES, 16, 1024, SWZ_128B);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16(tmem_base, da + 2 * k, db + 2 * k, p.idesc, (i | k) != 0 ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(accum_bar);
    }
    __syncwarp();
  } else {
    // epilogue warps 2..5: TMEM lanes [32q, 32q+32) -> fp32 partial tile P[token][n] in shared memory
    const int q = warp & 3;
    float* P = reinterpret_cast<float*>(smem);
    const int n_local = q * 32 + lane;
    pdl_wait();
    if (kb_cnt > 0) {
      mbar_wait(accum_bar, 0, dead, KID_GEMM_SMALLM, 3);
      tc_fence_after_sync();
      constexpr int CH = MPAD < 32 ? MPAD : 32;
#pragma unroll 1
      for (int c0 = 0; c0 < MPAD; c0 += CH) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c0;
        if (CH == 32) tmem_ld_32x32b_x32(taddr, r); else tmem_ld_32x32b_x16(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < CH; ++j) P[(c0 + j) * 128 + n_local] = __uint_as_float(r[j]);
      }
    } else {
      for (int j = 0; j < MPAD; ++j) P[j * 128 + n_local] = 0.f;
    }
  }
  tc_fence_before_sync();
  cluster_sync_all();

  epi(p, smem, split, nsplit, n_tile);
  cluster_sync_all();   // peers may still be reading this CTA's partial tile
  tmem_base_out = tmem_base;
}

}  // namespace fb
