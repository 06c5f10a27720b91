// Bandwidth-bound row kernels for sm_100a: RMSNorm (+ residual), fused QKV post-processing
// (per-head RMSNorm + RoPE + paged-KV append), SiLU-mul, embedding gather, greedy arg-max, top-k router.
// All use 128-bit global accesses and fp32 math.
//
// Reference behaviour reproduced here:
//   RMSNorm                              src/devices/cuda/fastllm-cuda.cu:2733-3085
//   QKVRMSNormRopeSplitAppendPagedCache  src/devices/cuda/fastllm-cuda.cu:12190
//   Swiglu                               src/devices/cuda/fastllm-cuda.cu:1704-1727
//   greedy sampling                      src/devices/cuda/fastllm-cuda.cu:13579-13784
//   SelectExpert                         src/devices/cpu/cpudevice.cpp:8885-8955
#include "ptx.cuh"
#include "launch.h"

FB_DEFINE_ERROR_API(elementwise)

namespace fb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = l < nw ? sh[l] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm:  if residual != nullptr:  residual = residual + x (written back), y = norm(residual) * w
//           else                      y = norm(x) * w.        One CTA per row, H % 8 == 0.
// `unit_offset` adds 1 to the weight (Gemma convention).
// ------------------------------------------------------------------------------------------------
// Optional second output for the 8-bit-activation GEMMs that consume the normalised row: the row quantised per 128-wide block
// (QMODE 1: int8 with scale amax / 127 and the block sums of the quantised values; QMODE 2: e4m3 with scale amax / 448),
// computed from the 16-bit-rounded outputs so that it equals what the stand-alone quantiser would produce from y.
struct NormQuantOut {
  uint8_t* xq; int ldq;          // [M, H] bytes
  float* scales; float* sums;    // [H / 128, ld_a]
  int ld_a;
};

template <bool BF16, int QMODE = 0>
__global__ void rmsnorm_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w, uint16_t* __restrict__ y,
                               uint16_t* residual, int H, int ldx, int ldy, float eps, float unit_offset, NormQuantOut qo = {}) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sh[32];
  extern __shared__ float rowbuf[];   // H floats
  const int row = blockIdx.x;
  const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)row * ldx);
  uint4* rp = residual ? reinterpret_cast<uint4*>(residual + (size_t)row * H) : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    uint4 v = xp[i];
    float2 a = unpack_16<BF16>(v.x), b = unpack_16<BF16>(v.y), c = unpack_16<BF16>(v.z), d = unpack_16<BF16>(v.w);
    if (rp) {
      uint4 r = rp[i];
      float2 ra = unpack_16<BF16>(r.x), rb = unpack_16<BF16>(r.y), rc = unpack_16<BF16>(r.z), rd = unpack_16<BF16>(r.w);
      a.x += ra.x; a.y += ra.y; b.x += rb.x; b.y += rb.y; c.x += rc.x; c.y += rc.y; d.x += rd.x; d.y += rd.y;
      uint4 o;
      o.x = pack_16<BF16>(a.x, a.y); o.y = pack_16<BF16>(b.x, b.y); o.z = pack_16<BF16>(c.x, c.y); o.w = pack_16<BF16>(d.x, d.y);
      rp[i] = o;
      // keep the rounded value so that the norm sees exactly what later layers will read
      a = unpack_16<BF16>(o.x); b = unpack_16<BF16>(o.y); c = unpack_16<BF16>(o.z); d = unpack_16<BF16>(o.w);
    }
    float* rb_ = rowbuf + i * 8;
    rb_[0] = a.x; rb_[1] = a.y; rb_[2] = b.x; rb_[3] = b.y; rb_[4] = c.x; rb_[5] = c.y; rb_[6] = d.x; rb_[7] = d.y;
    ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + d.x * d.x + d.y * d.y;
  }
  ss = block_sum(ss, sh);
  const float inv = rsqrtf(ss / (float)H + eps);
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  uint4* yp = reinterpret_cast<uint4*>(y + (size_t)row * ldy);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    uint4 wv = wp[i];
    float2 wa = unpack_16<BF16>(wv.x), wb = unpack_16<BF16>(wv.y), wc = unpack_16<BF16>(wv.z), wd = unpack_16<BF16>(wv.w);
    const float* r = rowbuf + i * 8;
    uint4 o;
    o.x = pack_16<BF16>(r[0] * inv * (wa.x + unit_offset), r[1] * inv * (wa.y + unit_offset));
    o.y = pack_16<BF16>(r[2] * inv * (wb.x + unit_offset), r[3] * inv * (wb.y + unit_offset));
    o.z = pack_16<BF16>(r[4] * inv * (wc.x + unit_offset), r[5] * inv * (wc.y + unit_offset));
    o.w = pack_16<BF16>(r[6] * inv * (wd.x + unit_offset), r[7] * inv * (wd.y + unit_offset));
    yp[i] = o;
    if (QMODE != 0) {
      // 16 consecutive threads hold one 128-wide block (H % 128 == 0: a half-warp is inside the row or outside as a whole)
      const uint32_t mask = (threadIdx.x & 16) ? 0xFFFF0000u : 0x0000FFFFu;
      const float2 a = unpack_16<BF16>(o.x), b = unpack_16<BF16>(o.y), c = unpack_16<BF16>(o.z), d = unpack_16<BF16>(o.w);
      float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                         fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
#pragma unroll
      for (int sft = 8; sft > 0; sft >>= 1) amax = fmaxf(amax, __shfl_xor_sync(mask, amax, sft));
      const int kb = i >> 4;
      uint2 q;
      if (QMODE == 3 || QMODE == 4) {
        // y itself rounded to the int8 (3) / e4m3 (4) grid of its block: what a large batch feeds to the 16-bit-activation
        // kernels of a layer whose small batches run on 8-bit activations
        float v[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
        if (QMODE == 3) {
          const float scale = fmaxf(amax, 1e-12f) / 127.0f, iv = 1.0f / scale;
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = rintf(v[e] * iv) * scale;
        } else {
          const float scale = fmaxf(amax, 1e-12f) / 448.0f, iv = 1.0f / scale;
          const uint32_t p0 = pack_e4m3x4(v[0] * iv, v[1] * iv, v[2] * iv, v[3] * iv), p1 = pack_e4m3x4(v[4] * iv, v[5] * iv, v[6] * iv, v[7] * iv);
          const uint32_t pk[2] = {p0, p1};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            uint32_t h;
            asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h) : "h"((uint16_t)(pk[e >> 1] >> (16 * (e & 1)))));
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
            v[2 * e] = f.x * scale; v[2 * e + 1] = f.y * scale;
          }
        }
        uint4 ro;
        ro.x = pack_16<BF16>(v[0], v[1]); ro.y = pack_16<BF16>(v[2], v[3]); ro.z = pack_16<BF16>(v[4], v[5]); ro.w = pack_16<BF16>(v[6], v[7]);
        yp[i] = ro;
        continue;
      }
      if (QMODE == 1) {
        const float scale = fmaxf(amax, 1e-12f) / 127.0f, iv = 1.0f / scale;
        const int q0 = __float2int_rn(a.x * iv), q1 = __float2int_rn(a.y * iv), q2 = __float2int_rn(b.x * iv), q3 = __float2int_rn(b.y * iv);
        const int q4 = __float2int_rn(c.x * iv), q5 = __float2int_rn(c.y * iv), q6 = __float2int_rn(d.x * iv), q7 = __float2int_rn(d.y * iv);
        q.x = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
        q.y = (uint32_t)(q4 & 0xFF) | ((uint32_t)(q5 & 0xFF) << 8) | ((uint32_t)(q6 & 0xFF) << 16) | ((uint32_t)(q7 & 0xFF) << 24);
        int sm = q0 + q1 + q2 + q3 + q4 + q5 + q6 + q7;
#pragma unroll
        for (int sft = 8; sft > 0; sft >>= 1) sm += __shfl_xor_sync(mask, sm, sft);
        if ((threadIdx.x & 15) == 0) {
          qo.scales[(size_t)kb * qo.ld_a + row] = scale;
          qo.sums[(size_t)kb * qo.ld_a + row] = (float)sm;
        }
      } else {
        const float scale = fmaxf(amax, 1e-12f) / 448.0f, iv = 1.0f / scale;
        q.x = pack_e4m3x4(a.x * iv, a.y * iv, b.x * iv, b.y * iv);
        q.y = pack_e4m3x4(c.x * iv, c.y * iv, d.x * iv, d.y * iv);
        if ((threadIdx.x & 15) == 0) qo.scales[(size_t)kb * qo.ld_a + row] = scale;
      }
      *reinterpret_cast<uint2*>(qo.xq + (size_t)row * qo.ldq + i * 8) = q;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// QKV post-processing, one warp per (token, head):
//   q heads : optional per-head RMSNorm, RoPE, write to q_out [M, Hq*D]
//   k heads : optional per-head RMSNorm, RoPE, write to the K page pool at slot[token]
//   v heads : copy to the V page pool at slot[token]
// cos/sin tables are fp32 [max_pos, rot/2].  rope_mode: 0 none, 1 neox (rotate-half), 2 interleaved pairs.
// Page pools are [num_slots, Hkv, D] (slot = page * page_len + offset).  slot < 0 skips the cache write.
// ------------------------------------------------------------------------------------------------
struct QkvPostParams {
  const uint16_t* qkv; int ld_qkv;
  uint16_t* q_out; int ld_q;
  uint16_t* k_pool; uint16_t* v_pool;
  const int* positions; const int* slots;
  const uint16_t* q_norm_w; const uint16_t* k_norm_w;
  const float* cos_tab; const float* sin_tab;
  int M, Hq, Hkv, D, rot, rope_mode;
  float eps; float norm_unit_offset;
  // e4m3 page pools: K / V rows are stored as unscaled e4m3 bytes (the 16-bit value rounded once more), and the queries are
  // also written as two e4m3 terms q = a + b / 16 for the fp8 tensor-core decode attention ([M, Hq * D] bytes each, or null)
  int kv8; uint8_t* q8a; uint8_t* q8b;
};

__device__ __forceinline__ unsigned short e4m3x2_of(float lo, float hi) {
  unsigned short r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float2 e4m3x2_to_f2(unsigned short v) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h) : "h"(v));
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

template <bool BF16>
__global__ void qkv_post_kernel(const QkvPostParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps_per_block = blockDim.x >> 5;
  const int gw = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int heads = p.Hq + 2 * p.Hkv;
  if (gw >= p.M * heads) return;
  const int tok = gw / heads, head = gw - tok * heads;
  const uint16_t* src = p.qkv + (size_t)tok * p.ld_qkv + (size_t)head * p.D;
  const int D = p.D, half = p.rot >> 1;
  // each lane owns element pairs (2i, 2i+1) for i = lane, lane+32, ... (D <= 512)
  float v[16];
  const int npairs = D >> 1;
  int cnt = 0;
  float ss = 0.f;
  for (int i = lane; i < npairs; i += 32, ++cnt) {
    float2 f = unpack_16<BF16>(*reinterpret_cast<const uint32_t*>(src + 2 * i));
    v[2 * cnt] = f.x; v[2 * cnt + 1] = f.y;
    ss += f.x * f.x + f.y * f.y;
  }
  const bool is_q = head < p.Hq, is_k = !is_q && head < p.Hq + p.Hkv;
  const uint16_t* nw = is_q ? p.q_norm_w : (is_k ? p.k_norm_w : nullptr);
  if (nw) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)D + p.eps);
    cnt = 0;
    for (int i = lane; i < npairs; i += 32, ++cnt) {
      float2 w = unpack_16<BF16>(*reinterpret_cast<const uint32_t*>(nw + 2 * i));
      // round to the storage dtype after the norm, as a separate norm op would
      float2 r = unpack_16<BF16>(pack_16<BF16>(v[2 * cnt] * inv * (w.x + p.norm_unit_offset),
                                               v[2 * cnt + 1] * inv * (w.y + p.norm_unit_offset)));
      v[2 * cnt] = r.x; v[2 * cnt + 1] = r.y;
    }
  }
  uint16_t* dst;
  uint8_t* dst8 = nullptr;
  if (is_q) {
    dst = p.q_out + (size_t)tok * p.ld_q + (size_t)head * D;
  } else {
    const int slot = p.slots[tok];
    if (slot < 0) return;
    const int kvh = is_k ? head - p.Hq : head - p.Hq - p.Hkv;
    dst = (is_k ? p.k_pool : p.v_pool) + ((size_t)slot * p.Hkv + kvh) * D;
    if (p.kv8) dst8 = reinterpret_cast<uint8_t*>(is_k ? p.k_pool : p.v_pool) + ((size_t)slot * p.Hkv + kvh) * D;
  }
  if ((is_q || is_k) && p.rope_mode != 0) {
    const int pos = p.positions[tok];
    const float* ct = p.cos_tab + (size_t)pos * half;
    const float* st = p.sin_tab + (size_t)pos * half;
    if (p.rope_mode == 2) {
      // interleaved: pair (2i, 2i+1) rotates with frequency i
      cnt = 0;
      for (int i = lane; i < npairs; i += 32, ++cnt) {
        if (i < half) {
          const float c = ct[i], s = st[i];
          const float a = v[2 * cnt], b = v[2 * cnt + 1];
          v[2 * cnt] = a * c - b * s;
          v[2 * cnt + 1] = a * s + b * c;
        }
      }
    } else {
      // neox: element j < half pairs with j + half.  Lane's pair index i covers elements 2i, 2i+1; the partner
      // elements 2i + half, 2i + 1 + half belong to pair index i + half/2, owned by lane (i + half/2) % 32.
      // half/2 is a multiple of 32 for D = 128 / rot = 128 (half = 64, half/2 = 32) -> same lane, next slot.
      // General case goes through shared-free shuffles: handled by staging via registers only when half/2 % 32 == 0,
      // otherwise fall back to a shuffle exchange.
      const int hp = half >> 1;  // number of pairs in the first half
      if ((hp & 31) == 0) {
        const int step = hp >> 5;  // register slots between an element and its partner
        cnt = 0;
        for (int i = lane; i < hp; i += 32, ++cnt) {
          const float c0 = ct[2 * i], s0 = st[2 * i], c1 = ct[2 * i + 1], s1 = st[2 * i + 1];
          const float a0 = v[2 * cnt], a1 = v[2 * cnt + 1];
          const float b0 = v[2 * (cnt + step)], b1 = v[2 * (cnt + step) + 1];
          v[2 * cnt] = a0 * c0 - b0 * s0;
          v[2 * cnt + 1] = a1 * c1 - b1 * s1;
          v[2 * (cnt + step)] = b0 * c0 + a0 * s0;
          v[2 * (cnt + step) + 1] = b1 * c1 + a1 * s1;
        }
      } else {
        // partner pair index = i + hp (first half) or i - hp (second half); owner lane = partner % 32, slot = partner / 32
        const int total_slots = (npairs + 31) >> 5;
        float nv[16];
        for (int s = 0; s < total_slots; ++s) { nv[2 * s] = v[2 * s]; nv[2 * s + 1] = v[2 * s + 1]; }
        for (int s = 0; s < total_slots; ++s) {
          const int i = lane + 32 * s;
          const bool in_rot = i < 2 * hp;
          const int partner = i < hp ? i + hp : i - hp;
          for (int ps = 0; ps < total_slots; ++ps) {
            // every lane publishes slot ps; readers pick the lane they need
            const float px = __shfl_sync(0xffffffffu, v[2 * ps], partner & 31);
            const float py = __shfl_sync(0xffffffffu, v[2 * ps + 1], partner & 31);
            if (in_rot && i < npairs && (partner >> 5) == ps) {
              const int f = 2 * (i < hp ? i : i - hp);
              const float c0 = ct[f], s0 = st[f], c1 = ct[f + 1], s1 = st[f + 1];
              if (i < hp) { nv[2 * s] = v[2 * s] * c0 - px * s0; nv[2 * s + 1] = v[2 * s + 1] * c1 - py * s1; }
              else        { nv[2 * s] = v[2 * s] * c0 + px * s0; nv[2 * s + 1] = v[2 * s + 1] * c1 + py * s1; }
            }
          }
        }
        for (int s = 0; s < total_slots; ++s) { v[2 * s] = nv[2 * s]; v[2 * s + 1] = nv[2 * s + 1]; }
      }
    }
  }
  cnt = 0;
  if (dst8 != nullptr) {
    for (int i = lane; i < npairs; i += 32, ++cnt) {
      const float2 r = unpack_16<BF16>(pack_16<BF16>(v[2 * cnt], v[2 * cnt + 1]));
      *reinterpret_cast<unsigned short*>(dst8 + 2 * i) = e4m3x2_of(r.x, r.y);
    }
    return;
  }
  for (int i = lane; i < npairs; i += 32, ++cnt)
    *reinterpret_cast<uint32_t*>(dst + 2 * i) = pack_16<BF16>(v[2 * cnt], v[2 * cnt + 1]);
  if (is_q && p.q8a != nullptr) {
    uint8_t* da = p.q8a + ((size_t)tok * p.Hq + head) * D;
    uint8_t* db = p.q8b + ((size_t)tok * p.Hq + head) * D;
    cnt = 0;
    for (int i = lane; i < npairs; i += 32, ++cnt) {
      const float2 r = unpack_16<BF16>(pack_16<BF16>(v[2 * cnt], v[2 * cnt + 1]));
      const unsigned short a8 = e4m3x2_of(r.x, r.y);
      const float2 af = e4m3x2_to_f2(a8);
      *reinterpret_cast<unsigned short*>(da + 2 * i) = a8;
      *reinterpret_cast<unsigned short*>(db + 2 * i) = e4m3x2_of((r.x - af.x) * 16.0f, (r.y - af.y) * 16.0f);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Multi-head latent attention, post-processing of the projections of one token (one CTA per token):
//   latent row  ckv[t, :lora]  -> RMSNorm -> cache entry [0, lora)
//   shared key  ckv[t, lora:]  -> RoPE    -> cache entry [lora, lora + rope)           (slot < 0: the spare last slot)
//   query rope  q[t, h, nope:] -> RoPE    -> q_full[t, h, lora:]   for every head
// The reference runs these as separate operators (RMSNorm, NearlyRotatePosition2D, cache append; src/models/deepseekv2.cpp:283-697).
// ------------------------------------------------------------------------------------------------
struct MlaPostParams {
  const uint16_t* ckv; int ld_ckv;
  const uint16_t* q; int ld_q;             // [T, H * (nope + rope)]
  uint16_t* q_full; int ld_qf;             // [T, H * (lora + rope)]
  uint16_t* pool;                          // [slots, lora + rope]
  const int* positions; const int* slots;
  const uint16_t* norm_w;
  const float* cos_tab; const float* sin_tab;
  int H, nope, rope, lora, rope_mode, spare_slot;
  float eps;
};

template <bool BF16>
__device__ __forceinline__ void mla_rope_pair(const uint16_t* src, uint16_t* dst, int i, int half, int mode, const float* ct, const float* st) {
  // pair index i < half: interleaved rotates (2i, 2i+1); neox rotates (i, i + half)
  const int a_idx = mode == 2 ? 2 * i : i, b_idx = mode == 2 ? 2 * i + 1 : i + half;
  const float a = BF16 ? __bfloat162float(__ushort_as_bfloat16(src[a_idx])) : __half2float(__ushort_as_half(src[a_idx]));
  const float b = BF16 ? __bfloat162float(__ushort_as_bfloat16(src[b_idx])) : __half2float(__ushort_as_half(src[b_idx]));
  const float c = ct[i], sn = st[i];
  const float ra = a * c - b * sn, rb = mode == 2 ? a * sn + b * c : b * c + a * sn;
  dst[a_idx] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(ra)) : __half_as_ushort(__float2half_rn(ra));
  dst[b_idx] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(rb)) : __half_as_ushort(__float2half_rn(rb));
}

template <bool BF16>
__global__ void mla_post_kernel(const MlaPostParams p) {
  __shared__ float red[8];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x, nthr = blockDim.x;
  const uint16_t* row = p.ckv + (size_t)t * p.ld_ckv;
  int slot = p.slots[t];
  if (slot < 0) slot = p.spare_slot;
  uint16_t* entry = p.pool + (size_t)slot * (p.lora + p.rope);
  // latent RMSNorm
  float ss = 0.f;
  for (int i = tid; i < p.lora; i += nthr) {
    const float v = BF16 ? __bfloat162float(__ushort_as_bfloat16(row[i])) : __half2float(__ushort_as_half(row[i]));
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (nthr >> 5); ++w) tot += red[w];
  const float inv = rsqrtf(tot / (float)p.lora + p.eps);
  for (int i = tid; i < p.lora; i += nthr) {
    const float v = BF16 ? __bfloat162float(__ushort_as_bfloat16(row[i])) : __half2float(__ushort_as_half(row[i]));
    const float w = BF16 ? __bfloat162float(__ushort_as_bfloat16(p.norm_w[i])) : __half2float(__ushort_as_half(p.norm_w[i]));
    const float y = v * inv * w;
    entry[i] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(y)) : __half_as_ushort(__float2half_rn(y));
  }
  // rotary parts
  const int half = p.rope >> 1;
  const int pos = p.positions[t];
  const float* ct = p.cos_tab + (size_t)pos * half;
  const float* st = p.sin_tab + (size_t)pos * half;
  const int total = (p.H + 1) * half;          // head index H = the shared key
  for (int it = tid; it < total; it += nthr) {
    const int h = it / half, i = it - h * half;
    if (h == p.H) {
      mla_rope_pair<BF16>(row + p.lora, entry + p.lora, i, half, p.rope_mode, ct, st);
    } else {
      const uint16_t* src = p.q + (size_t)t * p.ld_q + (size_t)h * (p.nope + p.rope) + p.nope;
      uint16_t* dst = p.q_full + (size_t)t * p.ld_qf + (size_t)h * (p.lora + p.rope) + p.lora;
      mla_rope_pair<BF16>(src, dst, i, half, p.rope_mode, ct, st);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// SiLU(gate) * up :  x [M, 2I] (gate | up) -> y [M, I]
// ------------------------------------------------------------------------------------------------
template <bool BF16>
__global__ void silu_mul_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y, int M, int I, int ldx, int ldy) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)M * (I / 8);
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(idx / (I / 8)), c = (int)(idx % (I / 8)) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + c);
    const uint4 u = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + I + c);
    const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = unpack_16<BF16>(gs[k]), b = unpack_16<BF16>(us[k]);
      o[k] = pack_16<BF16>(a.x / (1.f + __expf(-a.x)) * b.x, a.y / (1.f + __expf(-a.y)) * b.y);
    }
    *reinterpret_cast<uint4*>(y + (size_t)m * ldy + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// act(gate) * up for the other gated MLPs (GeGLU of the Gemma family, ReGLU): ACT 1 = GELU tanh approximation, 2 = GELU (erf),
// 3 = ReLU, 0 = SiLU.  Two layouts of x [M, 2I]: gate | up halves, or interleaved per 128 columns (64 gate, 64 up), the layout
// the fused gate/up weights are stored in.  The reference runs these as separate Gelu / Mul launches
// (src/devices/cuda/fastllm-cuda.cu GeluNew / MulTo kernels).
// ------------------------------------------------------------------------------------------------
template <int ACT>
__device__ __forceinline__ float glu_act(float v) {
  if (ACT == 1) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  if (ACT == 2) return 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
  if (ACT == 3) return v > 0.f ? v : 0.f;
  return v / (1.f + __expf(-v));
}
template <bool BF16, int ACT>
__global__ void glu_act_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ y, int M, int I, int ldx, int ldy, int interleaved) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)M * (I / 8);
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(idx / (I / 8)), c = (int)(idx % (I / 8)) * 8;
    const int gc = interleaved ? (c >> 6) * 128 + (c & 63) : c;
    const int uc = interleaved ? gc + 64 : I + c;
    const uint4 g = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + gc);
    const uint4 u = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + uc);
    const uint32_t gs[4] = {g.x, g.y, g.z, g.w}, us[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      float2 a = unpack_16<BF16>(gs[k]), b = unpack_16<BF16>(us[k]);
      o[k] = pack_16<BF16>(glu_act<ACT>(a.x) * b.x, glu_act<ACT>(a.y) * b.y);
    }
    *reinterpret_cast<uint4*>(y + (size_t)m * ldy + c) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ------------------------------------------------------------------------------------------------
// Append new K / V rows to e4m3 page pools: 16-bit rows [T, row_elems] -> unscaled e4m3 (round to nearest even, saturating at
// +-448) at pool row slots[t]; rows with a negative slot (padding of a CUDA-graph bucket) are skipped.
// ------------------------------------------------------------------------------------------------
template <bool BF16>
__global__ void kv_append_fp8_kernel(const uint16_t* __restrict__ k, const uint16_t* __restrict__ v, uint8_t* __restrict__ k_pool,
                                     uint8_t* __restrict__ v_pool, const int* __restrict__ slots, int T, int row_elems) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_row = row_elems >> 3;                      // 8 values per thread
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)T * per_row * 2) return;
  const int which = (int)(idx / ((long long)T * per_row));  // 0: K, 1: V
  const long long rem = idx - (long long)which * T * per_row;
  const int t = (int)(rem / per_row), c = (int)(rem - (long long)t * per_row) * 8;
  const int slot = slots[t];
  if (slot < 0) return;
  const uint16_t* src = (which ? v : k) + (size_t)t * row_elems + c;
  uint8_t* dst = (which ? v_pool : k_pool) + (size_t)slot * row_elems + c;
  const uint4 x = *reinterpret_cast<const uint4*>(src);
  const uint32_t w[4] = {x.x, x.y, x.z, x.w};
  uint32_t o[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = unpack_16<BF16>(w[j]);
    unsigned short pr;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(pr) : "f"(f.y), "f"(f.x));      // first source -> upper byte
    o[j >> 1] |= (uint32_t)pr << ((j & 1) * 16);
  }
  *reinterpret_cast<uint2*>(dst) = make_uint2(o[0], o[1]);
}

// ------------------------------------------------------------------------------------------------
// Causal row softmax for attention evaluated as two GEMMs (MLA prefill: rows = (query, head) pairs, columns = keys):
//   P[r, k] = softmax_k(scale * S[r, k]) over k <= first_pos + r / heads, 0 beyond (also over the padded columns), 16-bit out.
// One CTA per row; the row is read once (held in registers up to 8192 keys, re-read from L2 beyond that).
// ------------------------------------------------------------------------------------------------
template <bool BF16>
__global__ void __launch_bounds__(256) softmax_causal_rows_kernel(const float* __restrict__ S, int lds, uint16_t* __restrict__ P, int ldp,
                                                                  int cols, int heads, int first_pos, float scale) {
  __shared__ float red[8];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, tid = threadIdx.x;
  int limit = first_pos + r / heads + 1;                 // keys [0, limit) are visible
  if (limit > cols) limit = cols;
  const float* row = S + (size_t)r * lds;
  constexpr int CACHE = 32;                              // 256 threads x 32 = 8192 keys in registers
  float v[CACHE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < CACHE; ++i) {
    const int k = tid + i * 256;
    v[i] = k < limit ? row[k] * scale : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  for (int k = tid + CACHE * 256; k < limit; k += 256) mx = fmaxf(mx, row[k] * scale);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if ((tid & 31) == 0) red[tid >> 5] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3])), fmaxf(fmaxf(red[4], red[5]), fmaxf(red[6], red[7])));
  __syncthreads();
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < CACHE; ++i) {
    v[i] = (tid + i * 256) < limit ? __expf(v[i] - mx) : 0.f;
    sum += v[i];
  }
  for (int k = tid + CACHE * 256; k < limit; k += 256) sum += __expf(row[k] * scale - mx);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  if ((tid & 31) == 0) red[tid >> 5] = sum;
  __syncthreads();
  sum = red[0] + red[1] + red[2] + red[3] + red[4] + red[5] + red[6] + red[7];
  const float inv = sum > 0.f ? 1.0f / sum : 0.f;
  uint16_t* out = P + (size_t)r * ldp;
#pragma unroll
  for (int i = 0; i < CACHE; ++i) {
    const int k = tid + i * 256;
    if (k < cols) out[k] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v[i] * inv)) : __half_as_ushort(__float2half_rn(v[i] * inv));
  }
  for (int k = tid + CACHE * 256; k < cols; k += 256) {
    const float pv = k < limit ? __expf(row[k] * scale - mx) * inv : 0.f;
    out[k] = BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(pv)) : __half_as_ushort(__float2half_rn(pv));
  }
}

// ------------------------------------------------------------------------------------------------
// Embedding gather: out[m, :] = table[ids[m], :]
// ------------------------------------------------------------------------------------------------
__global__ void embedding_kernel(const int* __restrict__ ids, const uint16_t* __restrict__ table, uint16_t* __restrict__ out,
                                 int H, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  const int m = blockIdx.x;
  int id = ids[m];
  if (id < 0 || id >= vocab) id = 0;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)m * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

// ------------------------------------------------------------------------------------------------
// Greedy arg-max over logits rows (fp32 or 16-bit); ties resolve to the lowest index.
// Writes ids[m] and, if vals != nullptr, the max logit (used when merging vocab shards across ranks).
// ------------------------------------------------------------------------------------------------
template <int KIND>  // 0 = f32, 1 = bf16, 2 = f16
__global__ void argmax_kernel(const void* __restrict__ logits, int* __restrict__ ids, float* __restrict__ vals, int V, int ld,
                              int id_offset) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sv[32];
  __shared__ int si[32];
  const int m = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  int i0 = 0;
  if (KIND == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {
    // fp32 rows: 16-byte loads, four independent loads in flight per thread (a row is read by one CTA, so the loop has to
    // hide the memory latency itself); indices ascend within a thread, so "greater than" keeps the lowest index of a tie
    const float4* row = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(logits) + (size_t)m * ld);
    const int n4 = V >> 2;
    int j = threadIdx.x;
    for (; j + 3 * (int)blockDim.x < n4; j += 4 * blockDim.x) {
      float4 t[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) t[u] = row[j + u * blockDim.x];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int b = (j + u * blockDim.x) << 2;
        if (t[u].x > best) { best = t[u].x; bi = b; }
        if (t[u].y > best) { best = t[u].y; bi = b + 1; }
        if (t[u].z > best) { best = t[u].z; bi = b + 2; }
        if (t[u].w > best) { best = t[u].w; bi = b + 3; }
      }
    }
    for (; j < n4; j += blockDim.x) {
      const float4 t = row[j];
      const int b = j << 2;
      if (t.x > best) { best = t.x; bi = b; }
      if (t.y > best) { best = t.y; bi = b + 1; }
      if (t.z > best) { best = t.z; bi = b + 2; }
      if (t.w > best) { best = t.w; bi = b + 3; }
    }
    i0 = n4 << 2;
  }
  for (int i = i0 + threadIdx.x; i < V; i += blockDim.x) {
    float x;
    if (KIND == 0) x = reinterpret_cast<const float*>(logits)[(size_t)m * ld + i];
    else if (KIND == 1) x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[(size_t)m * ld + i]);
    else x = __half2float(reinterpret_cast<const __half*>(logits)[(size_t)m * ld + i]);
    if (x > best || (x == best && i < bi)) { best = x; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) { sv[w] = best; si[w] = bi; }
  __syncthreads();
  if (w == 0) {
    const int nw = blockDim.x >> 5;
    best = l < nw ? sv[l] : -INFINITY;
    bi = l < nw ? si[l] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (l == 0) { ids[m] = (bi == 0x7fffffff ? 0 : bi) + id_offset; if (vals) vals[m] = best; }
  }
}

// ------------------------------------------------------------------------------------------------
// Router: scores = softmax / sigmoid / identity of logits [M, E] (fp32), optional bias added for selection
// only, optional group-limited selection (n_group groups, keep topk_group groups ranked by the sum of their
// two best biased scores), top-k, optional renormalisation, times route_scale.  One warp per token, E <= 512.
// ------------------------------------------------------------------------------------------------
struct RouteParams {
  const float* logits; const float* bias; int* out_idx; float* out_w;
  int M, E, topk, score_mode /*0 softmax 1 sigmoid 2 none*/, renorm, n_group, topk_group;
  float route_scale;
};
__global__ void route_topk_kernel(const RouteParams p) {
  pdl_launch_dependents();
  pdl_wait();
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= p.M) return;
  const float* lg = p.logits + (size_t)gw * p.E;
  float sc[16], sel[16];
  const int per = (p.E + 31) >> 5;
  float mx = -INFINITY;
  for (int s = 0; s < per; ++s) { const int e = lane + 32 * s; sc[s] = e < p.E ? lg[e] : -INFINITY; mx = fmaxf(mx, sc[s]); }
  if (p.score_mode == 0) {
    mx = warp_max(mx);
    float sum = 0.f;
    for (int s = 0; s < per; ++s) { const int e = lane + 32 * s; sc[s] = e < p.E ? __expf(sc[s] - mx) : 0.f; sum += sc[s]; }
    sum = warp_sum(sum);
    for (int s = 0; s < per; ++s) sc[s] /= sum;
  } else if (p.score_mode == 1) {
    for (int s = 0; s < per; ++s) sc[s] = 1.f / (1.f + __expf(-sc[s]));
  }
  for (int s = 0; s < per; ++s) {
    const int e = lane + 32 * s;
    sel[s] = e < p.E ? sc[s] + (p.bias ? p.bias[e] : 0.f) : -INFINITY;
  }
  if (p.n_group > 1 && p.topk_group < p.n_group) {
    // group g = e / (E / n_group); score(g) = sum of top-2 biased scores in the group
    const int gs = p.E / p.n_group;
    float gscore[32];
    for (int g = 0; g < p.n_group; ++g) {
      float m1 = -INFINITY, m2 = -INFINITY;
      for (int s = 0; s < per; ++s) {
        const int e = lane + 32 * s;
        if (e < p.E && e / gs == g) { const float x = sel[s]; if (x > m1) { m2 = m1; m1 = x; } else if (x > m2) m2 = x; }
      }
      // merge (m1, m2) across lanes
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, m1, o), o2 = __shfl_xor_sync(0xffffffffu, m2, o);
        const float n1 = fmaxf(m1, o1);
        const float n2 = fmaxf(fminf(m1, o1), fmaxf(m2, o2));
        m1 = n1; m2 = n2;
      }
      gscore[g] = m1 + m2;
    }
    // keep the topk_group best groups (ties to the lower index)
    unsigned keep = 0;
    for (int r = 0; r < p.topk_group; ++r) {
      int bg = -1; float bv = -INFINITY;
      for (int g = 0; g < p.n_group; ++g)
        if (!((keep >> g) & 1u) && (bg < 0 || gscore[g] > bv)) { bg = g; bv = gscore[g]; }
      keep |= 1u << bg;
    }
    for (int s = 0; s < per; ++s) {
      const int e = lane + 32 * s;
      if (e < p.E && !((keep >> (e / gs)) & 1u)) sel[s] = -INFINITY;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f; int my_i = 0;
  for (int k = 0; k < p.topk; ++k) {
    float bv = -INFINITY; int bi = 0x7fffffff; float bs = 0.f;
    for (int s = 0; s < per; ++s) {
      const int e = lane + 32 * s;
      if (e < p.E && (sel[s] > bv || (sel[s] == bv && e < bi))) { bv = sel[s]; bi = e; bs = sc[s]; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const float os = __shfl_xor_sync(0xffffffffu, bs, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; bs = os; }
    }
    if ((bi & 31) == lane) sel[bi >> 5] = -INFINITY;   // remove from further rounds
    wsum += bs;
    if (lane == k) { my_w = bs; my_i = bi; }
  }
  if (lane < p.topk) {
    float w = my_w;
    if (p.renorm) w = w / (wsum + 1e-20f);
    p.out_idx[(size_t)gw * p.topk + lane] = my_i;
    p.out_w[(size_t)gw * p.topk + lane] = w * p.route_scale;
  }
}

}  // namespace fb

using namespace fb;

// RMSNorm that also emits the row quantised for an 8-bit-activation GEMM (mode 1: int8 + scales + block sums, mode 2: e4m3 +
// scales; scale tables [H / 128, ld_a]), or writes y rounded to the int8 (mode 3) / e4m3 (mode 4) grid.  H % 128 == 0.
extern "C" int fb_rmsnorm_quant(const void* x, const void* w, void* y, void* residual, int M, int H, int ldx, int ldy, float eps,
                                float unit_offset, int dtype, int mode, void* xq, int ldq, float* scales, float* sums, int ld_a,
                                void* stream) {
  if (M <= 0) return 0;
  if (H % 128 != 0 || H > 32768 || mode < 1 || mode > 4 || (mode <= 2 && ldq % 8 != 0)) return -1;
  int threads = H / 8;
  threads = threads > 1024 ? 1024 : ((threads + 31) / 32) * 32;
  const size_t smem = (size_t)H * sizeof(float);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  NormQuantOut qo;
  qo.xq = (uint8_t*)xq; qo.ldq = ldq; qo.scales = scales; qo.sums = sums; qo.ld_a = ld_a;
#define FB_NQ(BF, QM)                                                                                                          \
  {                                                                                                                            \
    static DeviceOnce cfg;                                                                                                     \
    if (cfg.need()) { cudaFuncSetAttribute(rmsnorm_kernel<BF, QM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4); }  \
    launch_k(rmsnorm_kernel<BF, QM>, dim3(M), dim3(threads), smem, s, 0, (const uint16_t*)x, (const uint16_t*)w, (uint16_t*)y, \
             (uint16_t*)residual, H, ldx, ldy, eps, unit_offset, qo);                                                          \
  }
  if (dtype == 1) { if (mode == 1) FB_NQ(true, 1) else if (mode == 2) FB_NQ(true, 2) else if (mode == 3) FB_NQ(true, 3) else FB_NQ(true, 4) }
  else { if (mode == 1) FB_NQ(false, 1) else if (mode == 2) FB_NQ(false, 2) else if (mode == 3) FB_NQ(false, 3) else FB_NQ(false, 4) }
#undef FB_NQ
  return (int)cudaGetLastError();
}

extern "C" int fb_rmsnorm(const void* x, const void* w, void* y, void* residual, int M, int H, int ldx, int ldy, float eps,
                          float unit_offset, int dtype, void* stream) {
  if (M <= 0) return 0;
  if (H % 8 != 0 || H > 32768) return -1;
  int threads = H / 8;
  threads = threads > 1024 ? 1024 : ((threads + 31) / 32) * 32;
  const size_t smem = (size_t)H * sizeof(float);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) {
    static DeviceOnce cfg;
    if (cfg.need()) { cudaFuncSetAttribute(rmsnorm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4); }
    launch_k(rmsnorm_kernel<true>, dim3(M), dim3(threads), smem, s, 0, (const uint16_t*)x, (const uint16_t*)w, (uint16_t*)y, (uint16_t*)residual, H, ldx, ldy, eps, unit_offset, NormQuantOut{});
  } else {
    static DeviceOnce cfg;
    if (cfg.need()) { cudaFuncSetAttribute(rmsnorm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4); }
    launch_k(rmsnorm_kernel<false>, dim3(M), dim3(threads), smem, s, 0, (const uint16_t*)x, (const uint16_t*)w, (uint16_t*)y, (uint16_t*)residual, H, ldx, ldy, eps, unit_offset, NormQuantOut{});
  }
  return (int)cudaGetLastError();
}

extern "C" int fb_qkv_post(const void* qkv, int ld_qkv, void* q_out, int ld_q, void* k_pool, void* v_pool, const int* positions,
                           const int* slots, const void* q_norm_w, const void* k_norm_w, const float* cos_tab,
                           const float* sin_tab, int M, int Hq, int Hkv, int D, int rot, int rope_mode, float eps,
                           float norm_unit_offset, int dtype, void* stream) {
  if (M <= 0) return 0;
  if (D % 2 != 0 || D > 512 || rot > D || (rot & 3) != 0) return -1;
  QkvPostParams p;
  p.qkv = (const uint16_t*)qkv; p.ld_qkv = ld_qkv; p.q_out = (uint16_t*)q_out; p.ld_q = ld_q;
  p.k_pool = (uint16_t*)k_pool; p.v_pool = (uint16_t*)v_pool; p.positions = positions; p.slots = slots;
  p.q_norm_w = (const uint16_t*)q_norm_w; p.k_norm_w = (const uint16_t*)k_norm_w; p.cos_tab = cos_tab; p.sin_tab = sin_tab;
  p.M = M; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.rot = rot; p.rope_mode = rope_mode; p.eps = eps; p.norm_unit_offset = norm_unit_offset;
  p.kv8 = 0; p.q8a = nullptr; p.q8b = nullptr;
  const long long warps = (long long)M * (Hq + 2 * Hkv);
  const int wpb = 8;
  const int blocks = (int)((warps + wpb - 1) / wpb);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) launch_k(qkv_post_kernel<true>, dim3(blocks), dim3(wpb * 32), 0, s, 0, p);
  else launch_k(qkv_post_kernel<false>, dim3(blocks), dim3(wpb * 32), 0, s, 0, p);
  return (int)cudaGetLastError();
}

// Same for e4m3 page pools: K / V rows are appended as e4m3 bytes; q8a / q8b (null: not wanted) receive the two e4m3 terms of
// the queries for the fp8 tensor-core decode attention.
extern "C" int fb_qkv_post_kv8(const void* qkv, int ld_qkv, void* q_out, int ld_q, void* k_pool, void* v_pool, const int* positions,
                               const int* slots, const void* q_norm_w, const void* k_norm_w, const float* cos_tab,
                               const float* sin_tab, int M, int Hq, int Hkv, int D, int rot, int rope_mode, float eps,
                               float norm_unit_offset, int dtype, void* q8a, void* q8b, void* stream) {
  if (M <= 0) return 0;
  if (D % 2 != 0 || D > 512 || rot > D || (rot & 3) != 0 || ((q8a == nullptr) != (q8b == nullptr))) return -1;
  QkvPostParams p;
  p.qkv = (const uint16_t*)qkv; p.ld_qkv = ld_qkv; p.q_out = (uint16_t*)q_out; p.ld_q = ld_q;
  p.k_pool = (uint16_t*)k_pool; p.v_pool = (uint16_t*)v_pool; p.positions = positions; p.slots = slots;
  p.q_norm_w = (const uint16_t*)q_norm_w; p.k_norm_w = (const uint16_t*)k_norm_w; p.cos_tab = cos_tab; p.sin_tab = sin_tab;
  p.M = M; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.rot = rot; p.rope_mode = rope_mode; p.eps = eps; p.norm_unit_offset = norm_unit_offset;
  p.kv8 = 1; p.q8a = (uint8_t*)q8a; p.q8b = (uint8_t*)q8b;
  const long long warps = (long long)M * (Hq + 2 * Hkv);
  const int wpb = 8;
  const int blocks = (int)((warps + wpb - 1) / wpb);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) launch_k(qkv_post_kernel<true>, dim3(blocks), dim3(wpb * 32), 0, s, 0, p);
  else launch_k(qkv_post_kernel<false>, dim3(blocks), dim3(wpb * 32), 0, s, 0, p);
  return (int)cudaGetLastError();
}

extern "C" int fb_silu_mul(const void* x, void* y, int M, int I, int ldx, int ldy, int dtype, void* stream) {
  if (M <= 0) return 0;
  if (I % 8 != 0) return -1;
  const size_t total = (size_t)M * (I / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) launch_k(silu_mul_kernel<true>, dim3(blocks), dim3(256), 0, s, 0, (const uint16_t*)x, (uint16_t*)y, M, I, ldx, ldy);
  else launch_k(silu_mul_kernel<false>, dim3(blocks), dim3(256), 0, s, 0, (const uint16_t*)x, (uint16_t*)y, M, I, ldx, ldy);
  return (int)cudaGetLastError();
}

// act: 0 SiLU, 1 GELU (tanh), 2 GELU (erf), 3 ReLU; interleaved != 0: gate / up alternate in blocks of 64 columns (I % 64 == 0)
extern "C" int fb_glu_act(const void* x, void* y, int M, int I, int ldx, int ldy, int act, int interleaved, int dtype, void* stream) {
  if (M <= 0) return 0;
  if (I % 8 != 0 || act < 0 || act > 3 || (interleaved && I % 64 != 0) || (dtype != 0 && dtype != 1)) return -1;
  const size_t total = (size_t)M * (I / 8);
  int blocks = (int)((total + 255) / 256);
  if (blocks > 148 * 16) blocks = 148 * 16;
  auto s = reinterpret_cast<cudaStream_t>(stream);
#define FB_GLU(A)                                                                                                                          \
  if (dtype == 1) launch_k(glu_act_kernel<true, A>, dim3(blocks), dim3(256), 0, s, 0, (const uint16_t*)x, (uint16_t*)y, M, I, ldx, ldy, interleaved); \
  else launch_k(glu_act_kernel<false, A>, dim3(blocks), dim3(256), 0, s, 0, (const uint16_t*)x, (uint16_t*)y, M, I, ldx, ldy, interleaved);
  switch (act) {
    case 0: FB_GLU(0) break;
    case 1: FB_GLU(1) break;
    case 2: FB_GLU(2) break;
    default: FB_GLU(3) break;
  }
#undef FB_GLU
  return (int)cudaGetLastError();
}

extern "C" int fb_kv_append_fp8(const void* k, const void* v, void* k_pool, void* v_pool, const int* slots, int T, int row_elems, int dtype,
                                void* stream) {
  if (T <= 0) return 0;
  if (row_elems % 8 != 0 || (dtype != 0 && dtype != 1)) return -1;
  const long long total = (long long)T * (row_elems / 8) * 2;
  const int blocks = (int)((total + 255) / 256);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) launch_k(kv_append_fp8_kernel<true>, dim3(blocks), dim3(256), 0, s, 0, (const uint16_t*)k, (const uint16_t*)v, (uint8_t*)k_pool, (uint8_t*)v_pool, slots, T, row_elems);
  else launch_k(kv_append_fp8_kernel<false>, dim3(blocks), dim3(256), 0, s, 0, (const uint16_t*)k, (const uint16_t*)v, (uint8_t*)k_pool, (uint8_t*)v_pool, slots, T, row_elems);
  return (int)cudaGetLastError();
}

// rows = queries x heads (query-major); row r sees keys [0, first_pos + r / heads]; P is zero elsewhere (all `cols` columns are written)
extern "C" int fb_softmax_causal_rows(const float* S, int lds, void* P, int ldp, int rows, int cols, int heads, int first_pos, float scale,
                                      int dtype, void* stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (heads <= 0 || (dtype != 0 && dtype != 1)) return -1;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) launch_k(softmax_causal_rows_kernel<true>, dim3(rows), dim3(256), 0, s, 0, S, lds, (uint16_t*)P, ldp, cols, heads, first_pos, scale);
  else launch_k(softmax_causal_rows_kernel<false>, dim3(rows), dim3(256), 0, s, 0, S, lds, (uint16_t*)P, ldp, cols, heads, first_pos, scale);
  return (int)cudaGetLastError();
}

extern "C" int fb_embedding(const int* ids, const void* table, void* out, int M, int H, int vocab, void* stream) {
  if (M <= 0) return 0;
  if (H % 8 != 0) return -1;
  launch_k(embedding_kernel, dim3(M), dim3(256), 0, reinterpret_cast<cudaStream_t>(stream), 0, ids, (const uint16_t*)table, (uint16_t*)out, H, vocab);
  return (int)cudaGetLastError();
}

// kind: 0 = f32, 1 = bf16, 2 = f16
extern "C" int fb_argmax(const void* logits, int* ids, float* vals, int M, int V, int ld, int id_offset, int kind, void* stream) {
  if (M <= 0) return 0;
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (kind == 0) launch_k(argmax_kernel<0>, dim3(M), dim3(1024), 0, s, 0, logits, ids, vals, V, ld, id_offset);
  else if (kind == 1) launch_k(argmax_kernel<1>, dim3(M), dim3(1024), 0, s, 0, logits, ids, vals, V, ld, id_offset);
  else launch_k(argmax_kernel<2>, dim3(M), dim3(1024), 0, s, 0, logits, ids, vals, V, ld, id_offset);
  return (int)cudaGetLastError();
}

extern "C" int fb_route_topk(const float* logits, const float* bias, int* out_idx, float* out_w, int M, int E, int topk,
                             int score_mode, int renorm, int n_group, int topk_group, float route_scale, void* stream) {
  if (M <= 0) return 0;
  if (E > 512 || topk > 32 || n_group > 32 || (n_group > 1 && E % n_group != 0)) return -1;
  RouteParams p{logits, bias, out_idx, out_w, M, E, topk, score_mode, renorm, n_group, topk_group, route_scale};
  const int wpb = 4;
  launch_k(route_topk_kernel, dim3((M + wpb - 1) / wpb), dim3(wpb * 32), 0, reinterpret_cast<cudaStream_t>(stream), 0, p);
  return (int)cudaGetLastError();
}

// See MlaPostParams.  rope_mode: 1 neox, 2 interleaved.  spare_slot: where rows with slots[t] < 0 are written (a slot no request reads).
extern "C" int fb_mla_post(const void* ckv, int ld_ckv, const void* q, int ld_q, void* q_full, int ld_qf, void* pool, const int* positions,
                           const int* slots, const void* norm_w, const float* cos_tab, const float* sin_tab, int T, int H, int nope,
                           int rope, int lora, int rope_mode, long long spare_slot, float eps, int dtype, void* stream_) {
  if (T <= 0) return 0;
  if ((dtype != 0 && dtype != 1) || (rope & 1) || (rope_mode != 1 && rope_mode != 2)) return -1;
  MlaPostParams p;
  p.ckv = (const uint16_t*)ckv; p.ld_ckv = ld_ckv; p.q = (const uint16_t*)q; p.ld_q = ld_q; p.q_full = (uint16_t*)q_full; p.ld_qf = ld_qf;
  p.pool = (uint16_t*)pool; p.positions = positions; p.slots = slots; p.norm_w = (const uint16_t*)norm_w; p.cos_tab = cos_tab;
  p.sin_tab = sin_tab; p.H = H; p.nope = nope; p.rope = rope; p.lora = lora; p.rope_mode = rope_mode; p.spare_slot = (int)spare_slot;
  p.eps = eps;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == 1) launch_k(mla_post_kernel<true>, dim3(T), dim3(256), 0, s, 0, p);
  else launch_k(mla_post_kernel<false>, dim3(T), dim3(256), 0, s, 0, p);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// Whole-matrix de-quantisation of a weight into the activations' 16-bit type (prefill-sized batches run the dense
// tensor-core GEMM on the result; the reference de-quantises to fp16 and calls cuBLAS there,
// src/devices/cuda/linear/fastllm-linear-int4group.cu:1919-2054).  One thread = eight consecutive k of one row.
//   mode 1 int8:  w = scale[n] * (q - zero[n])            (bytes hold q, or q - 128 when `flag`)
//   mode 2 int4g: w = min[n, g] + scale[n, g] * q          (two per byte, first value in the high nibble)
//   mode 3 fp8:   w = e4m3(q) * scale[n / 128, k / 128]
//   mode 4 fp4:   w = e2m1(q) * scale_bf16[n, k / group] * global   (two per byte, first value in the low nibble)
// ------------------------------------------------------------------------------------------------
namespace fb {
struct DequantParams {
  const uint8_t* q; const float* scale; const float* zero; uint16_t* out;
  int N, K, mode, group, groups, flag, ld_out;
};

template <bool BF16>
__global__ void dequant_weight_kernel(const DequantParams p) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int k8 = p.K >> 3;
  if (t >= (long long)p.N * k8) return;
  const int n = (int)(t / k8), k0 = (int)(t - (long long)n * k8) << 3;
  float v[8];
  if (p.mode == 1) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p.q + (size_t)n * p.K + k0);
    const float sc = p.scale[n], z = p.zero[n] - (p.flag ? 128.f : 0.f);
    const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t b = (w[j >> 2] >> (8 * (j & 3))) & 0xFFu;
      v[j] = sc * ((p.flag ? (float)(int8_t)b : (float)b) - z);
    }
  } else if (p.mode == 2) {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(p.q + (size_t)n * (p.K >> 1) + (k0 >> 1));
    const int g = k0 / p.group;
    const float sc = p.scale[(size_t)n * p.groups + g], mn = p.zero[(size_t)n * p.groups + g];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t b = (raw >> (8 * j)) & 0xFFu;
      v[2 * j] = mn + sc * (float)(b >> 4);
      v[2 * j + 1] = mn + sc * (float)(b & 0xFu);
    }
  } else if (p.mode == 3) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p.q + (size_t)n * p.K + k0);
    const float sc = p.scale[(size_t)(n >> 7) * p.groups + (k0 >> 7)];
    const uint32_t w[2] = {raw.x, raw.y};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = e4m3x2_to_f2((unsigned short)((w[j >> 1] >> (16 * (j & 1))) & 0xFFFFu));
      v[2 * j] = f.x * sc; v[2 * j + 1] = f.y * sc;
    }
  } else {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(p.q + (size_t)n * (p.K >> 1) + (k0 >> 1));
    const uint16_t sb = reinterpret_cast<const uint16_t*>(p.scale)[(size_t)n * p.groups + k0 / p.group];
    const float sc = __uint_as_float((uint32_t)sb << 16) * (p.zero != nullptr ? p.zero[0] : 1.f);
    uint32_t h[4];
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\tmov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\tcvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\tcvt.rn.f16x2.e2m1x2 %3, b3;\n\t}\n"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(raw));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h[j]));
      v[2 * j] = f.x * sc; v[2 * j + 1] = f.y * sc;
    }
  }
  uint4 o;
  o.x = pack_16<BF16>(v[0], v[1]); o.y = pack_16<BF16>(v[2], v[3]); o.z = pack_16<BF16>(v[4], v[5]); o.w = pack_16<BF16>(v[6], v[7]);
  *reinterpret_cast<uint4*>(p.out + (size_t)n * p.ld_out + k0) = o;
}
}  // namespace fb

// scale / zero: the weight's own tables (int8: [N] each; int4g: [N, K / group] scale and minimum; fp8: [ceil(N / 128), ceil(K / 128)];
// fp4: bf16 [N, K / group] and an optional one-element fp32 factor).  flag: int8 bytes hold q - 128.
extern "C" int fb_dequant_weight(const void* q, const void* scale, const void* zero, void* out, int N, int K, int ld_out, int mode,
                                 int group, int flag, int dtype, void* stream) {
  using namespace fb;
  if (N <= 0 || K <= 0) return 0;
  if (K % 8 != 0 || ld_out % 8 != 0 || mode < 1 || mode > 4 || (dtype != 0 && dtype != 1)) return -1;
  if ((mode == 2 || mode == 4) && (group <= 0 || group % 8 != 0 || K % group != 0)) return -1;
  DequantParams p;
  p.q = (const uint8_t*)q; p.scale = (const float*)scale; p.zero = (const float*)zero; p.out = (uint16_t*)out;
  p.N = N; p.K = K; p.mode = mode; p.group = group; p.flag = flag; p.ld_out = ld_out;
  p.groups = mode == 3 ? (K + 127) / 128 : ((mode == 2 || mode == 4) ? K / group : 0);
  const long long n = (long long)N * (K / 8);
  const int blocks = (int)((n + 255) / 256);
  auto s = reinterpret_cast<cudaStream_t>(stream);
  if (dtype == 1) dequant_weight_kernel<true><<<blocks, 256, 0, s>>>(p);
  else dequant_weight_kernel<false><<<blocks, 256, 0, s>>>(p);
  return (int)cudaGetLastError();
}
