// ISA-specific CPU kernels.  This file is compiled twice (AVX2+FMA+F16C, and AVX-512 F/BW/VL/DQ) with
// FB_ISA_SUFFIX set to _avx2 / _avx512; the dispatcher picks one set at run time.  Everything here is single-threaded
// over a range of independent work items.
//
// Reference kernels covered: fp32/bf16/fp16/int8/int4-group Linear (src/devices/cpu/linear.cpp:412-1278 and the
// AVX2/AVX-512 micro-kernels under src/devices/cpu/), RMSNorm / LayerNorm / Softmax / Swiglu / RoPE / Attention of
// src/devices/cpu/cpudevice.cpp.
#include <immintrin.h>

#include <cmath>
#include <cstdint>
#include <cstring>

#include "cpu_kernels.h"

#define FB_CAT2(a, b) a##b
#define FB_CAT(a, b) FB_CAT2(a, b)
#define FB_NAME(base) FB_CAT(base, FB_ISA_SUFFIX)

namespace {

#if defined(__AVX512F__)
struct V {
  static constexpr int W = 16;
  using T = __m512;
  static T zero() { return _mm512_setzero_ps(); }
  static T set1(float v) { return _mm512_set1_ps(v); }
  static T load(const float* p) { return _mm512_loadu_ps(p); }
  static void store(float* p, T v) { _mm512_storeu_ps(p, v); }
  static T fma(T a, T b, T c) { return _mm512_fmadd_ps(a, b, c); }
  static T mul(T a, T b) { return _mm512_mul_ps(a, b); }
  static float sum(T a) { return _mm512_reduce_add_ps(a); }
  static T from_bf16(const uint16_t* p) {
    return _mm512_castsi512_ps(_mm512_slli_epi32(_mm512_cvtepu16_epi32(_mm256_loadu_si256((const __m256i*)p)), 16));
  }
  static T from_f16(const uint16_t* p) { return _mm512_cvtph_ps(_mm256_loadu_si256((const __m256i*)p)); }
  static T from_u8(const uint8_t* p) { return _mm512_cvtepi32_ps(_mm512_cvtepu8_epi32(_mm_loadu_si128((const __m128i*)p))); }
  // W four-bit values from W/2 bytes, first value of each byte in the high nibble
  static T from_u4(const uint8_t* p) {
    const __m128i b = _mm_cvtepu8_epi16(_mm_loadl_epi64((const __m128i*)p));
    const __m128i v = _mm_and_si128(_mm_or_si128(_mm_srli_epi16(b, 4), _mm_slli_epi16(b, 8)), _mm_set1_epi16(0x0F0F));
    return _mm512_cvtepi32_ps(_mm512_cvtepu8_epi32(v));
  }
};
#else
struct V {
  static constexpr int W = 8;
  using T = __m256;
  static T zero() { return _mm256_setzero_ps(); }
  static T set1(float v) { return _mm256_set1_ps(v); }
  static T load(const float* p) { return _mm256_loadu_ps(p); }
  static void store(float* p, T v) { _mm256_storeu_ps(p, v); }
  static T fma(T a, T b, T c) { return _mm256_fmadd_ps(a, b, c); }
  static T mul(T a, T b) { return _mm256_mul_ps(a, b); }
  static float sum(T a) {
    __m128 s = _mm_add_ps(_mm256_castps256_ps128(a), _mm256_extractf128_ps(a, 1));
    s = _mm_add_ps(s, _mm_movehl_ps(s, s));
    s = _mm_add_ss(s, _mm_shuffle_ps(s, s, 1));
    return _mm_cvtss_f32(s);
  }
  static T from_bf16(const uint16_t* p) {
    return _mm256_castsi256_ps(_mm256_slli_epi32(_mm256_cvtepu16_epi32(_mm_loadu_si128((const __m128i*)p)), 16));
  }
  static T from_f16(const uint16_t* p) { return _mm256_cvtph_ps(_mm_loadu_si128((const __m128i*)p)); }
  static T from_u8(const uint8_t* p) { return _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(_mm_loadl_epi64((const __m128i*)p))); }
  static T from_u4(const uint8_t* p) {
    int32_t raw;
    std::memcpy(&raw, p, 4);
    const __m128i b = _mm_cvtepu8_epi16(_mm_cvtsi32_si128(raw));
    const __m128i v = _mm_and_si128(_mm_or_si128(_mm_srli_epi16(b, 4), _mm_slli_epi16(b, 8)), _mm_set1_epi16(0x0F0F));
    return _mm256_cvtepi32_ps(_mm256_cvtepu8_epi32(v));
  }
};
#endif

inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
inline float f16_to_f32(uint16_t h) { return _cvtsh_ss(h); }

// storage accessors: vector of W consecutive k values of one weight row, and the scalar for k tails
template <int WT>
inline V::T wload(const void* row, int k) {
  if (WT == 0) return V::load((const float*)row + k);
  if (WT == 1) return V::from_bf16((const uint16_t*)row + k);
  if (WT == 2) return V::from_f16((const uint16_t*)row + k);
  if (WT == 3) return V::from_u8((const uint8_t*)row + k);
  return V::from_u4((const uint8_t*)row + (k >> 1));
}
template <int WT>
inline float wscalar(const void* row, int k) {
  if (WT == 0) return ((const float*)row)[k];
  if (WT == 1) return bf16_to_f32(((const uint16_t*)row)[k]);
  if (WT == 2) return f16_to_f32(((const uint16_t*)row)[k]);
  if (WT == 3) return (float)((const uint8_t*)row)[k];
  const uint8_t b = ((const uint8_t*)row)[k >> 1];
  return (float)((k & 1) ? (b & 0xF) : (b >> 4));
}
template <int WT>
inline size_t row_bytes(int K) {
  return WT == 0 ? (size_t)K * 4 : (WT == 1 || WT == 2) ? (size_t)K * 2 : WT == 3 ? (size_t)K : (size_t)K / 2;
}

// raw dot products of R weight rows with MB activation rows over k in [k0, k1) (k0, k1 multiples of the group for int4g)
template <int WT, int R, int MB>
inline void dot_block(const uint8_t* w, size_t wstride, const float* x, int ldx, int k0, int k1, V::T acc[R][MB]) {
  int k = k0;
  for (; k + V::W <= k1; k += V::W) {
    V::T wv[R];
#pragma GCC unroll 4
    for (int r = 0; r < R; ++r) wv[r] = wload<WT>(w + r * wstride, k);
#pragma GCC unroll 4
    for (int j = 0; j < MB; ++j) {
      const V::T xv = V::load(x + (size_t)j * ldx + k);
#pragma GCC unroll 4
      for (int r = 0; r < R; ++r) acc[r][j] = V::fma(wv[r], xv, acc[r][j]);
    }
  }
}

template <int WT, int R, int MB>
void linear_block(const FbLinearArgs* a, int n, int m) {
  const size_t ws = row_bytes<WT>(a->K);
  const uint8_t* w = (const uint8_t*)a->w + (size_t)n * ws;
  const float* x = a->x + (size_t)m * a->ldx;
  const int K = a->K;
  float res[R][MB];
  if (WT != 4) {
    V::T acc[R][MB];
    for (int r = 0; r < R; ++r)
      for (int j = 0; j < MB; ++j) acc[r][j] = V::zero();
    dot_block<WT, R, MB>(w, ws, x, a->ldx, 0, K, acc);
    const int kt = K - K % V::W;
    for (int r = 0; r < R; ++r)
      for (int j = 0; j < MB; ++j) {
        float s = V::sum(acc[r][j]);
        for (int k = kt; k < K; ++k) s += wscalar<WT>(w + r * ws, k) * x[(size_t)j * a->ldx + k];
        if (WT == 3) s = a->scale[n + r] * (s - a->zero[n + r] * a->xsum[m + j]);
        res[r][j] = s;
      }
  } else {
    const int G = a->group, ng = K / G;
    V::T tot[R][MB];
    for (int r = 0; r < R; ++r)
      for (int j = 0; j < MB; ++j) tot[r][j] = V::zero();
    for (int g = 0; g < ng; ++g) {
      V::T acc[R][MB];
      for (int r = 0; r < R; ++r)
        for (int j = 0; j < MB; ++j) acc[r][j] = V::zero();
      dot_block<WT, R, MB>(w, ws, x, a->ldx, g * G, (g + 1) * G, acc);
      for (int r = 0; r < R; ++r) {
        const V::T sv = V::set1(a->scale[(size_t)(n + r) * ng + g]);
        for (int j = 0; j < MB; ++j) tot[r][j] = V::fma(acc[r][j], sv, tot[r][j]);
      }
    }
    for (int r = 0; r < R; ++r)
      for (int j = 0; j < MB; ++j) {
        float s = V::sum(tot[r][j]);
        const float* mn = a->zero + (size_t)(n + r) * ng;
        const float* xs = a->xsum + (size_t)(m + j) * ng;
        float c = 0.f;
        for (int g = 0; g < ng; ++g) c += mn[g] * xs[g];
        res[r][j] = s + c;
      }
  }
  for (int r = 0; r < R; ++r) {
    const float b = a->bias ? a->bias[n + r] : 0.f;
    for (int j = 0; j < MB; ++j) a->y[(size_t)(m + j) * a->ldy + n + r] = res[r][j] + b;
  }
}

template <int WT>
void linear_rows_t(const FbLinearArgs* a, int n0, int n1) {
  constexpr int R = V::W == 16 ? 2 : 1;      // AVX2 has 16 vector registers: one weight row per block
  int n = n0;
  for (; n + R <= n1; n += R) {
    int m = 0;
    for (; m + 4 <= a->M; m += 4) linear_block<WT, R, 4>(a, n, m);
    for (; m < a->M; ++m) linear_block<WT, R, 1>(a, n, m);
  }
  for (; n < n1; ++n) {
    int m = 0;
    for (; m + 4 <= a->M; m += 4) linear_block<WT, 1, 4>(a, n, m);
    for (; m < a->M; ++m) linear_block<WT, 1, 1>(a, n, m);
  }
}

}  // namespace

extern "C" void FB_NAME(fbk_linear_rows)(const FbLinearArgs* a, int n0, int n1) {
  switch (a->wtype) {
    case 0: linear_rows_t<0>(a, n0, n1); break;
    case 1: linear_rows_t<1>(a, n0, n1); break;
    case 2: linear_rows_t<2>(a, n0, n1); break;
    case 3: linear_rows_t<3>(a, n0, n1); break;
    default: linear_rows_t<4>(a, n0, n1); break;
  }
}

// out[m][g] = sum of x[m][g*group .. (g+1)*group)
extern "C" void FB_NAME(fbk_group_sums)(const float* x, int ldx, int M, int K, int group, float* out) {
  const int ng = K / group;
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < ng; ++g) {
      const float* p = x + (size_t)m * ldx + (size_t)g * group;
      float s = 0.f;
      for (int k = 0; k < group; ++k) s += p[k];
      out[(size_t)m * ng + g] = s;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// row kernels (auto-vectorised by the compiler for the ISA of this translation unit)
// ---------------------------------------------------------------------------------------------------------------
extern "C" void FB_NAME(fbk_rmsnorm_rows)(const float* x, int ldx, const float* w, float* y, int ldy, int H, float eps,
                                          float unit_offset, int r0, int r1) {
  for (int r = r0; r < r1; ++r) {
    const float* p = x + (size_t)r * ldx;
    float ss = 0.f;
    for (int i = 0; i < H; ++i) ss += p[i] * p[i];
    const float inv = 1.0f / std::sqrt(ss / (float)H + eps);
    float* o = y + (size_t)r * ldy;
    for (int i = 0; i < H; ++i) o[i] = p[i] * inv * (w[i] + unit_offset);
  }
}

extern "C" void FB_NAME(fbk_layernorm_rows)(const float* x, int ldx, const float* w, const float* b, float* y, int ldy, int H,
                                            float eps, int r0, int r1) {
  for (int r = r0; r < r1; ++r) {
    const float* p = x + (size_t)r * ldx;
    float mean = 0.f;
    for (int i = 0; i < H; ++i) mean += p[i];
    mean /= (float)H;
    float var = 0.f;
    for (int i = 0; i < H; ++i) var += (p[i] - mean) * (p[i] - mean);
    const float inv = 1.0f / std::sqrt(var / (float)H + eps);
    float* o = y + (size_t)r * ldy;
    for (int i = 0; i < H; ++i) o[i] = (p[i] - mean) * inv * w[i] + (b ? b[i] : 0.f);
  }
}

// gu = [gate (inter) | up (inter)] per row;  out = silu(gate) * up
extern "C" void FB_NAME(fbk_swiglu_rows)(const float* gu, int ld, float* out, int ldo, int inter, int r0, int r1) {
  for (int r = r0; r < r1; ++r) {
    const float* g = gu + (size_t)r * ld;
    const float* u = g + inter;
    float* o = out + (size_t)r * ldo;
    for (int i = 0; i < inter; ++i) o[i] = g[i] / (1.0f + std::exp(-g[i])) * u[i];
  }
}

// kind: 0 silu, 1 gelu (erf), 2 gelu (tanh approximation), 3 relu, 4 sigmoid, 5 tanh, 6 exp
extern "C" void FB_NAME(fbk_act_rows)(float* x, int n, int kind) {
  switch (kind) {
    case 0: for (int i = 0; i < n; ++i) x[i] = x[i] / (1.0f + std::exp(-x[i])); break;
    case 1: for (int i = 0; i < n; ++i) x[i] = 0.5f * x[i] * (1.0f + std::erf(x[i] * 0.70710678f)); break;
    case 2: for (int i = 0; i < n; ++i) x[i] = 0.5f * x[i] * (1.0f + std::tanh(0.7978845608f * (x[i] + 0.044715f * x[i] * x[i] * x[i]))); break;
    case 3: for (int i = 0; i < n; ++i) x[i] = x[i] > 0.f ? x[i] : 0.f; break;
    case 4: for (int i = 0; i < n; ++i) x[i] = 1.0f / (1.0f + std::exp(-x[i])); break;
    case 5: for (int i = 0; i < n; ++i) x[i] = std::tanh(x[i]); break;
    default: for (int i = 0; i < n; ++i) x[i] = std::exp(x[i]); break;
  }
}

extern "C" void FB_NAME(fbk_softmax_rows)(float* x, int ld, int cols, int r0, int r1) {
  for (int r = r0; r < r1; ++r) {
    float* p = x + (size_t)r * ld;
    float mx = -INFINITY;
    for (int i = 0; i < cols; ++i) mx = p[i] > mx ? p[i] : mx;
    if (mx == -INFINITY) { for (int i = 0; i < cols; ++i) p[i] = 0.f; continue; }
    float s = 0.f;
    for (int i = 0; i < cols; ++i) { p[i] = std::exp(p[i] - mx); s += p[i]; }
    const float inv = 1.0f / s;
    for (int i = 0; i < cols; ++i) p[i] *= inv;
  }
}

// x: [rows, heads * D]; tables [max_pos, rot / 2]; mode 1 = half-split (neox), 2 = interleaved pairs
extern "C" void FB_NAME(fbk_rope_rows)(float* x, int ld, const int* pos, const float* cos_t, const float* sin_t, int heads, int D,
                                       int rot, int mode, int r0, int r1) {
  const int half = rot / 2;
  for (int r = r0; r < r1; ++r) {
    const float* c = cos_t + (size_t)pos[r] * half;
    const float* s = sin_t + (size_t)pos[r] * half;
    for (int h = 0; h < heads; ++h) {
      float* p = x + (size_t)r * ld + (size_t)h * D;
      if (mode == 1) {
        for (int i = 0; i < half; ++i) {
          const float a = p[i], b = p[i + half];
          p[i] = a * c[i] - b * s[i];
          p[i + half] = b * c[i] + a * s[i];
        }
      } else {
        for (int i = 0; i < half; ++i) {
          const float a = p[2 * i], b = p[2 * i + 1];
          p[2 * i] = a * c[i] - b * s[i];
          p[2 * i + 1] = b * c[i] + a * s[i];
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------
// causal attention of packed new tokens over the paged fp32 cache; item = request * Hq + query head.
// Online softmax over blocks of 32 cached tokens.
// ---------------------------------------------------------------------------------------------------------------
extern "C" void FB_NAME(fbk_attention_items)(const FbAttnArgs* a, int i0, int i1) {
  constexpr int TB = 32;
  const int D = a->D, G = a->Hq / a->Hkv;
  float acc_buf[512];
  for (int item = i0; item < i1; ++item) {
    const int b = item / a->Hq, h = item - b * a->Hq, kvh = h / G;
    const int q0 = a->cu_q[b], q1 = a->cu_q[b + 1];
    const int L = a->kv_lens[b];
    const int* pages = a->page_table + (size_t)b * a->max_pages;
    for (int qi = q0; qi < q1; ++qi) {
      const int qpos = L - (q1 - q0) + (qi - q0);
      const float* q = a->q + (size_t)qi * a->ldq + (size_t)h * D;
      float* acc = acc_buf;
      for (int d = 0; d < D; ++d) acc[d] = 0.f;
      float m = -INFINITY, l = 0.f;
      if (a->sinks) { m = a->sinks[h]; l = 1.f; }
      int t_begin = 0;
      if (a->window > 0 && qpos + 1 > a->window) t_begin = qpos + 1 - a->window;
      for (int t0 = t_begin; t0 <= qpos; t0 += TB) {
        const int nt = (qpos + 1 - t0) < TB ? (qpos + 1 - t0) : TB;
        float s[TB];
        const float* kp[TB];
        const float* vp[TB];
        float bm = -INFINITY;
        for (int i = 0; i < nt; ++i) {
          const int t = t0 + i;
          const size_t slot = (size_t)pages[t / a->page_len] * a->page_len + (size_t)(t % a->page_len);
          kp[i] = a->k_pool + (slot * a->Hkv + kvh) * D;
          vp[i] = a->v_pool + (slot * a->Hkv + kvh) * D;
          V::T av = V::zero();
          int d = 0;
          for (; d + V::W <= D; d += V::W) av = V::fma(V::load(q + d), V::load(kp[i] + d), av);
          float dot = V::sum(av);
          for (; d < D; ++d) dot += q[d] * kp[i][d];
          s[i] = dot * a->scale;
          bm = s[i] > bm ? s[i] : bm;
        }
        const float m_new = bm > m ? bm : m;
        const float corr = m == -INFINITY ? 0.f : std::exp(m - m_new);
        l *= corr;
        for (int d = 0; d < D; ++d) acc[d] *= corr;
        for (int i = 0; i < nt; ++i) {
          const float p = std::exp(s[i] - m_new);
          l += p;
          const V::T pv = V::set1(p);
          int d = 0;
          for (; d + V::W <= D; d += V::W) V::store(acc + d, V::fma(pv, V::load(vp[i] + d), V::load(acc + d)));
          for (; d < D; ++d) acc[d] += p * vp[i][d];
        }
        m = m_new;
      }
      float* o = a->out + (size_t)qi * a->ldo + (size_t)h * D;
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      for (int d = 0; d < D; ++d) o[d] = acc[d] * inv;
    }
  }
}
