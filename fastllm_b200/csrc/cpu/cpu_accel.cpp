// Reduced-precision-activation CPU kernels: AVX-512 VNNI (int8 / int4-group weights x int8 activations), AVX-512 BF16
// (bf16 weights x bf16 activations) and AMX tiles (both, for batches of 16 rows and more).  Opt-in (fbcpu_set_accel): the
// default CPU path keeps fp32 activations and is exact with respect to the stored weights; these paths round the
// activations -- to int8 per (row, 128-wide k block), or to bf16 -- the way the GPU's 8-bit-activation kernels do.
//
//   int8  (w = s_n (q - z_n)):        y[m][n] = s_n * sum_g a[m,g] * (dot_g - z_n * xs[m,g])
//   int4g (w = min_ng + s_ng q):      y[m][n] = sum_g a[m,g] * (s_ng * dot_g + min_ng * xs[m,g])
// with dot_g the exact integer dot product of one 128-wide block, a the activation scale and xs the sum of the block's
// quantised activations.  A block's int32 lanes are scaled and accumulated in fp32 vectors; one horizontal sum per output.
//
// Reference counterparts: src/devices/cpu/avx512vnni.cpp, avx512bf16.cpp, amx.cpp.
#include <immintrin.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cmath>
#include <cstdint>
#include <cstring>

#include "cpu_kernels.h"

namespace {

constexpr int BLK = 128;          // activation quantisation block (and the int4 group the fast path takes)

inline float hsum(__m512 v) { return _mm512_reduce_add_ps(v); }

// AMX needs the kernel's permission to use the tile state (Linux: arch_prctl ARCH_REQ_XCOMP_PERM, XFEATURE_XTILEDATA = 18)
bool amx_permitted() {
  static int ok = -1;
  if (ok < 0) {
    ok = 0;
    if (__builtin_cpu_supports("amx-tile") && __builtin_cpu_supports("amx-int8") && __builtin_cpu_supports("amx-bf16"))
      ok = syscall(SYS_arch_prctl, 0x1023 /* ARCH_REQ_XCOMP_PERM */, 18) == 0 ? 1 : 0;
  }
  return ok == 1;
}

struct alignas(64) TileCfg {
  uint8_t palette = 1, start_row = 0;
  uint8_t reserved[14] = {};
  uint16_t colsb[16] = {};
  uint8_t rows[16] = {};
};

// tiles: 0 = C (16 x 16 x 4 bytes), 1 = A (16 weight rows x 64 bytes of k), 2 = B (16 k-quads x 16 activation rows x 4 bytes)
void amx_config() {
  static thread_local bool done = false;
  if (done) return;
  TileCfg c;
  for (int t = 0; t < 3; ++t) { c.colsb[t] = 64; c.rows[t] = 16; }
  _tile_loadconfig(&c);
  done = true;
}

}  // namespace

extern "C" {

// bit 0: AVX-512 VNNI, bit 1: AVX-512 BF16, bit 2: AMX (tile, int8, bf16; permission granted)
int fbx_caps() {
  int c = 0;
  if (__builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl")) {
    if (__builtin_cpu_supports("avx512vnni")) c |= 1;
    if (__builtin_cpu_supports("avx512bf16")) c |= 2;
    if (amx_permitted()) c |= 4;
  }
  return c;
}

// x [M, K] fp32 -> int8 per (row, 128-block): xq [M, K] (deint != 0: every block stored as its 64 even-k values followed by its
// 64 odd-k values, the order the nibble planes of packed int4 weights come in), scale / sum [M, K / 128]
void fbx_quant_act_s8(const float* x, int ldx, int M, int K, int deint, int8_t* xq, float* scale, float* sum) {
  const int nb = K / BLK;
  for (int m = 0; m < M; ++m)
    for (int g = 0; g < nb; ++g) {
      const float* p = x + (size_t)m * ldx + (size_t)g * BLK;
      __m512 mx = _mm512_setzero_ps();
      for (int k = 0; k < BLK; k += 16) mx = _mm512_max_ps(mx, _mm512_abs_ps(_mm512_loadu_ps(p + k)));
      const float amax = _mm512_reduce_max_ps(mx);
      const float sc = amax > 1e-20f ? amax / 127.0f : 1e-20f;
      const __m512 inv = _mm512_set1_ps(1.0f / sc);
      int8_t q[BLK];
      __m512i tot = _mm512_setzero_si512();
      for (int k = 0; k < BLK; k += 16) {
        const __m512i v = _mm512_cvtps_epi32(_mm512_mul_ps(_mm512_loadu_ps(p + k), inv));      // round to nearest even
        tot = _mm512_add_epi32(tot, v);
        _mm_storeu_si128((__m128i*)(q + k), _mm512_cvtsepi32_epi8(v));
      }
      int8_t* o = xq + (size_t)m * K + (size_t)g * BLK;
      if (deint) {
        for (int k = 0; k < BLK / 2; ++k) { o[k] = q[2 * k]; o[BLK / 2 + k] = q[2 * k + 1]; }
      } else {
        std::memcpy(o, q, BLK);
      }
      scale[(size_t)m * nb + g] = sc;
      sum[(size_t)m * nb + g] = (float)_mm512_reduce_add_epi32(tot);
    }
}

void fbx_to_bf16(const float* x, int ldx, int M, int K, uint16_t* xb) {
  for (int m = 0; m < M; ++m) {
    const float* p = x + (size_t)m * ldx;
    uint16_t* o = xb + (size_t)m * K;
    int k = 0;
    for (; k + 32 <= K; k += 32)
      _mm512_storeu_si512((void*)(o + k), (__m512i)_mm512_cvtne2ps_pbh(_mm512_loadu_ps(p + k + 16), _mm512_loadu_ps(p + k)));
    for (; k < K; ++k) {
      uint32_t u;
      std::memcpy(&u, p + k, 4);
      o[k] = (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
    }
  }
}

// ---- AVX-512 BF16: y[m][n] for weight rows [n0, n1), bf16 weights [N, K], activations already bf16 ----
void fbx_linear_rows_bf16(const FbLinearArgs* a, const uint16_t* xb, int n0, int n1) {
  const int K = a->K, M = a->M;
  const uint16_t* W = (const uint16_t*)a->w;
  for (int n = n0; n < n1; ++n) {
    const uint16_t* w = W + (size_t)n * K;
    for (int m0 = 0; m0 < M; m0 += 4) {
      const int mb = M - m0 < 4 ? M - m0 : 4;
      __m512 acc[4] = {_mm512_setzero_ps(), _mm512_setzero_ps(), _mm512_setzero_ps(), _mm512_setzero_ps()};
      int k = 0;
      for (; k + 32 <= K; k += 32) {
        const __m512bh wv = (__m512bh)_mm512_loadu_si512((const void*)(w + k));
        for (int j = 0; j < mb; ++j)
          acc[j] = _mm512_dpbf16_ps(acc[j], wv, (__m512bh)_mm512_loadu_si512((const void*)(xb + (size_t)(m0 + j) * K + k)));
      }
      for (int j = 0; j < mb; ++j) {
        float s = hsum(acc[j]);
        for (int kk = k; kk < K; ++kk) {
          uint32_t wu = (uint32_t)w[kk] << 16, xu = (uint32_t)xb[(size_t)(m0 + j) * K + kk] << 16;
          float wf, xf;
          std::memcpy(&wf, &wu, 4); std::memcpy(&xf, &xu, 4);
          s += wf * xf;
        }
        a->y[(size_t)(m0 + j) * a->ldy + n] = s + (a->bias ? a->bias[n] : 0.f);
      }
    }
  }
}

// ---- AVX-512 VNNI: int8 (wtype 3, per-row scale / zero) and int4 group-128 (wtype 4) weights, int8 activations ----
// xq / xscale / xsum from fbx_quant_act_s8 (deint = 1 for int4g).  K % 128 == 0; int4g needs group == 128.
void fbx_linear_rows_i8(const FbLinearArgs* a, const int8_t* xq, const float* xscale, const float* xsum, int n0, int n1) {
  const int K = a->K, M = a->M, nb = K / BLK;
  const bool i4 = a->wtype == 4;
  const __m512i nib = _mm512_set1_epi8(0x0F);
  for (int n = n0; n < n1; ++n) {
    const uint8_t* w = (const uint8_t*)a->w + (size_t)n * (i4 ? K / 2 : K);
    for (int m = 0; m < M; ++m) {
      const int8_t* xr = xq + (size_t)m * K;
      __m512 acc = _mm512_setzero_ps();
      float corr = 0.f;                                   // the zero-point / minimum term
      for (int g = 0; g < nb; ++g) {
        __m512i d = _mm512_setzero_si512();
        const float as = xscale[(size_t)m * nb + g];
        if (i4) {
          const __m512i pk = _mm512_loadu_si512((const void*)(w + (size_t)g * 64));
          const __m512i hi = _mm512_and_si512(_mm512_srli_epi16(pk, 4), nib), lo = _mm512_and_si512(pk, nib);
          d = _mm512_dpbusd_epi32(d, hi, _mm512_loadu_si512((const void*)(xr + (size_t)g * BLK)));
          d = _mm512_dpbusd_epi32(d, lo, _mm512_loadu_si512((const void*)(xr + (size_t)g * BLK + 64)));
          const float ws = a->scale[(size_t)n * nb + g];
          acc = _mm512_fmadd_ps(_mm512_cvtepi32_ps(d), _mm512_set1_ps(as * ws), acc);
          corr += as * a->zero[(size_t)n * nb + g] * xsum[(size_t)m * nb + g];
        } else {
          d = _mm512_dpbusd_epi32(d, _mm512_loadu_si512((const void*)(w + (size_t)g * BLK)), _mm512_loadu_si512((const void*)(xr + (size_t)g * BLK)));
          d = _mm512_dpbusd_epi32(d, _mm512_loadu_si512((const void*)(w + (size_t)g * BLK + 64)), _mm512_loadu_si512((const void*)(xr + (size_t)g * BLK + 64)));
          acc = _mm512_fmadd_ps(_mm512_cvtepi32_ps(d), _mm512_set1_ps(as), acc);
          corr += as * xsum[(size_t)m * nb + g];
        }
      }
      float y = hsum(acc);
      if (i4) y += corr;
      else y = a->scale[n] * (y - a->zero[n] * corr);
      a->y[(size_t)m * a->ldy + n] = y + (a->bias ? a->bias[n] : 0.f);
    }
  }
}

// ---- AMX: 16 weight rows x 16 activation rows per tile product ----
// C^T[n][m] = W[n][:] . X[m][:]: the weight rows are the A tile straight from row-major storage, the activations are packed
// once per call into the B layout ([k / 4][m][4] for int8, [k / 2][m][2] for bf16), M padded to a multiple of 16.

// xq [M, K] int8 (plain order) -> pk [(M16 / 16)][K / 4][16][4]
void fbx_amx_pack_i8(const int8_t* xq, int M, int K, int8_t* pk) {
  const int M16 = (M + 15) / 16 * 16;
  std::memset(pk, 0, (size_t)M16 * K);
  for (int m = 0; m < M; ++m) {
    int8_t* base = pk + (size_t)(m / 16) * K * 16 + (size_t)(m % 16) * 4;
    const int8_t* src = xq + (size_t)m * K;
    for (int k4 = 0; k4 < K / 4; ++k4) std::memcpy(base + (size_t)k4 * 64, src + (size_t)k4 * 4, 4);
  }
}

// xb [M, K] bf16 -> pk [(M16 / 16)][K / 2][16][2]
void fbx_amx_pack_bf16(const uint16_t* xb, int M, int K, uint16_t* pk) {
  const int M16 = (M + 15) / 16 * 16;
  std::memset(pk, 0, (size_t)M16 * K * 2);
  for (int m = 0; m < M; ++m) {
    uint16_t* base = pk + (size_t)(m / 16) * K * 16 + (size_t)(m % 16) * 2;
    const uint16_t* src = xb + (size_t)m * K;
    for (int k2 = 0; k2 < K / 2; ++k2) std::memcpy(base + (size_t)k2 * 32, src + (size_t)k2 * 2, 4);
  }
}

// bf16 weights, rows [n0, n1) with n0 % 16 == 0 (the last tile may be partial), K % 32 == 0
void fbx_amx_linear_rows_bf16(const FbLinearArgs* a, const uint16_t* pk, int n0, int n1) {
  amx_config();
  const int K = a->K, M = a->M, N = a->N;
  const uint16_t* W = (const uint16_t*)a->w;
  alignas(64) float c[16 * 16];
  alignas(64) uint16_t wt[16 * 32];
  for (int n = n0; n < n1; n += 16) {
    const int rows = N - n < 16 ? N - n : 16;
    for (int mt = 0; mt * 16 < M; ++mt) {
      _tile_zero(0);
      const uint16_t* b = pk + (size_t)mt * K * 16;
      for (int k = 0; k < K; k += 32) {
        if (rows == 16) {
          _tile_loadd(1, W + (size_t)n * K + k, K * 2);
        } else {                                          // ragged last tile: stage the rows that exist, zeros below
          std::memset(wt, 0, sizeof(wt));
          for (int r = 0; r < rows; ++r) std::memcpy(wt + r * 32, W + (size_t)(n + r) * K + k, 64);
          _tile_loadd(1, wt, 64);
        }
        _tile_loadd(2, b + (size_t)(k / 2) * 32, 64);
        _tile_dpbf16ps(0, 1, 2);
      }
      _tile_stored(0, c, 64);
      for (int r = 0; r < rows; ++r)
        for (int j = 0; j < 16 && mt * 16 + j < M; ++j)
          a->y[(size_t)(mt * 16 + j) * a->ldy + n + r] = c[r * 16 + j] + (a->bias ? a->bias[n + r] : 0.f);
    }
  }
}

// int8 weights (wtype 3), rows [n0, n1) with n0 % 16 == 0, K % 128 == 0; activations quantised in plain order
void fbx_amx_linear_rows_i8(const FbLinearArgs* a, const int8_t* pk, const float* xscale, const float* xsum, int n0, int n1) {
  amx_config();
  const int K = a->K, M = a->M, N = a->N, nb = K / BLK;
  const uint8_t* W = (const uint8_t*)a->w;
  alignas(64) int32_t c[16 * 16];
  alignas(64) uint8_t wt[16 * 64];
  for (int n = n0; n < n1; n += 16) {
    const int rows = N - n < 16 ? N - n : 16;
    for (int mt = 0; mt * 16 < M; ++mt) {
      const int cols = M - mt * 16 < 16 ? M - mt * 16 : 16;
      float acc[16][16] = {};
      float corr[16] = {};
      const int8_t* b = pk + (size_t)mt * K * 16;
      for (int g = 0; g < nb; ++g) {
        _tile_zero(0);
        for (int k = g * BLK; k < (g + 1) * BLK; k += 64) {
          if (rows == 16) {
            _tile_loadd(1, W + (size_t)n * K + k, K);
          } else {
            std::memset(wt, 0, sizeof(wt));
            for (int r = 0; r < rows; ++r) std::memcpy(wt + r * 64, W + (size_t)(n + r) * K + k, 64);
            _tile_loadd(1, wt, 64);
          }
          _tile_loadd(2, b + (size_t)(k / 4) * 64, 64);
          _tile_dpbusd(0, 1, 2);
        }
        _tile_stored(0, c, 64);
        for (int j = 0; j < cols; ++j) {
          const float as = xscale[(size_t)(mt * 16 + j) * nb + g];
          corr[j] += as * xsum[(size_t)(mt * 16 + j) * nb + g];
          for (int r = 0; r < rows; ++r) acc[r][j] += as * (float)c[r * 16 + j];
        }
      }
      for (int r = 0; r < rows; ++r)
        for (int j = 0; j < cols; ++j)
          a->y[(size_t)(mt * 16 + j) * a->ldy + n + r] = a->scale[n + r] * (acc[r][j] - a->zero[n + r] * corr[j]) + (a->bias ? a->bias[n + r] : 0.f);
    }
  }
}

}  // extern "C"
