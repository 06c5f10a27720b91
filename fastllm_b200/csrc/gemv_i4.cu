// int4-group-128 weights x int8 activations for ONE TO FOUR rows per weight matrix (sm_100a, CUDA cores, dp4a).
//
// Where it runs: routed experts at decode sizes when a rank's experts see about one row each (DeepSeek-V3 on 8 ranks at 32
// requests: 32 rows over 32 local experts), and single-request decoding with int4 weights.  At one or two rows the tensor-core
// route (gemm_i8.cu: nibble unpack in shared memory, MMA, fp32 promotion per k block) spends ~1500 warp instructions per
// 8 KB of packed weights and is instruction-bound (measured 2.4 TB/s of weight stream, issue slots 46 % busy); here a warp
// streams the packed rows straight from global memory and needs ~100 per row chunk:
//     word w = eight weights (high nibble first):  hi = (w >> 4) & 0x0F0F0F0F -> weights 0,2,4,6   lo = w & 0x0F0F0F0F -> 1,3,5,7
//     dot += dp4a(hi, a_even) + dp4a(lo, a_odd)          activations de-interleaved (even | odd bytes per 8) once per CTA
//     y[m][n] = sum_kb a[m,kb] * (s[n,kb] * dot[m,n,kb] + min[n,kb] * xs[m,kb])      same arithmetic as the tensor-core route
// A warp owns eight weight rows at a time (eight 16-byte loads in flight per lane); its 32 lanes cover 1024 consecutive k of
// each row per step, i.e. eight k blocks, four lanes per block.  The (scale, min) pairs of the warp's rows at one k block are
// contiguous in the [kb, n] table the tensor-core route uses, so the same table serves both.
// SwiGLU layout: tiles of 64 gate rows + 64 up rows; a warp takes four gate rows and the four matching up rows.
//
// Reference counterpart: the CUDA-core GEMV kernels for int4 group weights (src/devices/cuda/linear/fastllm-linear-int4group.cu),
// which multiply fp16 activations one weight at a time.
#include "ptx.cuh"
#include "launch.h"
#include "gemm_smallm.cuh"

FB_DEFINE_ERROR_API(gemv_i4)

namespace fb {

struct I4GemvParams {
  const int8_t* xq; int ldq;               // quantised activations [rows, K]
  const float* a_scale; const float* a_sum; int ld_a;     // [kb_total, ld_a]
  const uint8_t* w;                        // packed weights [n_local * N, K / 2]
  const float* pairs;                      // (scale, min) [n_local, kb_total, N, 2]
  void* out; int ld_out;                   // 16-bit [rows, N] (SwiGLU: [rows, N / 2])
  int N, K, kb_total;
  const int* counts; const int* offsets;   // per expert (nullptr: one matrix, rows [0, M))
  int M;
  int swiglu;
};

constexpr int I4_MAX_K = 16384;            // activation rows staged in shared memory: MR * K bytes

__device__ __forceinline__ int dp4a_s(int a, int b, int c) { return __dp4a(a, b, c); }
// streaming 16-byte load of weights (read once: no L1 allocation)
__device__ __forceinline__ uint4 ld_nc_b128(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// One pass of a CTA over its 128 weight rows for MR activation rows starting at `row0` of the activation buffer.
template <int MR, bool BF16>
__device__ __forceinline__ void i4_gemv_pass(const I4GemvParams& p, const uint8_t* __restrict__ w_mat, const float* __restrict__ pairs,
                                             int row0, int valid, int tile, uint8_t* smem) {
  const int K = p.K, kb_total = p.kb_total;
  int* act = reinterpret_cast<int*>(smem);                               // [MR][K / 4] words: per 8 k one even word, one odd word
  float* a_s = reinterpret_cast<float*>(smem + (size_t)MR * K);          // [MR][kb_total]
  float* a_xs = a_s + MR * kb_total;                                     // a_scale * block sum
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __syncthreads();                                                       // the previous pass is done with the staged rows
  for (int i = tid; i < MR * (K >> 3); i += blockDim.x) {
    const int m = i / (K >> 3), j = i - m * (K >> 3);
    int2 o = make_int2(0, 0);
    if (m < valid) {
      const uint2 x = *reinterpret_cast<const uint2*>(p.xq + (size_t)(row0 + m) * p.ldq + (size_t)j * 8);
      o.x = (int)__byte_perm(x.x, x.y, 0x6420);
      o.y = (int)__byte_perm(x.x, x.y, 0x7531);
    }
    *reinterpret_cast<int2*>(act + (size_t)m * (K >> 2) + (size_t)j * 2) = o;
  }
  for (int i = tid; i < MR * kb_total; i += blockDim.x) {
    const int m = i / kb_total, kb = i - m * kb_total;
    float s = 0.f, xs = 0.f;
    if (m < valid) {
      s = p.a_scale[(size_t)kb * p.ld_a + row0 + m];
      xs = p.a_sum[(size_t)kb * p.ld_a + row0 + m] * s;
    }
    a_s[i] = s; a_xs[i] = xs;
  }
  __syncthreads();
  const size_t row_bytes = (size_t)K >> 1;
  const int steps = (K + 1023) >> 10;                                    // 1024 k (512 packed bytes) per warp step
#pragma unroll 1
  for (int pass = 0; pass < 2; ++pass) {
    // rows of this warp: SwiGLU -> gate rows g0..g0+3 and up rows g0+64..g0+67 of the tile; plain -> eight adjacent rows
    const int sub = warp + 8 * pass;                                     // 0..15
    int rows[8];
    if (p.swiglu) {
#pragma unroll
      for (int r = 0; r < 4; ++r) { rows[r] = tile * 128 + sub * 4 + r; rows[4 + r] = rows[r] + 64; }
    } else {
#pragma unroll
      for (int r = 0; r < 8; ++r) rows[r] = tile * 128 + sub * 8 + r;
    }
    float acc[8][MR];
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) acc[r][m] = 0.f;
#pragma unroll 1
    for (int st = 0; st < steps; ++st) {
      const int k0 = (st << 10) + (lane << 5);                           // first k of this lane's 32 weights
      if (k0 >= K) continue;
      const int kb = k0 >> 7;
      uint4 wv[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) wv[r] = ld_nc_b128(w_mat + (size_t)rows[r] * row_bytes + (k0 >> 1));
      // (scale, min) of the eight rows at this k block: two runs of four adjacent rows (SwiGLU) or one run of eight
      float2 sm[8];
      {
        const float2* pr = reinterpret_cast<const float2*>(pairs) + (size_t)kb * p.N;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float4* q = reinterpret_cast<const float4*>(pr + rows[4 * h]);
          const float4 u = __ldg(q), v = __ldg(q + 1);
          sm[4 * h] = make_float2(u.x, u.y); sm[4 * h + 1] = make_float2(u.z, u.w);
          sm[4 * h + 2] = make_float2(v.x, v.y); sm[4 * h + 3] = make_float2(v.z, v.w);
        }
      }
      int4 ae[MR][2];                                                    // this lane's 32 activations per row: e0 o0 e1 o1 | e2 o2 e3 o3
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const int4* ap = reinterpret_cast<const int4*>(act + (size_t)m * (K >> 2) + (k0 >> 2));
        ae[m][0] = ap[0]; ae[m][1] = ap[1];
      }
      const bool first_of_block = (lane & 3) == 0;
      float sa[MR], sx[MR];
#pragma unroll
      for (int m = 0; m < MR; ++m) { sa[m] = a_s[m * kb_total + kb]; sx[m] = first_of_block ? a_xs[m * kb_total + kb] : 0.f; }
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const uint32_t ww[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
        int dot[MR];
#pragma unroll
        for (int m = 0; m < MR; ++m) dot[m] = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int hi = (int)((ww[j] >> 4) & 0x0F0F0F0Fu), lo = (int)(ww[j] & 0x0F0F0F0Fu);
#pragma unroll
          for (int m = 0; m < MR; ++m) {
            const int4 a4 = ae[m][j >> 1];
            const int e = (j & 1) ? a4.z : a4.x, o = (j & 1) ? a4.w : a4.y;
            dot[m] = dp4a_s(hi, e, dp4a_s(lo, o, dot[m]));
          }
        }
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          acc[r][m] += fmaf((float)dot[m] * sm[r].x, sa[m], sm[r].y * sx[m]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < 8; ++r)
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        float v = acc[r][m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        acc[r][m] = v;
      }
    if (lane == 0) {
      if (p.swiglu) {
        uint16_t* out = reinterpret_cast<uint16_t*>(p.out);
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          if (m >= valid) continue;
          float y[4];
#pragma unroll
          for (int r = 0; r < 4; ++r) y[r] = silu_f(acc[r][m]) * acc[4 + r][m];
          const int col = tile * 64 + sub * 4;
          *reinterpret_cast<uint2*>(out + (size_t)(row0 + m) * p.ld_out + col) = make_uint2(pack_16<BF16>(y[0], y[1]), pack_16<BF16>(y[2], y[3]));
        }
      } else {
        uint16_t* out = reinterpret_cast<uint16_t*>(p.out);
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          if (m >= valid) continue;
          const int col = tile * 128 + sub * 8;
          *reinterpret_cast<uint4*>(out + (size_t)(row0 + m) * p.ld_out + col) =
              make_uint4(pack_16<BF16>(acc[0][m], acc[1][m]), pack_16<BF16>(acc[2][m], acc[3][m]), pack_16<BF16>(acc[4][m], acc[5][m]),
                         pack_16<BF16>(acc[6][m], acc[7][m]));
        }
      }
    }
  }
}

// grid (N / 128, experts): a CTA of 256 threads does one 128-row tile of one expert for all of that expert's rows
template <bool BF16>
__global__ void __launch_bounds__(256, 2) i4_gemv_kernel(const I4GemvParams p) {
  extern __shared__ __align__(16) uint8_t smem[];
  pdl_launch_dependents();
  pdl_wait();
  const int e = blockIdx.y, tile = blockIdx.x;
  int cnt = p.M, seg = 0;
  if (p.counts != nullptr) { cnt = p.counts[e]; seg = p.offsets[e]; }
  if (cnt <= 0) return;
  const uint8_t* w_mat = p.w + (size_t)e * p.N * ((size_t)p.K >> 1);
  const float* pairs = p.pairs + (size_t)e * p.kb_total * p.N * 2;
  for (int r0 = 0; r0 < cnt; r0 += 4) {
    const int left = cnt - r0;
    if (left == 1) i4_gemv_pass<1, BF16>(p, w_mat, pairs, seg + r0, 1, tile, smem);
    else if (left == 2) i4_gemv_pass<2, BF16>(p, w_mat, pairs, seg + r0, 2, tile, smem);
    else i4_gemv_pass<4, BF16>(p, w_mat, pairs, seg + r0, left < 4 ? left : 4, tile, smem);
  }
}

}  // namespace fb

using namespace fb;

// out[rows of expert e] = act(xq) x W_e^T for every local expert (counts / offsets as produced by the routing plan), or for one
// matrix and rows [0, M) when counts == nullptr.  Same operands as the tensor-core route (fb_gemm_i8 with wkind = int4 group):
// xq int8 [rows, K] (row stride ldq), a_scale / a_sum [K / 128, ld_a], packed weights [n_local * N, K / 2], (scale, min) pairs
// [n_local, K / 128, N, 2].  flags: GEMM_SWIGLU.  N % 128 == 0, K % 128 == 0, K <= 16384.
extern "C" int fb_gemv_i4(const void* xq, int ldq, const float* a_scale, const float* a_sum, int ld_a, const void* Wq, const float* pairs,
                          void* out, int M, int N, int K, int ld_out, int dtype, int flags, const int* counts, const int* offsets,
                          int n_local, void* stream_) {
  if (counts == nullptr && M <= 0) return 0;
  if (N % 128 != 0 || K % 128 != 0 || K > I4_MAX_K || ldq % 8 != 0 || (dtype != 0 && dtype != 1) || n_local <= 0) return -1;
  if (flags & ~GEMM_SWIGLU) return -1;
  I4GemvParams p;
  p.xq = (const int8_t*)xq; p.ldq = ldq; p.a_scale = a_scale; p.a_sum = a_sum; p.ld_a = ld_a; p.w = (const uint8_t*)Wq; p.pairs = pairs;
  p.out = out; p.ld_out = ld_out; p.N = N; p.K = K; p.kb_total = K / 128; p.counts = counts; p.offsets = offsets; p.M = M;
  p.swiglu = (flags & GEMM_SWIGLU) ? 1 : 0;
  const size_t smem = (size_t)4 * K + (size_t)2 * 4 * (K / 128) * 4;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  static DeviceOnce configured;
  if (configured.need()) {
    cudaError_t e1 = cudaFuncSetAttribute(i4_gemv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * I4_MAX_K + 8 * (I4_MAX_K / 128) * 4);
    cudaError_t e2 = cudaFuncSetAttribute(i4_gemv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * I4_MAX_K + 8 * (I4_MAX_K / 128) * 4);
    if (e1 != cudaSuccess || e2 != cudaSuccess) return (int)(e1 != cudaSuccess ? e1 : e2);
  }
  const dim3 grid(N / 128, counts != nullptr ? n_local : 1);
  if (dtype == 1) launch_k<PDL_GEMM>(i4_gemv_kernel<true>, grid, dim3(256), smem, stream, 0, p);
  else launch_k<PDL_GEMM>(i4_gemv_kernel<false>, grid, dim3(256), smem, stream, 0, p);
  return (int)cudaGetLastError();
}
