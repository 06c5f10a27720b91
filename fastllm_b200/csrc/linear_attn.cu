// Gated-DeltaNet decode kernels (Qwen3-Next / Qwen3.5 linear-attention layers), one new token per request.
//
//  * gdn_conv_update_kernel: causal depth-wise convolution step.  Every (request, channel) keeps its last K-1 inputs;
//    the step forms silu(sum_j w[c][j] * window[j]) over those plus the new input and shifts the window.
//  * gdn_recurrent_kernel: one CTA per (value head, request), 256 threads.  A thread owns half a column of the head's
//    fp32 state S[Dk = 128][Dv = 128] in registers: decay, read (S^T k), delta write and read-out (S^T q) are per
//    column, the two halves meet through shared memory; the other reductions are the two L2 norms and the gated
//    RMSNorm of the output row.
//    The state is read once and written once per step (128 KB per head and request): the kernel is a pure state stream.
//
// Reference counterparts: the ShiftAppendConv1D family and RecurrentGatedDeltaRule
// (src/devices/cuda/fastllm-cuda.cu:14238-15096, 16514-17912), which run the same steps as separate launches.
#include "ptx.cuh"
#include "launch.h"

FB_DEFINE_ERROR_API(linear_attn)

namespace fb {

template <bool BF16>
__device__ __forceinline__ float ld16(const uint16_t* p) {
  return BF16 ? __bfloat162float(__ushort_as_bfloat16(*p)) : __half2float(__ushort_as_half(*p));
}
template <bool BF16>
__device__ __forceinline__ uint16_t st16(float v) {
  return BF16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}
template <bool BF16>
__global__ void gdn_conv_update_kernel(const uint16_t* __restrict__ x, int ldx, const uint16_t* __restrict__ w,
                                       uint16_t* __restrict__ state, const int* __restrict__ slots, uint16_t* __restrict__ out,
                                       int B, int C, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)B * C) return;
  const int b = (int)(idx / C), c = (int)(idx - (long long)b * C);
  const int slot = slots[b];
  uint16_t* st = state + ((size_t)slot * C + c) * (K - 1);
  float win[8];
  for (int j = 0; j < K - 1; ++j) win[j] = ld16<BF16>(st + j);
  const uint16_t xin = x[(size_t)b * ldx + c];
  win[K - 1] = ld16<BF16>(&xin);
  float acc = 0.f;
  for (int j = 0; j < K; ++j) acc += ld16<BF16>(w + (size_t)c * K + j) * win[j];
  for (int j = 0; j + 1 < K - 1; ++j) st[j] = st[j + 1];
  if (K > 1) st[K - 2] = xin;
  out[(size_t)b * C + c] = st16<BF16>(acc / (1.0f + __expf(-acc)));
}

struct GdnParams {
  const uint16_t* mixed; int ld_mixed;      // [B, 2*Hk*128 + Hv*128] post-convolution q | k | v
  const uint16_t* a; int ld_a;              // [B, Hv] decay gate input
  const uint16_t* b;                        // [B, Hv] write-strength input (same row stride as a)
  const uint16_t* z; int ld_z;              // [B, Hv*128] output gate
  const float* A_log; const float* dt_bias; // [Hv]
  const uint16_t* norm_w;                   // [128]
  float* state;                             // [slots, Hv, 128, 128]
  const int* slots;
  uint16_t* out;                            // [B, Hv*128]
  int B, Hk, Hv;
  float eps;
};

// sum over the first 128 threads' values (threads 128..255 pass 0 and receive the same total)
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return red[0] + red[1] + red[2] + red[3] + red[4] + red[5] + red[6] + red[7];
}

// 256 threads: thread t owns rows [64 * (t / 128), +64) of state column t % 128 (64 registers); the two halves of a column
// meet through shared memory twice (the read S^T k, the read-out S^T q).
template <bool BF16>
__global__ void __launch_bounds__(256) gdn_recurrent_kernel(const GdnParams p) {
  __shared__ float qs[128], ks[128], red[8], part[2][128];
  pdl_launch_dependents();
  pdl_wait();
  const int hv = blockIdx.x, b = blockIdx.y, j = threadIdx.x & 127, half = threadIdx.x >> 7;
  const int rep = p.Hv / p.Hk, hk = hv / rep;
  const int kd = p.Hk * 128;
  const uint16_t* row = p.mixed + (size_t)b * p.ld_mixed;
  const float qv = half == 0 ? ld16<BF16>(row + hk * 128 + j) : 0.f;
  const float kv_in = half == 0 ? ld16<BF16>(row + kd + hk * 128 + j) : 0.f;
  const float vj = ld16<BF16>(row + 2 * kd + hv * 128 + j);
  const float qn = block_sum(qv * qv, red);
  const float kn = block_sum(kv_in * kv_in, red);
  if (half == 0) {
    qs[j] = qv * rsqrtf(qn + 1e-6f) * 0.08838834764831845f;        // 128^-1/2
    ks[j] = kv_in * rsqrtf(kn + 1e-6f);
  }
  const float av = ld16<BF16>(p.a + (size_t)b * p.ld_a + hv) + p.dt_bias[hv];
  const float sp = av > 20.f ? av : log1pf(__expf(av));             // softplus
  const float eg = __expf(-__expf(p.A_log[hv]) * sp);
  const float beta = 1.0f / (1.0f + __expf(-ld16<BF16>(p.b + (size_t)b * p.ld_a + hv)));
  __syncthreads();
  float* S = p.state + ((size_t)p.slots[b] * p.Hv + hv) * 128 * 128 + (size_t)half * 64 * 128;
  const float* kh = ks + half * 64;
  const float* qh = qs + half * 64;
  float s[64];
  float mem = 0.f;
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    s[i] = S[i * 128 + j] * eg;
    mem += s[i] * kh[i];
  }
  part[half][j] = mem;
  __syncthreads();
  const float delta = (vj - (part[0][j] + part[1][j])) * beta;
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < 64; ++i) {
    s[i] += kh[i] * delta;
    o += s[i] * qh[i];
    S[i * 128 + j] = s[i];
  }
  __syncthreads();                     // everyone has read part[] for delta
  part[half][j] = o;
  __syncthreads();
  o = part[0][j] + part[1][j];
  // gated RMSNorm of the head's output row, with the roundings of the unfused sequence (16-bit row, 16-bit normalised row,
  // 16-bit weighted row, then the gate in fp32)
  uint16_t ob = st16<BF16>(o);
  const float of = ld16<BF16>(&ob);
  const float var = block_sum(half == 0 ? of * of : 0.f, red) * (1.0f / 128.0f);
  if (half == 0) {
    uint16_t y1 = st16<BF16>(of * rsqrtf(var + p.eps));
    uint16_t y2 = st16<BF16>(ld16<BF16>(p.norm_w + j) * ld16<BF16>(&y1));
    const float zf = ld16<BF16>(p.z + (size_t)b * p.ld_z + hv * 128 + j);
    p.out[((size_t)b * p.Hv + hv) * 128 + j] = st16<BF16>(ld16<BF16>(&y2) * (zf / (1.0f + __expf(-zf))));
  }
}

}  // namespace fb

using namespace fb;

// x [B, C] (row stride ldx), w [C, K], state [slots, C, K-1] (same 16-bit dtype), slots int32 [B]; out [B, C] = silu(conv step).
extern "C" int fb_gdn_conv_update(const void* x, const void* w, void* state, const int* slots, void* out, int B, int C, int K, int ldx,
                                  int dtype, void* stream_) {
  if (B <= 0) return 0;
  if (K < 1 || K > 8 || (dtype != 0 && dtype != 1)) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const long long total = (long long)B * C;
  const int blocks = (int)((total + 255) / 256);
  if (dtype == 1)
    launch_k(gdn_conv_update_kernel<true>, dim3(blocks), dim3(256), 0, stream, 0, (const uint16_t*)x, ldx, (const uint16_t*)w, (uint16_t*)state, slots, (uint16_t*)out, B, C, K);
  else
    launch_k(gdn_conv_update_kernel<false>, dim3(blocks), dim3(256), 0, stream, 0, (const uint16_t*)x, ldx, (const uint16_t*)w, (uint16_t*)state, slots, (uint16_t*)out, B, C, K);
  return (int)cudaGetLastError();
}

// One gated-delta-rule step for every (request, value head); see GdnParams.  Dk = Dv = 128.
extern "C" int fb_gdn_recurrent(const void* mixed, int ld_mixed, const void* a, int ld_a, const void* b, const void* z, const float* A_log,
                                const float* dt_bias, const void* norm_w, float* state, const int* slots, void* out, int B, int Hk, int Hv,
                                int Dk, int Dv, int ld_z, float eps, int dtype, void* stream_) {
  if (B <= 0) return 0;
  if (Dk != 128 || Dv != 128 || Hk <= 0 || Hv % Hk != 0 || B > 65535 || (dtype != 0 && dtype != 1)) return -1;
  GdnParams p;
  p.mixed = (const uint16_t*)mixed; p.ld_mixed = ld_mixed; p.a = (const uint16_t*)a; p.ld_a = ld_a; p.b = (const uint16_t*)b;
  p.z = (const uint16_t*)z; p.ld_z = ld_z; p.A_log = A_log; p.dt_bias = dt_bias; p.norm_w = (const uint16_t*)norm_w; p.state = state;
  p.slots = slots; p.out = (uint16_t*)out; p.B = B; p.Hk = Hk; p.Hv = Hv; p.eps = eps;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (dtype == 1) launch_k(gdn_recurrent_kernel<true>, dim3(Hv, B), dim3(256), 0, stream, 0, p);
  else launch_k(gdn_recurrent_kernel<false>, dim3(Hv, B), dim3(256), 0, stream, 0, p);
  return (int)cudaGetLastError();
}
