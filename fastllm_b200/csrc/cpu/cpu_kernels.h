// Argument blocks shared by the dispatcher (cpu_ops.cpp) and the ISA-specific kernel file (cpu_kernels.cpp, compiled
// once per instruction set with FB_ISA_SUFFIX = _avx2 / _avx512).  Every kernel entry processes a half-open range of
// independent work items, so the dispatcher can hand ranges to the thread pool.
#pragma once
#include <cstdint>

struct FbLinearArgs {
  const float* x; int ldx;           // [M, K] activations
  const void* w;                     // [N, K] weights in `wtype` storage (int4-group: K/2 bytes per row)
  int wtype;                         // 0 f32, 1 bf16, 2 f16, 3 int8, 4 int4-group
  const float* scale;                // int8: [N]; int4g: [N, K/group]
  const float* zero;                 // int8: zero points [N]; int4g: group minima [N, K/group]
  int group;                         // int4g group length
  const float* bias;                 // [N] or null
  const float* xsum;                 // int8: [M] row sums of x; int4g: [M, K/group] group sums of x
  float* y; int ldy;                 // [M, N]
  int M, N, K;
};

struct FbAttnArgs {
  const float* q; int ldq;           // packed new tokens [T, Hq*D]
  const float* k_pool; const float* v_pool;   // [slots, Hkv, D]
  const int* page_table; int max_pages;       // [B, max_pages]
  const int* kv_lens; const int* cu_q;        // [B], [B+1]
  float* out; int ldo;
  int B, Hq, Hkv, D, page_len;
  float scale;
  int window;                        // sliding window length (0: full causal)
  const float* sinks;                // per-q-head attention-sink logits or null
};

#define FB_DECLARE_KERNELS(SUFFIX)                                                                                      \
  void fbk_linear_rows##SUFFIX(const FbLinearArgs* a, int n0, int n1);                                                  \
  void fbk_group_sums##SUFFIX(const float* x, int ldx, int M, int K, int group, float* out);                            \
  void fbk_rmsnorm_rows##SUFFIX(const float* x, int ldx, const float* w, float* y, int ldy, int H, float eps,           \
                                float unit_offset, int r0, int r1);                                                     \
  void fbk_layernorm_rows##SUFFIX(const float* x, int ldx, const float* w, const float* b, float* y, int ldy, int H,    \
                                  float eps, int r0, int r1);                                                           \
  void fbk_swiglu_rows##SUFFIX(const float* gu, int ld, float* out, int ldo, int inter, int r0, int r1);                \
  void fbk_act_rows##SUFFIX(float* x, int n, int kind);                                                                 \
  void fbk_softmax_rows##SUFFIX(float* x, int ld, int cols, int r0, int r1);                                            \
  void fbk_rope_rows##SUFFIX(float* x, int ld, const int* pos, const float* cos_t, const float* sin_t, int heads, int D, \
                             int rot, int mode, int r0, int r1);                                                        \
  void fbk_attention_items##SUFFIX(const FbAttnArgs* a, int i0, int i1);

extern "C" {
FB_DECLARE_KERNELS(_avx2)
FB_DECLARE_KERNELS(_avx512)
}
