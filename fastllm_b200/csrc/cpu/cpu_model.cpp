// Whole-model forward for dense llama-family decoders on the CPU backend: one native call per scheduler step instead of
// one per operator, so a decode step costs a single foreign-function transition and the worker threads stay hot between
// operators.  Covers: RMSNorm, packed QKV projection (+bias), per-head QK-RMSNorm, RoPE (half-split or interleaved, partial
// rotary), paged-KV append, causal paged attention (GQA, optional sliding window), output projection + residual, SwiGLU MLP
// + residual, final norm and lm_head on selected rows.  Weights may be fp32 / bf16 / fp16 / int8 / int4-group.
//
// The reference runs its CPU models the same way, as a C++ layer loop (src/models/llama.cpp:157-421, src/models/qwen3.cpp
// ForwardV2 :3058-3210); this file is that loop for the paged-KV engine.
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" {
int fbcpu_linear(const float* x, int ldx, const void* w, int wtype, const float* scale, const float* zero, int group,
                 const float* bias, float* y, int ldy, int M, int N, int K);
void fbcpu_rmsnorm(const float* x, int ldx, const float* w, float* y, int ldy, int M, int H, float eps, float unit_offset);
void fbcpu_swiglu(const float* gu, int ld, float* out, int ldo, int M, int inter);
void fbcpu_rope(float* x, int ld, const int* pos, const float* cos_t, const float* sin_t, int rows, int heads, int D, int rot, int mode);
void fbcpu_kv_append(const float* k, int ldk, const float* v, int ldv, const int* slots, float* k_pool, float* v_pool, int T, int row_elems);
int fbcpu_attention_paged(const float* q, int ldq, const float* k_pool, const float* v_pool, const int* page_table, int max_pages,
                          const int* kv_lens, const int* cu_q, float* out, int ldo, int B, int Hq, int Hkv, int D, int page_len,
                          float scale, int window, const float* sinks);
void fbcpu_embedding(const float* table, const int* ids, float* out, int T, int H, float scale);
}

struct FbCpuLinear {
  const void* w; int wtype; const float* scale; const float* zero; int group; const float* bias; int N, K;
  int interleaved;      // gate/up only: rows stored as tiles of 64 gate rows + 64 up rows
};

struct FbCpuLayer {
  const float* ln1; const float* ln2; const float* q_norm; const float* k_norm;
  FbCpuLinear qkv, o, gate_up, down;
};

struct FbCpuModelCfg {
  int hidden, layers, Hq, Hkv, D, inter, vocab, rot, rope_mode, page_len, window;
  float eps, unit_offset, embed_scale, attn_scale, logit_scale;
};

namespace {

struct Model {
  FbCpuModelCfg c;
  std::vector<FbCpuLayer> layers;
  const float* embed = nullptr;
  const float* final_norm = nullptr;
  const float* cos_t = nullptr;
  const float* sin_t = nullptr;
  FbCpuLinear head{};
  std::vector<float> h, x, qkv, attn, gu, act, sel;
};

inline int lin(const FbCpuLinear& l, const float* x, int ldx, float* y, int ldy, int M) {
  return fbcpu_linear(x, ldx, l.w, l.wtype, l.scale, l.zero, l.group, l.bias, y, ldy, M, l.N, l.K);
}

// out[m][i] = silu(gate) * up for tile-interleaved columns (64 gate, 64 up per 128-column tile)
void swiglu_interleaved(const float* gu, int ld, float* out, int ldo, int M, int inter) {
  for (int m = 0; m < M; ++m) {
    const float* r = gu + (size_t)m * ld;
    float* o = out + (size_t)m * ldo;
    for (int t = 0; t < inter / 64; ++t) {
      const float* g = r + (size_t)t * 128;
      const float* u = g + 64;
      for (int i = 0; i < 64; ++i) o[t * 64 + i] = g[i] / (1.0f + std::exp(-g[i])) * u[i];
    }
  }
}

}  // namespace

extern "C" {

void* fbcpu_model_create(const FbCpuModelCfg* cfg) {
  Model* m = new Model();
  m->c = *cfg;
  m->layers.resize(cfg->layers);
  return m;
}

void fbcpu_model_destroy(void* h) { delete static_cast<Model*>(h); }

void fbcpu_model_set_layer(void* h, int i, const FbCpuLayer* l) { static_cast<Model*>(h)->layers[i] = *l; }

void fbcpu_model_set_top(void* h, const float* embed, const float* final_norm, const FbCpuLinear* head, const float* cos_t,
                         const float* sin_t) {
  Model* m = static_cast<Model*>(h);
  m->embed = embed; m->final_norm = final_norm; m->head = *head; m->cos_t = cos_t; m->sin_t = sin_t;
}

// logits_out: [R, vocab] fp32 for the rows in logit_rows (all T rows when logit_rows is null, R = T).
// Returns 0, or a negative code naming the failing stage.
int fbcpu_model_forward(void* handle, const int* ids, const int* pos, const int* slots, int T, const int* page_table, int max_pages,
                        const int* kv_lens, const int* cu_q, int B, float* const* k_pools, float* const* v_pools,
                        const long long* logit_rows, int R, float* logits_out) {
  Model* m = static_cast<Model*>(handle);
  const FbCpuModelCfg& c = m->c;
  const int H = c.hidden, qw = c.Hq * c.D, kw = c.Hkv * c.D, qkvw = qw + 2 * kw;
  m->h.resize((size_t)T * H); m->x.resize((size_t)T * H); m->qkv.resize((size_t)T * qkvw); m->attn.resize((size_t)T * qw);
  m->gu.resize((size_t)T * 2 * c.inter); m->act.resize((size_t)T * c.inter);
  float* h = m->h.data(); float* x = m->x.data(); float* qkv = m->qkv.data(); float* attn = m->attn.data();
  float* gu = m->gu.data(); float* act = m->act.data();

  fbcpu_embedding(m->embed, ids, h, T, H, c.embed_scale);
  for (int li = 0; li < c.layers; ++li) {
    const FbCpuLayer& L = m->layers[li];
    fbcpu_rmsnorm(h, H, L.ln1, x, H, T, H, c.eps, c.unit_offset);
    if (lin(L.qkv, x, H, qkv, qkvw, T) != 0) return -1;
    if (L.q_norm) {
      for (int t = 0; t < T; ++t) fbcpu_rmsnorm(qkv + (size_t)t * qkvw, c.D, L.q_norm, qkv + (size_t)t * qkvw, c.D, c.Hq, c.D, c.eps, c.unit_offset);
    }
    if (L.k_norm) {
      for (int t = 0; t < T; ++t)
        fbcpu_rmsnorm(qkv + (size_t)t * qkvw + qw, c.D, L.k_norm, qkv + (size_t)t * qkvw + qw, c.D, c.Hkv, c.D, c.eps, c.unit_offset);
    }
    fbcpu_rope(qkv, qkvw, pos, m->cos_t, m->sin_t, T, c.Hq, c.D, c.rot, c.rope_mode);
    fbcpu_rope(qkv + qw, qkvw, pos, m->cos_t, m->sin_t, T, c.Hkv, c.D, c.rot, c.rope_mode);
    fbcpu_kv_append(qkv + qw, qkvw, qkv + qw + kw, qkvw, slots, k_pools[li], v_pools[li], T, kw);
    if (fbcpu_attention_paged(qkv, qkvw, k_pools[li], v_pools[li], page_table, max_pages, kv_lens, cu_q, attn, qw, B, c.Hq, c.Hkv,
                              c.D, c.page_len, c.attn_scale, c.window, nullptr) != 0)
      return -2;
    if (lin(L.o, attn, qw, x, H, T) != 0) return -3;
    for (size_t i = 0; i < (size_t)T * H; ++i) h[i] += x[i];
    fbcpu_rmsnorm(h, H, L.ln2, x, H, T, H, c.eps, c.unit_offset);
    if (lin(L.gate_up, x, H, gu, 2 * c.inter, T) != 0) return -4;
    if (L.gate_up.interleaved) swiglu_interleaved(gu, 2 * c.inter, act, c.inter, T, c.inter);
    else fbcpu_swiglu(gu, 2 * c.inter, act, c.inter, T, c.inter);
    if (lin(L.down, act, c.inter, x, H, T) != 0) return -5;
    for (size_t i = 0; i < (size_t)T * H; ++i) h[i] += x[i];
  }
  const float* src = h;
  int rows = T;
  if (logit_rows != nullptr) {
    m->sel.resize((size_t)R * H);
    for (int r = 0; r < R; ++r) std::memcpy(m->sel.data() + (size_t)r * H, h + (size_t)logit_rows[r] * H, (size_t)H * 4);
    src = m->sel.data();
    rows = R;
  }
  fbcpu_rmsnorm(src, H, m->final_norm, x, H, rows, H, c.eps, c.unit_offset);
  if (lin(m->head, x, H, logits_out, m->head.N, rows) != 0) return -6;
  if (c.logit_scale != 1.0f)
    for (size_t i = 0; i < (size_t)rows * m->head.N; ++i) logits_out[i] *= c.logit_scale;
  return 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Routed-expert FFN on the host (hybrid placement: attention and dense layers on the GPU, experts in CPU memory).
//   out[t] += sum_k w[t,k] * down_e( silu(gate_e x_t) * up_e x_t )     over the experts in [first, first + n_local)
// Tokens are bucketed by expert (counting sort), each non-empty expert runs two Linear calls on its bucket.
// Reference: CPU MergeMOE, src/devices/cpu/cpudevice.cpp (MergeMOE op) and the `--moe_device cpu` placement of
// tools/fastllm_pytools/util.py:818-826.
// ---------------------------------------------------------------------------------------------------------------
extern "C" int fbcpu_moe(const float* x, int T, int H, const int* idx, const float* w, int topk, int first, int n_local,
                         const FbCpuLinear* gate_up, const FbCpuLinear* down, float* out) {
  std::vector<int> count(n_local + 1, 0);
  const int pairs = T * topk;
  for (int i = 0; i < pairs; ++i) {
    const int e = idx[i] - first;
    if (e >= 0 && e < n_local) ++count[e + 1];
  }
  for (int e = 0; e < n_local; ++e) count[e + 1] += count[e];
  std::vector<int> order(count[n_local]), fill(count.begin(), count.end() - 1);
  for (int i = 0; i < pairs; ++i) {
    const int e = idx[i] - first;
    if (e >= 0 && e < n_local) order[fill[e]++] = i;
  }
  std::vector<float> xe, gu, act, ye;
  for (int e = 0; e < n_local; ++e) {
    const int n = count[e + 1] - count[e];
    if (n == 0) continue;
    const FbCpuLinear& G = gate_up[e];
    const FbCpuLinear& D = down[e];
    const int inter = G.N / 2;
    xe.resize((size_t)n * H); gu.resize((size_t)n * G.N); act.resize((size_t)n * inter); ye.resize((size_t)n * H);
    for (int r = 0; r < n; ++r) std::memcpy(xe.data() + (size_t)r * H, x + (size_t)(order[count[e] + r] / topk) * H, (size_t)H * 4);
    if (lin(G, xe.data(), H, gu.data(), G.N, n) != 0) return -1;
    if (G.interleaved) swiglu_interleaved(gu.data(), G.N, act.data(), inter, n, inter);
    else fbcpu_swiglu(gu.data(), G.N, act.data(), inter, n, inter);
    if (lin(D, act.data(), inter, ye.data(), H, n) != 0) return -2;
    for (int r = 0; r < n; ++r) {
      const int pair = order[count[e] + r];
      const float wk = w[pair];
      float* o = out + (size_t)(pair / topk) * H;
      const float* y = ye.data() + (size_t)r * H;
      for (int i = 0; i < H; ++i) o[i] += wk * y[i];
    }
  }
  return 0;
}
