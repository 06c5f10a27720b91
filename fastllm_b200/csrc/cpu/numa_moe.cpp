// NUMA-aware routed experts on the host (`--moe_device numa`).
//
// Every expert is cut ACROSS the memory nodes: node j keeps rows [a_j, b_j) of the expert's intermediate dimension of the
// fused gate/up matrix and rows [h_j, h'_j) of the down matrix, in memory that its own pinned threads allocated and first
// touched (so the pages sit on that node).  A forward pass is two phases, the teams of all nodes meeting between them:
//   phase 1  every node: its slice of act = silu(gate) * up for all routed (token, expert) pairs -> shared activation buffer
//   phase 2  every node: its output columns of the down projection for every routed row
// then the rows of a token are scaled by their routing weights and summed in ascending expert order.
// A node streams only its own slice of every expert from its local DRAM; the activations that cross nodes are a few KB per
// token.  Rows of a quantised matrix are independent (per-row scales / per-row groups), so slices are pointer arithmetic
// plus a copy, and the row kernels are the ones the single-node path uses: results equal `fbcpu_moe` bit for bit.
//
// Reference counterpart: the numa expert device (src/devices/numas/numasdevice.cpp:225-231, numas.cpp), which splits
// experts over per-node thread groups the same way and reduces partial sums instead of cutting the down projection by rows.
#ifndef _GNU_SOURCE
#define _GNU_SOURCE
#endif
#include <pthread.h>
#include <sched.h>
#include <unistd.h>

#include <atomic>
#include <cctype>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "cpu_kernels.h"

struct FbCpuLinear {
  const void* w; int wtype; const float* scale; const float* zero; int group; const float* bias; int N, K;
  int interleaved;
};

namespace {

enum WType { W_F32 = 0, W_BF16 = 1, W_F16 = 2, W_INT8 = 3, W_INT4G = 4 };

inline bool has_avx512() {
  static const bool v = __builtin_cpu_supports("avx512f") && __builtin_cpu_supports("avx512bw") && __builtin_cpu_supports("avx512vl");
  return v;
}

// "0-3,8,10-11" -> cpu ids
std::vector<int> parse_cpulist(const std::string& s) {
  std::vector<int> out;
  size_t i = 0;
  while (i < s.size()) {
    while (i < s.size() && !std::isdigit((unsigned char)s[i])) ++i;
    if (i >= s.size()) break;
    int a = 0;
    while (i < s.size() && std::isdigit((unsigned char)s[i])) a = a * 10 + (s[i++] - '0');
    int b = a;
    if (i < s.size() && s[i] == '-') {
      ++i; b = 0;
      while (i < s.size() && std::isdigit((unsigned char)s[i])) b = b * 10 + (s[i++] - '0');
    }
    for (int c = a; c <= b && c < 4096; ++c) out.push_back(c);
  }
  return out;
}

// Memory nodes and the CPUs of each that this process may run on.  FB_NUMA_NODES="0-3;4-7" overrides the system's view
// (one group per ';'), which is also how a single-node machine exercises the multi-node code.
std::vector<std::vector<int>> detect_nodes() {
  cpu_set_t allowed;
  CPU_ZERO(&allowed);
  const bool have_mask = sched_getaffinity(0, sizeof(allowed), &allowed) == 0;
  std::vector<std::vector<int>> nodes;
  auto keep = [&](const std::vector<int>& cpus) {
    std::vector<int> ok;
    for (int c : cpus) if (!have_mask || (c < CPU_SETSIZE && CPU_ISSET(c, &allowed))) ok.push_back(c);
    if (!ok.empty()) nodes.push_back(ok);
  };
  if (const char* e = std::getenv("FB_NUMA_NODES")) {
    std::string s(e);
    size_t p = 0;
    while (p <= s.size()) {
      const size_t q = s.find(';', p);
      keep(parse_cpulist(s.substr(p, q == std::string::npos ? std::string::npos : q - p)));
      if (q == std::string::npos) break;
      p = q + 1;
    }
  } else {
    for (int n = 0; n < 64; ++n) {
      std::ifstream f("/sys/devices/system/node/node" + std::to_string(n) + "/cpulist");
      if (!f) continue;
      std::string line;
      std::getline(f, line);
      keep(parse_cpulist(line));
    }
  }
  if (nodes.empty()) {
    std::vector<int> all;
    const int n = (int)std::thread::hardware_concurrency();
    for (int c = 0; c < (n > 0 ? n : 1); ++c) all.push_back(c);
    nodes.push_back(all);
  }
  return nodes;
}

// One group of pinned threads per node.  run(fn) executes fn(node, worker, workers_of_node) on every worker of every node
// and returns when all are done; meet() is a barrier over all workers, for use inside fn.
class NodeTeams {
 public:
  explicit NodeTeams(const std::vector<std::vector<int>>& nodes, int max_per_node) {
    for (size_t n = 0; n < nodes.size(); ++n) {
      int k = (int)nodes[n].size();
      if (max_per_node > 0 && k > max_per_node) k = max_per_node;
      per_node_.push_back(k);
      total_ += k;
    }
    for (size_t n = 0; n < nodes.size(); ++n)
      for (int w = 0; w < per_node_[n]; ++w) threads_.emplace_back([this, n, w, cpus = nodes[n]] { loop((int)n, w, cpus); });
  }
  ~NodeTeams() {
    { std::lock_guard<std::mutex> lk(mu_); quit_ = true; ++epoch_; }
    cv_.notify_all();
    for (auto& t : threads_) t.join();
  }
  int nodes() const { return (int)per_node_.size(); }
  int workers(int node) const { return per_node_[node]; }

  void run(const std::function<void(int, int, int)>& fn) {
    std::unique_lock<std::mutex> lk(mu_);
    fn_ = &fn;
    pending_ = total_;
    ++epoch_;
    cv_.notify_all();
    done_.wait(lk, [&] { return pending_ == 0; });
    fn_ = nullptr;
  }
  void meet() {                     // sense-reversing barrier over all workers
    const int gen = bar_gen_.load(std::memory_order_acquire);
    if (bar_count_.fetch_add(1, std::memory_order_acq_rel) == total_ - 1) {
      bar_count_.store(0, std::memory_order_relaxed);
      bar_gen_.fetch_add(1, std::memory_order_release);
    } else {
      int spins = 0;
      while (bar_gen_.load(std::memory_order_acquire) == gen) {
        if (++spins > 2000) { std::this_thread::yield(); spins = 0; }
      }
    }
  }

 private:
  void loop(int node, int worker, const std::vector<int>& cpus) {
    cpu_set_t set;
    CPU_ZERO(&set);
    for (int c : cpus) if (c < CPU_SETSIZE) CPU_SET(c, &set);
    pthread_setaffinity_np(pthread_self(), sizeof(set), &set);      // any CPU of the node: the kernel balances inside it
    uint64_t seen = 0;
    for (;;) {
      const std::function<void(int, int, int)>* fn;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return epoch_ != seen; });
        seen = epoch_;
        if (quit_) return;
        fn = fn_;
      }
      (*fn)(node, worker, per_node_[node]);
      {
        std::lock_guard<std::mutex> lk(mu_);
        if (--pending_ == 0) done_.notify_all();
      }
    }
  }
  std::vector<int> per_node_;
  int total_ = 0;
  std::vector<std::thread> threads_;
  std::mutex mu_;
  std::condition_variable cv_, done_;
  const std::function<void(int, int, int)>* fn_ = nullptr;
  uint64_t epoch_ = 0;
  int pending_ = 0;
  bool quit_ = false;
  std::atomic<int> bar_count_{0}, bar_gen_{0};
};

size_t row_bytes(int wtype, int K) {
  switch (wtype) {
    case W_F32: return (size_t)K * 4;
    case W_BF16: case W_F16: return (size_t)K * 2;
    case W_INT8: return (size_t)K;
    default: return (size_t)K / 2;
  }
}

// rows [r0, r1) of a linear layer, copied into memory owned by the caller (the node's thread: first touch decides the node)
struct Slice {
  std::vector<uint8_t> w;
  std::vector<float> scale, zero, bias;
  FbCpuLinear lin{};
  void take(const FbCpuLinear& src, const std::vector<std::pair<int, int>>& ranges) {
    const size_t rb = row_bytes(src.wtype, src.K);
    const int spr = src.wtype == W_INT8 ? 1 : src.wtype == W_INT4G ? src.K / src.group : 0;      // scale entries per row
    int rows = 0;
    for (auto& r : ranges) rows += r.second - r.first;
    w.resize(rb * rows);
    if (spr) { scale.resize((size_t)spr * rows); if (src.zero) zero.resize((size_t)spr * rows); }
    if (src.bias) bias.resize(rows);
    int at = 0;
    for (auto& r : ranges) {
      const int n = r.second - r.first;
      std::memcpy(w.data() + rb * at, (const uint8_t*)src.w + rb * r.first, rb * n);
      if (spr) {
        std::memcpy(scale.data() + (size_t)spr * at, src.scale + (size_t)spr * r.first, (size_t)spr * n * 4);
        if (src.zero) std::memcpy(zero.data() + (size_t)spr * at, src.zero + (size_t)spr * r.first, (size_t)spr * n * 4);
      }
      if (src.bias) std::memcpy(bias.data() + at, src.bias + r.first, (size_t)n * 4);
      at += n;
    }
    lin = src;
    lin.w = w.data(); lin.scale = spr ? scale.data() : nullptr; lin.zero = (spr && src.zero) ? zero.data() : nullptr;
    lin.bias = src.bias ? bias.data() : nullptr; lin.N = rows;
  }
};

struct NodeExpert {
  Slice gate_up, down;      // gate_up: [2 * (b - a), H] gate rows then up rows of the node's intermediate range; down: [h1 - h0, I]
  int a = 0, b = 0, h0 = 0, h1 = 0;
};

struct NumaMoE {
  std::vector<std::vector<int>> node_cpus;
  NodeTeams* teams = nullptr;
  int n_local = 0, H = 0, I = 0;
  std::vector<std::vector<NodeExpert>> ex;       // [node][expert]
  ~NumaMoE() { delete teams; }
};

// rows [r0, r1) of a linear layer as a view (rows of every storage format are independent)
FbCpuLinear sub_rows(const FbCpuLinear& l, int r0, int r1) {
  FbCpuLinear v = l;
  const int spr = l.wtype == W_INT8 ? 1 : l.wtype == W_INT4G ? l.K / l.group : 0;
  v.w = (const uint8_t*)l.w + row_bytes(l.wtype, l.K) * r0;
  if (l.scale) v.scale = l.scale + (size_t)spr * r0;
  if (l.zero) v.zero = l.zero + (size_t)spr * r0;
  if (l.bias) v.bias = l.bias + r0;
  v.N = r1 - r0;
  return v;
}

void linear_rows(const FbCpuLinear& l, const float* x, int ldx, const float* xsum, float* y, int ldy, int M, int n0, int n1) {
  FbLinearArgs a;
  a.x = x; a.ldx = ldx; a.w = l.w; a.wtype = l.wtype; a.scale = l.scale; a.zero = l.zero; a.group = l.group; a.bias = l.bias;
  a.xsum = xsum; a.y = y; a.ldy = ldy; a.M = M; a.N = l.N; a.K = l.K;
  if (has_avx512()) fbk_linear_rows_avx512(&a, n0, n1); else fbk_linear_rows_avx2(&a, n0, n1);
}
void group_sums(const float* x, int ldx, int M, int K, int g, float* out) {
  if (has_avx512()) fbk_group_sums_avx512(x, ldx, M, K, g, out); else fbk_group_sums_avx2(x, ldx, M, K, g, out);
}

}  // namespace

extern "C" {

int fbnuma_node_count() { return (int)detect_nodes().size(); }

// Builds the per-node slices (copies made by each node's own threads).  gate_up[e]: [2I, H] (gate | up halves, or tiles of
// 64 gate + 64 up rows when `interleaved`), down[e]: [H, I].  threads_per_node <= 0: every allowed CPU of the node.
void* fbnuma_create(const FbCpuLinear* gate_up, const FbCpuLinear* down, int n_local, int threads_per_node) {
  if (n_local <= 0) return nullptr;
  NumaMoE* m = new NumaMoE();
  m->node_cpus = detect_nodes();
  const int nodes = (int)m->node_cpus.size();
  m->teams = new NodeTeams(m->node_cpus, threads_per_node);
  m->n_local = n_local;
  m->H = down[0].N;
  m->I = down[0].K;
  const int I = m->I, H = m->H;
  const int unit = gate_up[0].interleaved ? 64 : 8;          // the intermediate range of a node is a multiple of this
  m->ex.assign(nodes, std::vector<NodeExpert>(n_local));
  std::atomic<int> bad{0};
  m->teams->run([&](int node, int worker, int) {
    if (worker != 0) return;                                   // one thread per node allocates and touches the node's copy
    const int units = I / unit;
    const int a = (int)((long long)units * node / nodes) * unit, b = (int)((long long)units * (node + 1) / nodes) * unit;
    const int h0 = (int)((long long)(H / 8) * node / nodes) * 8;
    const int h1 = node == nodes - 1 ? H : (int)((long long)(H / 8) * (node + 1) / nodes) * 8;
    for (int e = 0; e < n_local; ++e) {
      const FbCpuLinear& G = gate_up[e];
      const FbCpuLinear& D = down[e];
      if (G.N != 2 * I || D.K != I || D.N != H || I % unit != 0) { bad++; return; }
      NodeExpert& ne = m->ex[node][e];
      ne.a = a; ne.b = (node == nodes - 1) ? I : b; ne.h0 = h0; ne.h1 = h1;
      std::vector<std::pair<int, int>> gr, ur;
      if (G.interleaved) {
        for (int t = ne.a / 64; t < ne.b / 64; ++t) { gr.push_back({t * 128, t * 128 + 64}); ur.push_back({t * 128 + 64, t * 128 + 128}); }
      } else {
        gr.push_back({ne.a, ne.b});
        ur.push_back({I + ne.a, I + ne.b});
      }
      gr.insert(gr.end(), ur.begin(), ur.end());               // local layout: all gate rows, then all up rows
      ne.gate_up.take(G, gr);
      ne.gate_up.lin.interleaved = 0;
      ne.down.take(D, {{ne.h0, ne.h1}});
    }
  });
  if (bad.load()) { delete m; return nullptr; }
  return m;
}

void fbnuma_destroy(void* h) { delete static_cast<NumaMoE*>(h); }
int fbnuma_nodes(void* h) { return (int)static_cast<NumaMoE*>(h)->node_cpus.size(); }

// out[T, H] += sum over the routed local experts of w * down(silu(gate(x)) * up(x)); same arguments and the same summation
// order per token (ascending expert) as fbcpu_moe.
int fbnuma_moe(void* h, const float* x, int T, int H, const int* idx, const float* w, int topk, int first, float* out) {
  NumaMoE& m = *static_cast<NumaMoE*>(h);
  if (H != m.H) return -1;
  const int n_local = m.n_local, I = m.I, pairs = T * topk;
  const int nodes = (int)m.node_cpus.size();
  std::vector<int> count(n_local + 1, 0);
  for (int i = 0; i < pairs; ++i) {
    const int e = idx[i] - first;
    if (e >= 0 && e < n_local) ++count[e + 1];
  }
  int active = 0;
  for (int e = 0; e < n_local; ++e) { active += count[e + 1] > 0; count[e + 1] += count[e]; }
  const int routed = count[n_local];
  if (routed == 0) return 0;
  std::vector<int> order(routed), fill(count.begin(), count.end() - 1), row_of_pair(pairs, -1);
  for (int i = 0; i < pairs; ++i) {
    const int e = idx[i] - first;
    if (e >= 0 && e < n_local) { row_of_pair[i] = fill[e]; order[fill[e]++] = i; }
  }
  // tasks of a phase: (expert, chunk of the node's slice); about four per worker so a slow core takes fewer
  int max_workers = 1;
  for (int n = 0; n < nodes; ++n) if (m.teams->workers(n) > max_workers) max_workers = m.teams->workers(n);
  int chunks = (4 * max_workers + active - 1) / active;
  if (chunks < 1) chunks = 1;
  if (chunks > 16) chunks = 16;
  std::vector<int> active_experts;
  for (int e = 0; e < n_local; ++e) if (count[e + 1] > count[e]) active_experts.push_back(e);
  const int n_tasks = (int)active_experts.size() * chunks;
  // gathered inputs, the shared activation buffer and the per-row expert outputs, in routed order
  std::vector<float> xe((size_t)routed * H), act((size_t)routed * I), ys((size_t)routed * H);
  const FbCpuLinear& g0 = m.ex[0][0].gate_up.lin;
  const FbCpuLinear& d0 = m.ex[0][0].down.lin;
  const int gx = g0.wtype == W_INT8 ? H : g0.wtype == W_INT4G ? g0.group : 0;       // group length of the activation sums
  const int gd = d0.wtype == W_INT8 ? I : d0.wtype == W_INT4G ? d0.group : 0;
  std::vector<float> xsum(gx ? (size_t)routed * (H / gx) : 0), asum(gd ? (size_t)routed * (I / gd) : 0);
  std::vector<std::atomic<int>> claim1(nodes), claim2(nodes);
  for (auto& c : claim1) c.store(0);
  for (auto& c : claim2) c.store(0);
  std::atomic<int> gather_claim{0}, asum_claim{0}, token_claim{0};
  NodeTeams& teams = *m.teams;
  auto chunk_range = [](int width, int unit, int k, int K, int& r0, int& r1) {
    const int units = width / unit;
    r0 = (int)((long long)units * k / K) * unit;
    r1 = k == K - 1 ? width : (int)((long long)units * (k + 1) / K) * unit;
  };
  teams.run([&](int node, int, int) {
    // gather + activation group sums: rows are claimed by all workers of all nodes
    for (;;) {
      const int r = gather_claim.fetch_add(1, std::memory_order_relaxed);
      if (r >= routed) break;
      std::memcpy(xe.data() + (size_t)r * H, x + (size_t)(order[r] / topk) * H, (size_t)H * 4);
      if (gx) group_sums(xe.data() + (size_t)r * H, H, 1, H, gx, xsum.data() + (size_t)r * (H / gx));
    }
    teams.meet();
    // phase 1: this node's intermediate range of every routed expert
    std::vector<float> gbuf, ubuf;
    for (;;) {
      const int t = claim1[node].fetch_add(1, std::memory_order_relaxed);
      if (t >= n_tasks) break;
      const int e = active_experts[t / chunks];
      const int n = count[e + 1] - count[e];
      const NodeExpert& ne = m.ex[node][e];
      const int width = ne.b - ne.a;
      int i0, i1;
      chunk_range(width, 8, t % chunks, chunks, i0, i1);
      if (i1 <= i0) continue;
      const int cw = i1 - i0;
      gbuf.resize((size_t)n * cw); ubuf.resize((size_t)n * cw);
      const float* xin = xe.data() + (size_t)count[e] * H;
      const float* xs = gx ? xsum.data() + (size_t)count[e] * (H / gx) : nullptr;
      const FbCpuLinear gv = sub_rows(ne.gate_up.lin, i0, i1), uv = sub_rows(ne.gate_up.lin, width + i0, width + i1);
      linear_rows(gv, xin, H, xs, gbuf.data(), cw, n, 0, cw);
      linear_rows(uv, xin, H, xs, ubuf.data(), cw, n, 0, cw);
      for (int r = 0; r < n; ++r) {
        const float* g = gbuf.data() + (size_t)r * cw;
        const float* u = ubuf.data() + (size_t)r * cw;
        float* o = act.data() + (size_t)(count[e] + r) * I + ne.a + i0;
        for (int i = 0; i < cw; ++i) o[i] = g[i] / (1.0f + std::exp(-g[i])) * u[i];
      }
    }
    teams.meet();
    if (gd) {
      for (;;) {
        const int r = asum_claim.fetch_add(1, std::memory_order_relaxed);
        if (r >= routed) break;
        group_sums(act.data() + (size_t)r * I, I, 1, I, gd, asum.data() + (size_t)r * (I / gd));
      }
      teams.meet();
    }
    // phase 2: this node's output columns of every routed row
    for (;;) {
      const int t = claim2[node].fetch_add(1, std::memory_order_relaxed);
      if (t >= n_tasks) break;
      const int e = active_experts[t / chunks];
      const int n = count[e + 1] - count[e];
      const NodeExpert& ne = m.ex[node][e];
      const int width = ne.h1 - ne.h0;
      int c0, c1;
      chunk_range(width, 8, t % chunks, chunks, c0, c1);
      if (c1 <= c0) continue;
      const FbCpuLinear dv = sub_rows(ne.down.lin, c0, c1);
      linear_rows(dv, act.data() + (size_t)count[e] * I, I, gd ? asum.data() + (size_t)count[e] * (I / gd) : nullptr,
                  ys.data() + (size_t)count[e] * H + ne.h0 + c0, H, n, 0, c1 - c0);
    }
    teams.meet();
    // weighted sum per token, experts in ascending order (the order of the single-node path)
    for (;;) {
      const int tkn = token_claim.fetch_add(1, std::memory_order_relaxed);
      if (tkn >= T) break;
      int rows[64], exps[64], k = 0;
      for (int j = 0; j < topk && k < 64; ++j) {
        const int r = row_of_pair[tkn * topk + j];
        if (r < 0) continue;
        int at = k++;
        const int e = idx[tkn * topk + j];
        while (at > 0 && exps[at - 1] > e) { exps[at] = exps[at - 1]; rows[at] = rows[at - 1]; --at; }
        exps[at] = e; rows[at] = r;
      }
      float* o = out + (size_t)tkn * H;
      for (int j = 0; j < k; ++j) {
        const float wk = w[order[rows[j]]];
        const float* y = ys.data() + (size_t)rows[j] * H;
        for (int i = 0; i < H; ++i) o[i] += wk * y[i];
      }
    }
  });
  return 0;
}

}  // extern "C"
