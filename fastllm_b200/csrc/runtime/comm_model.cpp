// Host-thread model of the cross-rank counter protocol of the fused tensor-parallel kernels (csrc/comm.cu, comm.cuh):
// one thread per (rank, CTA), std::atomic words in place of the arena header, the same sequence of operations --
//   base = EXPECT (read at launch)           target = base + tp
//   phase 1: write partial rows into every owner's arena
//   sync 1 : CTAs of a rank meet on LOCAL1, the last sends ONE arrival to CNT1 of every rank; wait CNT1 >= target
//   phase 2: the owner sums the tp slots of its rows, writes the result to every rank
//   sync 2 : same through LOCAL2 / CNT2; wait (or, deferred, leave the wait to the consumer of the rows)
//   ticket : the last CTA of the rank publishes EXPECT = target
// and a consumer step that waits CNT2 >= EXPECT before it reads the gathered rows.  The model checks, over many launches with
// random delays, the properties the kernels rely on: every slot read in phase 2 holds this launch's value, every gathered
// row read by the consumer is this launch's, counters only grow, and no wait runs out.  It has no GPU counterpart in the
// reference (its custom all-reduce spins on flags without a bound: src/devices/multicuda/fastllm-custom-allreduce.cu:242-368).
#include <atomic>
#include <chrono>
#include <cstdint>
#include <random>
#include <thread>
#include <vector>

namespace {

struct RankState {
  std::atomic<uint32_t> cnt1{0}, cnt2{0}, expect{0}, ticket{0}, local1{0}, local2{0};
  std::atomic<uint32_t> launch_gate{0};                 // CTAs of a launch start after the previous launch of this rank ended
  std::vector<std::atomic<uint32_t>> part;              // [tp][rows_per] slot s = value pushed by rank s
  std::vector<std::atomic<uint32_t>> x;                 // [tp * rows_per] gathered rows
  explicit RankState(int tp, int rows_per) : part(tp * rows_per), x(tp * rows_per) {}
};

struct Model {
  int tp, ctas, launches, defer, rows_per;
  std::vector<RankState*> ranks;
  std::atomic<int> violations{0}, timeouts{0};
};

bool wait_ge(std::atomic<uint32_t>& c, uint32_t target, Model& m) {
  const auto t0 = std::chrono::steady_clock::now();
  while ((int32_t)(c.load(std::memory_order_acquire) - target) < 0) {
    if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) { m.timeouts++; return false; }
    std::this_thread::yield();
  }
  return true;
}

void jitter(std::mt19937& rng) {
  const int k = (int)(rng() % 64);
  if (k < 4) std::this_thread::sleep_for(std::chrono::microseconds(rng() % 200));
  else if (k < 24) std::this_thread::yield();
}

// value a rank pushes for (launch, source rank, row): distinct per launch so a stale slot is recognised
inline uint32_t val(int launch, int src, int row) { return (uint32_t)(launch * 1000003 + src * 1009 + row + 1); }

void cta_thread(Model& m, int rank, int cta, uint32_t seed) {
  std::mt19937 rng(seed);
  RankState& me = *m.ranks[rank];
  const int tp = m.tp, rp = m.rows_per;
  for (int L = 0; L < m.launches; ++L) {
    // stream order: this launch's CTAs start when the previous launch of this rank has fully ended
    while (me.launch_gate.load(std::memory_order_acquire) < (uint32_t)(L * m.ctas)) std::this_thread::yield();
    jitter(rng);
    if (m.defer && L > 0) {
      // the consumer of launch L-1 (a GEMM of this rank, before launch L in stream order): waits itself, then reads x
      // defer == 2 is the deliberately broken variant (no wait): the model must notice stale rows
      if (m.defer != 2 && !wait_ge(me.cnt2, me.expect.load(std::memory_order_acquire), m)) return;
      for (int i = cta; i < tp * rp; i += m.ctas) {
        uint32_t want = 0;
        for (int s = 0; s < tp; ++s) want += val(L - 1, s, i);
        if (me.x[i].load(std::memory_order_relaxed) != want) m.violations++;
      }
    }
    const uint32_t base = me.expect.load(std::memory_order_acquire);
    const uint32_t target = base + (uint32_t)tp;
    if (base != (uint32_t)(L * tp)) m.violations++;
    // phase 1: push this rank's partial of every row to the row's owner (rows striped over the CTAs)
    for (int i = cta; i < tp * rp; i += m.ctas) {
      const int owner = i / rp;
      m.ranks[owner]->part[rank * rp + (i - owner * rp)].store(val(L, rank, i), std::memory_order_relaxed);
    }
    jitter(rng);
    // sync 1 (aggregated arrival)
    if (me.local1.fetch_add(1, std::memory_order_acq_rel) == (uint32_t)(m.ctas - 1)) {
      me.local1.store(0, std::memory_order_relaxed);
      for (int r = 0; r < tp; ++r) m.ranks[r]->cnt1.fetch_add(1, std::memory_order_release);
    }
    if (!wait_ge(me.cnt1, target, m)) return;
    // phase 2: own rows
    for (int j = cta; j < rp; j += m.ctas) {
      uint32_t sum = 0, want = 0;
      const int row = rank * rp + j;
      for (int s = 0; s < tp; ++s) { sum += me.part[s * rp + j].load(std::memory_order_relaxed); want += val(L, s, row); }
      if (sum != want) m.violations++;
      for (int r = 0; r < tp; ++r) m.ranks[r]->x[row].store(sum, std::memory_order_relaxed);
    }
    jitter(rng);
    // sync 2
    if (me.local2.fetch_add(1, std::memory_order_acq_rel) == (uint32_t)(m.ctas - 1)) {
      me.local2.store(0, std::memory_order_relaxed);
      for (int r = 0; r < tp; ++r) m.ranks[r]->cnt2.fetch_add(1, std::memory_order_release);
    }
    if (!m.defer) {
      if (!wait_ge(me.cnt2, target, m)) return;
      for (int i = cta; i < tp * rp; i += m.ctas) {        // what the next kernel on the stream would read
        uint32_t want = 0;
        for (int s = 0; s < tp; ++s) want += val(L, s, i);
        if (me.x[i].load(std::memory_order_relaxed) != want) m.violations++;
      }
    }
    if (me.ticket.fetch_add(1, std::memory_order_acq_rel) == (uint32_t)(m.ctas - 1)) {
      me.ticket.store(0, std::memory_order_relaxed);
      me.expect.store(target, std::memory_order_release);
    }
    me.launch_gate.fetch_add(1, std::memory_order_acq_rel);
  }
}

}  // namespace

// Runs the model; returns violations + 1000000 * waits that ran out (0 = the protocol held).
extern "C" int fbmodel_comm_protocol(int tp, int ctas, int launches, int defer, int rows_per, unsigned seed) {
  if (tp < 1 || tp > 8 || ctas < 1 || ctas > 16 || launches < 1 || rows_per < 1) return -1;
  Model m;
  m.tp = tp; m.ctas = ctas; m.launches = launches; m.defer = defer; m.rows_per = rows_per;
  for (int r = 0; r < tp; ++r) m.ranks.push_back(new RankState(tp, rows_per));
  std::vector<std::thread> th;
  for (int r = 0; r < tp; ++r)
    for (int c = 0; c < ctas; ++c) th.emplace_back(cta_thread, std::ref(m), r, c, seed * 7919u + (unsigned)(r * 131 + c));
  for (auto& t : th) t.join();
  for (auto* r : m.ranks) delete r;
  return m.violations.load() + 1000000 * m.timeouts.load();
}
