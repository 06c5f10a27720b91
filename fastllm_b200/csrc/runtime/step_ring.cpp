// Step-plan ring: one publisher (the scheduler rank) hands small messages to N-1 consumer processes (the
// other tensor-parallel ranks) through a shared mapping (a file under /dev/shm mapped by every rank).
//
// The reference fans a step out to one host thread per GPU inside one process (spin 2^18 iterations, then a
// condition variable: src/devices/multicuda/multicudadevice.cpp:97-224).  Here every GPU has its own process,
// so the hand-over is a single-producer broadcast ring in shared memory with the same spin-then-sleep waiting.
//
// Layout of the mapping:
//   Header (4 KiB): magic, geometry, head sequence number, one read cursor per consumer, a closed flag
//   n_slots x (SlotHeader + slot_bytes payload)
// Message k lives in slot k % n_slots.  The publisher writes the payload, then the slot's sequence word, then
// the head (release stores); a consumer acquires the head, reads the slot, and publishes its cursor so the
// publisher knows when a slot may be overwritten.  All waits take a timeout and return a status; nothing here
// blocks for ever, so a rank whose peer died finds out and can leave.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>

namespace {

constexpr uint32_t kMagic = 0x46425352u;   // "FBSR"
constexpr int kMaxConsumers = 15;

struct alignas(64) Cursor {
  std::atomic<uint64_t> v;
  char pad[56];
};

struct Header {
  uint32_t magic;
  uint32_t n_slots;
  uint32_t slot_bytes;
  uint32_t n_consumers;
  alignas(64) std::atomic<uint64_t> head;        // number of messages published so far
  alignas(64) std::atomic<uint32_t> closed;
  Cursor cursor[kMaxConsumers];                  // messages consumed so far, per consumer
};

struct SlotHeader {
  std::atomic<uint64_t> seq;                     // index of the message stored here, plus one
  int32_t kind;
  uint32_t nbytes;
  char pad[48];
};

constexpr size_t kHeaderBytes = 4096;
static_assert(sizeof(Header) <= kHeaderBytes, "ring header must fit its page");
static_assert(sizeof(SlotHeader) == 64, "slot header is one cache line");

inline Header* hdr(void* base) { return reinterpret_cast<Header*>(base); }
inline SlotHeader* slot(void* base, uint64_t idx) {
  Header* h = hdr(base);
  char* p = reinterpret_cast<char*>(base) + kHeaderBytes + (idx % h->n_slots) * (sizeof(SlotHeader) + (size_t)h->slot_bytes);
  return reinterpret_cast<SlotHeader*>(p);
}

inline int64_t now_us() {
  return std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

inline void cpu_relax() {
#if defined(__x86_64__) || defined(__i386__)
  __builtin_ia32_pause();
#elif defined(__aarch64__)
  asm volatile("yield" ::: "memory");
#endif
}

// spin for spin_us, then sleep in 50 us naps until the deadline; returns false on timeout
template <class Pred>
bool wait_until(Pred ready, int64_t timeout_us, int64_t spin_us) {
  if (ready()) return true;
  const int64_t t0 = now_us();
  while (true) {
    for (int i = 0; i < 64; ++i) {
      if (ready()) return true;
      cpu_relax();
    }
    const int64_t dt = now_us() - t0;
    if (timeout_us >= 0 && dt > timeout_us) return false;
    if (dt > spin_us) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
}

}  // namespace

extern "C" {

enum { FBRING_OK = 0, FBRING_TIMEOUT = 1, FBRING_CLOSED = 2, FBRING_TOO_BIG = 3, FBRING_BAD = 4, FBRING_OVERRUN = 5 };

uint64_t fbring_bytes(uint32_t n_slots, uint32_t slot_bytes) {
  return kHeaderBytes + (uint64_t)n_slots * (sizeof(SlotHeader) + (uint64_t)slot_bytes);
}

int fbring_init(void* base, uint32_t n_slots, uint32_t slot_bytes, uint32_t n_consumers) {
  if (n_slots == 0 || n_consumers > (uint32_t)kMaxConsumers || (slot_bytes & 63u)) return FBRING_BAD;
  std::memset(base, 0, fbring_bytes(n_slots, slot_bytes));
  Header* h = hdr(base);
  h->n_slots = n_slots;
  h->slot_bytes = slot_bytes;
  h->n_consumers = n_consumers;
  h->head.store(0, std::memory_order_relaxed);
  h->closed.store(0, std::memory_order_relaxed);
  std::atomic_thread_fence(std::memory_order_release);
  h->magic = kMagic;
  return FBRING_OK;
}

int fbring_check(void* base) { return hdr(base)->magic == kMagic ? FBRING_OK : FBRING_BAD; }

void fbring_close(void* base) { hdr(base)->closed.store(1, std::memory_order_release); }

int fbring_is_closed(void* base) { return (int)hdr(base)->closed.load(std::memory_order_acquire); }

uint64_t fbring_head(void* base) { return hdr(base)->head.load(std::memory_order_acquire); }

uint64_t fbring_cursor(void* base, int consumer) { return hdr(base)->cursor[consumer].v.load(std::memory_order_acquire); }

// Publisher: waits until every consumer has released the slot this message goes to, then writes it.
int fbring_publish(void* base, int kind, const void* payload, uint32_t nbytes, int64_t timeout_us) {
  Header* h = hdr(base);
  if (h->magic != kMagic) return FBRING_BAD;
  if (nbytes > h->slot_bytes) return FBRING_TOO_BIG;
  if (h->closed.load(std::memory_order_acquire)) return FBRING_CLOSED;
  const uint64_t k = h->head.load(std::memory_order_relaxed);
  auto slot_free = [&]() {
    if (k < h->n_slots) return true;
    const uint64_t need = k - h->n_slots + 1;           // every consumer must have consumed this many messages
    for (uint32_t c = 0; c < h->n_consumers; ++c)
      if (h->cursor[c].v.load(std::memory_order_acquire) < need) return false;
    return true;
  };
  if (!wait_until(slot_free, timeout_us, 2000)) return FBRING_TIMEOUT;
  SlotHeader* s = slot(base, k);
  s->kind = kind;
  s->nbytes = nbytes;
  if (nbytes) std::memcpy(reinterpret_cast<char*>(s) + sizeof(SlotHeader), payload, nbytes);
  s->seq.store(k + 1, std::memory_order_release);
  h->head.store(k + 1, std::memory_order_release);
  return FBRING_OK;
}

// Consumer: waits for the next message after this consumer's cursor; copies it out and advances the cursor.
// spin_us: how long to busy-wait before napping (serving ranks spin through a decode step's gap, idle ones nap).
int fbring_consume(void* base, int consumer, int* kind, void* out, uint32_t cap, uint32_t* nbytes, int64_t timeout_us,
                   int64_t spin_us) {
  Header* h = hdr(base);
  if (h->magic != kMagic || consumer < 0 || consumer >= (int)h->n_consumers) return FBRING_BAD;
  const uint64_t k = h->cursor[consumer].v.load(std::memory_order_relaxed);
  auto ready = [&]() { return h->head.load(std::memory_order_acquire) > k || h->closed.load(std::memory_order_acquire) != 0; };
  if (!wait_until(ready, timeout_us, spin_us)) return FBRING_TIMEOUT;
  if (h->head.load(std::memory_order_acquire) <= k) return FBRING_CLOSED;      // closed and drained
  SlotHeader* s = slot(base, k);
  if (s->seq.load(std::memory_order_acquire) != k + 1) return FBRING_OVERRUN;   // cannot happen while cursors are honoured
  if (s->nbytes > cap) return FBRING_TOO_BIG;
  *kind = s->kind;
  *nbytes = s->nbytes;
  if (s->nbytes) std::memcpy(out, reinterpret_cast<const char*>(s) + sizeof(SlotHeader), s->nbytes);
  h->cursor[consumer].v.store(k + 1, std::memory_order_release);
  return FBRING_OK;
}

}  // extern "C"
