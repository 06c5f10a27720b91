// Paged-KV page manager with a prefix-reuse trie (host side, C ABI).
//
// Pages are fixed-size token slots shared by all layers.  A page is either free, private to running
// requests (refcount > 0, not in the trie) or cached: registered in the trie under the chain of
// page-token hashes that leads to it, where it survives with refcount 0 until evicted (leaf-first, least
// recently used).  A new request walks the trie with its prompt and reuses every fully matching page.
// Same role as the reference's PagedCacheManager / CacheTrieNode (include/fastllm.h:643-698,
// src/fastllm.cpp:5238-5558), including its page hash (polynomial, modulus 1000000007).
#include <cstdint>
#include <cstring>
#include <list>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace {

struct Node {
  int page = -1;
  int ref = 0;
  uint64_t tick = 0;
  Node* parent = nullptr;
  uint64_t key = 0;
  std::vector<int> tokens;                       // exact tokens of the page (collision check)
  std::unordered_map<uint64_t, Node*> children;
};

struct Manager {
  int num_pages, page_len;
  std::vector<int> free_list;
  std::vector<int> refcount;                     // per page, requests holding it
  std::vector<Node*> node_of_page;               // trie node if cached
  Node root;
  uint64_t tick = 0;
  long long hits = 0, lookups = 0;
  std::mutex mu;
};

uint64_t hash_page(const int* tok, int n) {
  const uint64_t mod = 1000000007ULL;
  uint64_t h = 0;
  for (int i = 0; i < n; ++i) h = (h * 1000003ULL + (uint64_t)(uint32_t)tok[i] + 1) % mod;
  return h;
}

void free_subtree(Node* n) {
  for (auto& kv : n->children) { free_subtree(kv.second); delete kv.second; }
  n->children.clear();
}

// evict one unreferenced leaf (LRU); returns its page or -1
int evict_one(Manager* m) {
  Node* best = nullptr;
  std::vector<Node*> stack{&m->root};
  while (!stack.empty()) {
    Node* n = stack.back();
    stack.pop_back();
    for (auto& kv : n->children) stack.push_back(kv.second);
    if (n != &m->root && n->children.empty() && n->ref == 0 && m->refcount[n->page] == 0)
      if (!best || n->tick < best->tick) best = n;
  }
  if (!best) return -1;
  const int page = best->page;
  best->parent->children.erase(best->key);
  m->node_of_page[page] = nullptr;
  delete best;
  return page;
}

}  // namespace

extern "C" {

void* fbpm_create(int num_pages, int page_len) {
  Manager* m = new Manager();
  m->num_pages = num_pages;
  m->page_len = page_len;
  m->refcount.assign(num_pages, 0);
  m->node_of_page.assign(num_pages, nullptr);
  m->free_list.reserve(num_pages);
  for (int i = num_pages - 1; i >= 0; --i) m->free_list.push_back(i);
  return m;
}

void fbpm_destroy(void* h) {
  Manager* m = (Manager*)h;
  free_subtree(&m->root);
  delete m;
}

// pages that an allocation could obtain right now: free + cached-but-unreferenced
int fbpm_num_available(void* h) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  int n = (int)m->free_list.size();
  for (int p = 0; p < m->num_pages; ++p)
    if (m->node_of_page[p] && m->refcount[p] == 0) ++n;
  return n;
}

int fbpm_num_free(void* h) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  return (int)m->free_list.size();
}

// allocate n pages (all or nothing); evicts cached pages when the free list runs dry. returns n or 0.
int fbpm_alloc(void* h, int n, int* out) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  std::vector<int> got;
  for (int i = 0; i < n; ++i) {
    int p = -1;
    if (!m->free_list.empty()) { p = m->free_list.back(); m->free_list.pop_back(); }
    else p = evict_one(m);
    if (p < 0) {
      for (int q : got) { m->refcount[q] = 0; m->free_list.push_back(q); }
      return 0;
    }
    m->refcount[p] = 1;
    got.push_back(p);
  }
  for (int i = 0; i < n; ++i) out[i] = got[i];
  return n;
}

// drop one reference on each page; uncached pages whose count reaches 0 return to the free list
void fbpm_release(void* h, const int* pages, int n) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  for (int i = 0; i < n; ++i) {
    const int p = pages[i];
    if (p < 0 || p >= m->num_pages || m->refcount[p] <= 0) continue;
    if (--m->refcount[p] == 0 && m->node_of_page[p] == nullptr) m->free_list.push_back(p);
  }
}

// longest cached prefix in whole pages; takes a reference on each returned page.
// never matches the page containing the last token (its logits must be recomputed).
int fbpm_query(void* h, const int* tokens, int n_tokens, int* out_pages, int max_pages) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  m->lookups++;
  Node* cur = &m->root;
  int matched = 0;
  const int full = (n_tokens - 1) / m->page_len;
  for (int i = 0; i < full && matched < max_pages; ++i) {
    const int* pt = tokens + (size_t)i * m->page_len;
    const uint64_t key = hash_page(pt, m->page_len) * 1000000007ULL + cur->key % 998244353ULL;
    auto it = cur->children.find(key);
    if (it == cur->children.end()) break;
    Node* nd = it->second;
    if (std::memcmp(nd->tokens.data(), pt, sizeof(int) * m->page_len) != 0) break;
    nd->tick = ++m->tick;
    m->refcount[nd->page]++;
    out_pages[matched++] = nd->page;
    cur = nd;
  }
  if (matched) m->hits++;
  return matched;
}

// register the full pages of a sequence (tokens[0 : n_pages*page_len]) in the trie.
// pages already cached under the same prefix keep their existing entry.
void fbpm_record(void* h, const int* tokens, int n_tokens, const int* pages, int n_pages) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  Node* cur = &m->root;
  const int full = n_tokens / m->page_len < n_pages ? n_tokens / m->page_len : n_pages;
  for (int i = 0; i < full; ++i) {
    const int* pt = tokens + (size_t)i * m->page_len;
    const uint64_t key = hash_page(pt, m->page_len) * 1000000007ULL + cur->key % 998244353ULL;
    auto it = cur->children.find(key);
    if (it != cur->children.end()) {
      if (std::memcmp(it->second->tokens.data(), pt, sizeof(int) * m->page_len) != 0) return;  // hash collision: stop
      cur = it->second;
      cur->tick = ++m->tick;
      continue;
    }
    const int p = pages[i];
    if (p < 0 || p >= m->num_pages || m->node_of_page[p] != nullptr) return;
    Node* nd = new Node();
    nd->page = p;
    nd->parent = cur;
    nd->key = key;
    nd->tick = ++m->tick;
    nd->tokens.assign(pt, pt + m->page_len);
    cur->children[key] = nd;
    m->node_of_page[p] = nd;
    cur = nd;
  }
}

// drop every cached page that no request holds
void fbpm_clear_cache(void* h) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  while (true) {
    const int p = evict_one(m);
    if (p < 0) break;
    m->free_list.push_back(p);
  }
}

void fbpm_stats(void* h, long long* out4) {
  Manager* m = (Manager*)h;
  std::lock_guard<std::mutex> g(m->mu);
  int cached = 0;
  for (int p = 0; p < m->num_pages; ++p) if (m->node_of_page[p]) ++cached;
  out4[0] = (long long)m->free_list.size();
  out4[1] = cached;
  out4[2] = m->lookups;
  out4[3] = m->hits;
}

}  // extern "C"
