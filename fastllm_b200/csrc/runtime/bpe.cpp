// Byte-level BPE tokenizer core (host, C ABI).
//
// Same role as the reference's Tokenizer::BytePairEncode / DecodeTokens (src/tokenizer.cpp:312, :664): the
// vocabulary and the merge list come from tokenizer.json (parsed by the Python layer and handed over once),
// encoding applies merges by rank with a priority queue over adjacent pairs, special tokens are split out
// first and mapped to their fixed ids, decoding concatenates token byte strings.  Pre-tokenisation follows
// the GPT-2 / Llama-3 pattern family in a simplified form: contractions, letter runs (non-ASCII bytes count
// as letters), digit runs of at most three, punctuation runs, whitespace handling with a leading space
// attached to the following word.
#include <cstdint>
#include <cstring>
#include <queue>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

struct PairHash {
  size_t operator()(const std::pair<int, int>& p) const { return ((size_t)(uint32_t)p.first << 32) ^ (uint32_t)p.second; }
};

struct Bpe {
  std::unordered_map<std::string, int> vocab;        // token bytes (in the byte->unicode alphabet) -> id
  std::vector<std::string> id_to_token;
  std::unordered_map<std::pair<int, int>, std::pair<int, int>, PairHash> merges;   // (left id, right id) -> (rank, merged id)
  std::vector<std::pair<std::string, int>> specials;  // raw text -> id
  std::string byte_to_uni[256];                        // byte -> UTF-8 of its printable stand-in
  std::unordered_map<std::string, int> uni_to_byte;
  std::vector<std::pair<std::string, std::string>> pending_merges;
  bool merges_ready = false;
  int pre_mode = 0;          // 0 = Llama-3 style split, 1 = GPT-2 style split
};

void append_utf8(std::string& s, int cp) {
  if (cp < 0x80) s.push_back((char)cp);
  else if (cp < 0x800) { s.push_back((char)(0xC0 | (cp >> 6))); s.push_back((char)(0x80 | (cp & 0x3F))); }
  else { s.push_back((char)(0xE0 | (cp >> 12))); s.push_back((char)(0x80 | ((cp >> 6) & 0x3F))); s.push_back((char)(0x80 | (cp & 0x3F))); }
}

void init_alphabet(Bpe* b) {
  // GPT-2 bytes_to_unicode: printable latin-1 bytes map to themselves, the rest to 256 + n
  bool keep[256] = {false};
  for (int c = '!'; c <= '~'; ++c) keep[c] = true;
  for (int c = 0xA1; c <= 0xAC; ++c) keep[c] = true;
  for (int c = 0xAE; c <= 0xFF; ++c) keep[c] = true;
  int n = 0;
  for (int c = 0; c < 256; ++c) {
    const int cp = keep[c] ? c : 256 + n++;
    std::string u;
    append_utf8(u, cp);
    b->byte_to_uni[c] = u;
    b->uni_to_byte[u] = c;
  }
}

bool is_letter(unsigned char c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || c >= 0x80; }
bool is_digit(unsigned char c) { return c >= '0' && c <= '9'; }
bool is_space(unsigned char c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r' || c == '\f' || c == '\v'; }

// split raw bytes into pre-tokens
void pretokenize(const std::string& s, std::vector<std::string>& out) {
  size_t i = 0, n = s.size();
  while (i < n) {
    size_t st = i;
    unsigned char c = s[i];
    // contractions
    if (c == '\'' && i + 1 < n) {
      static const char* suf[] = {"s", "t", "re", "ve", "m", "ll", "d"};
      bool hit = false;
      for (const char* x : suf) {
        size_t L = strlen(x);
        if (i + L < n + 0 && s.compare(i + 1, L, x) == 0) { out.push_back(s.substr(i, L + 1)); i += L + 1; hit = true; break; }
      }
      if (hit) continue;
    }
    // optional single leading non-letter/non-digit/non-newline char followed by letters ("[^\r\n\p{L}\p{N}]?\p{L}+")
    if (is_letter(c) || (!is_digit(c) && c != '\n' && c != '\r' && i + 1 < n && is_letter((unsigned char)s[i + 1]))) {
      if (!is_letter(c)) ++i;
      while (i < n && is_letter((unsigned char)s[i])) ++i;
      out.push_back(s.substr(st, i - st));
      continue;
    }
    if (is_digit(c)) {                       // \p{N}{1,3}
      int k = 0;
      while (i < n && is_digit((unsigned char)s[i]) && k < 3) { ++i; ++k; }
      out.push_back(s.substr(st, i - st));
      continue;
    }
    if (is_space(c)) {
      // \s*[\r\n]+ | \s+(?!\S) | \s+
      size_t j = i;
      while (j < n && is_space((unsigned char)s[j])) ++j;
      size_t last_nl = std::string::npos;
      for (size_t k = i; k < j; ++k) if (s[k] == '\n' || s[k] == '\r') last_nl = k;
      if (last_nl != std::string::npos) { out.push_back(s.substr(i, last_nl + 1 - i)); i = last_nl + 1; continue; }
      if (j < n && j - i > 1) { out.push_back(s.substr(i, j - i - 1)); i = j - 1; continue; }   // leave one space for the next word
      if (j < n && j - i == 1 && !is_space((unsigned char)s[j])) {
        // single space attaches to the following token
        unsigned char d = s[j];
        size_t k = j;
        if (is_letter(d)) { while (k < n && is_letter((unsigned char)s[k])) ++k; }
        else if (is_digit(d)) { out.push_back(s.substr(i, 1)); i = j; continue; }
        else { while (k < n && !is_letter((unsigned char)s[k]) && !is_digit((unsigned char)s[k]) && !is_space((unsigned char)s[k])) ++k; }
        out.push_back(s.substr(i, k - i));
        i = k;
        continue;
      }
      out.push_back(s.substr(i, j - i));
      i = j;
      continue;
    }
    // punctuation run (+ trailing newlines)
    while (i < n && !is_letter((unsigned char)s[i]) && !is_digit((unsigned char)s[i]) && !is_space((unsigned char)s[i])) ++i;
    while (i < n && (s[i] == '\n' || s[i] == '\r')) ++i;
    out.push_back(s.substr(st, i - st));
  }
}

// GPT-2 pattern: 's|'t|'re|'ve|'m|'ll|'d| ?L+| ?N+| ?[^\s L N]+|\s+(?!\S)|\s+
void pretokenize_gpt2(const std::string& s, std::vector<std::string>& out) {
  size_t i = 0, n = s.size();
  auto is_other = [](unsigned char c) { return !is_letter(c) && !is_digit(c) && !is_space(c); };
  while (i < n) {
    const size_t st = i;
    unsigned char c = s[i];
    if (c == '\'' && i + 1 < n) {
      static const char* suf[] = {"s", "t", "re", "ve", "m", "ll", "d"};
      bool hit = false;
      for (const char* x : suf) {
        size_t L = strlen(x);
        if (i + L < n + 0 && s.compare(i + 1, L, x) == 0) { out.push_back(s.substr(i, L + 1)); i += L + 1; hit = true; break; }
      }
      if (hit) continue;
    }
    size_t j = i;
    if (c == ' ' && i + 1 < n && !is_space((unsigned char)s[i + 1])) j = i + 1;     // optional leading space
    unsigned char d = s[j];
    if (!is_space(d)) {
      size_t k = j;
      if (is_letter(d)) while (k < n && is_letter((unsigned char)s[k])) ++k;
      else if (is_digit(d)) while (k < n && is_digit((unsigned char)s[k])) ++k;
      else while (k < n && is_other((unsigned char)s[k])) ++k;
      out.push_back(s.substr(st, k - st));
      i = k;
      continue;
    }
    // whitespace run
    size_t k = i;
    while (k < n && is_space((unsigned char)s[k])) ++k;
    if (k < n && k - i > 1) k -= 1;          // \s+(?!\S): leave the last blank for the next token
    out.push_back(s.substr(i, k - i));
    i = k;
  }
}

void prepare_merges(Bpe* b) {
  if (b->merges_ready) return;
  int rank = 0;
  for (auto& m : b->pending_merges) {
    auto l = b->vocab.find(m.first), r = b->vocab.find(m.second), j = b->vocab.find(m.first + m.second);
    if (l != b->vocab.end() && r != b->vocab.end() && j != b->vocab.end())
      b->merges[{l->second, r->second}] = {rank, j->second};
    ++rank;
  }
  b->pending_merges.clear();
  b->merges_ready = true;
}

void bpe_word(Bpe* b, const std::string& word, std::vector<int>& out) {
  // word: raw bytes.  Start from single-byte tokens, then merge by rank.
  std::string mapped;
  for (unsigned char c : word) mapped += b->byte_to_uni[c];
  auto whole = b->vocab.find(mapped);
  if (whole != b->vocab.end()) { out.push_back(whole->second); return; }
  struct Node { int id; int prev, next; bool alive; };
  std::vector<Node> nodes;
  for (unsigned char c : word) {
    auto it = b->vocab.find(b->byte_to_uni[c]);
    nodes.push_back({it == b->vocab.end() ? 0 : it->second, (int)nodes.size() - 1, (int)nodes.size() + 1, true});
  }
  if (nodes.empty()) return;
  nodes.back().next = -1;
  struct Cand { int rank, pos, left_id, right_id; };
  auto cmp = [](const Cand& a, const Cand& c) { return a.rank != c.rank ? a.rank > c.rank : a.pos > c.pos; };
  std::priority_queue<Cand, std::vector<Cand>, decltype(cmp)> pq(cmp);
  auto push = [&](int i) {
    if (i < 0 || nodes[i].next < 0) return;
    auto it = b->merges.find({nodes[i].id, nodes[nodes[i].next].id});
    if (it != b->merges.end()) pq.push({it->second.first, i, nodes[i].id, nodes[nodes[i].next].id});
  };
  for (int i = 0; i < (int)nodes.size(); ++i) push(i);
  while (!pq.empty()) {
    Cand c = pq.top();
    pq.pop();
    Node& l = nodes[c.pos];
    if (!l.alive || l.next < 0 || l.id != c.left_id || nodes[l.next].id != c.right_id) continue;   // stale
    Node& r = nodes[l.next];
    l.id = b->merges[{c.left_id, c.right_id}].second;
    r.alive = false;
    l.next = r.next;
    if (r.next >= 0) nodes[r.next].prev = c.pos;
    push(l.prev);
    push(c.pos);
  }
  for (int i = 0; i >= 0; i = nodes[i].next) out.push_back(nodes[i].id);
}

}  // namespace

extern "C" {

void* fbtok_create() {
  Bpe* b = new Bpe();
  init_alphabet(b);
  return b;
}
void fbtok_destroy(void* h) { delete (Bpe*)h; }

// token: UTF-8 string in the byte->unicode alphabet (as stored in tokenizer.json)
void fbtok_add_token(void* h, const char* token, int len, int id) {
  Bpe* b = (Bpe*)h;
  std::string t(token, len);
  b->vocab[t] = id;
  if ((int)b->id_to_token.size() <= id) b->id_to_token.resize(id + 1);
  b->id_to_token[id] = t;
}
void fbtok_add_merge(void* h, const char* left, int llen, const char* right, int rlen) {
  Bpe* b = (Bpe*)h;
  b->pending_merges.emplace_back(std::string(left, llen), std::string(right, rlen));
  b->merges_ready = false;
}
// special token: raw text matched verbatim before pre-tokenisation
void fbtok_add_special(void* h, const char* text, int len, int id) {
  Bpe* b = (Bpe*)h;
  b->specials.emplace_back(std::string(text, len), id);
  if ((int)b->id_to_token.size() <= id) b->id_to_token.resize(id + 1);
  if (b->id_to_token[id].empty()) b->id_to_token[id] = std::string("\x01") + std::string(text, len);   // \x01 marks raw text
}

// returns number of ids written (<= max_out); -needed if the buffer is too small
int fbtok_encode(void* h, const char* text, int len, int* out, int max_out) {
  Bpe* b = (Bpe*)h;
  prepare_merges(b);
  std::string s(text, len);
  std::vector<int> ids;
  size_t pos = 0;
  while (pos < s.size()) {
    // earliest special token occurrence (longest on ties)
    size_t best = std::string::npos, best_len = 0;
    int best_id = -1;
    for (auto& sp : b->specials) {
      size_t f = s.find(sp.first, pos);
      if (f != std::string::npos && (f < best || (f == best && sp.first.size() > best_len))) { best = f; best_len = sp.first.size(); best_id = sp.second; }
    }
    const size_t end = best == std::string::npos ? s.size() : best;
    if (end > pos) {
      std::vector<std::string> words;
      if (b->pre_mode == 1) pretokenize_gpt2(s.substr(pos, end - pos), words);
      else pretokenize(s.substr(pos, end - pos), words);
      for (auto& w : words) bpe_word(b, w, ids);
    }
    if (best == std::string::npos) break;
    ids.push_back(best_id);
    pos = best + best_len;
  }
  if ((int)ids.size() > max_out) return -(int)ids.size();
  for (size_t i = 0; i < ids.size(); ++i) out[i] = ids[i];
  return (int)ids.size();
}

// decode to raw bytes; returns byte count (<= max_out) or -needed
int fbtok_decode(void* h, const int* ids, int n, char* out, int max_out, int skip_special) {
  Bpe* b = (Bpe*)h;
  std::string res;
  for (int i = 0; i < n; ++i) {
    const int id = ids[i];
    if (id < 0 || id >= (int)b->id_to_token.size()) continue;
    const std::string& t = b->id_to_token[id];
    if (!t.empty() && t[0] == '\x01') { if (!skip_special) res += t.substr(1); continue; }
    // walk UTF-8 code points of the token and map each back to its byte
    size_t p = 0;
    while (p < t.size()) {
      unsigned char c = t[p];
      size_t L = c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : 4;
      auto it = b->uni_to_byte.find(t.substr(p, L));
      if (it != b->uni_to_byte.end()) res.push_back((char)it->second);
      else res += t.substr(p, L);
      p += L;
    }
  }
  if ((int)res.size() > max_out) return -(int)res.size();
  memcpy(out, res.data(), res.size());
  return (int)res.size();
}

void fbtok_set_pretokenizer(void* h, int mode) { ((Bpe*)h)->pre_mode = mode; }

int fbtok_vocab_size(void* h) { return (int)((Bpe*)h)->id_to_token.size(); }

}  // extern "C"
