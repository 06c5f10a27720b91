// Unigram (SentencePiece-style) tokenizer core: Viterbi segmentation over a scored piece vocabulary, with byte
// fallback pieces (<0xNN>) for characters outside the vocabulary, and the Metaspace convention (U+2581 for spaces).
// Counterpart of the reference's UnigramEncode (src/tokenizer.cpp:211-310); fed from the "Unigram" model of a
// tokenizer.json by fastllm_b200/tokenizer.py.
#include <cstdint>
#include <cstring>
#include <limits>
#include <string>
#include <unordered_map>
#include <vector>

namespace {

struct Unigram {
  std::unordered_map<std::string, int> piece_to_id;
  std::vector<std::string> pieces;
  std::vector<float> scores;
  std::unordered_map<std::string, int> specials;
  std::vector<char> is_special;
  int unk_id = 0;
  int byte_ids[256];
  bool has_bytes = false;
  size_t max_len = 1;
  float min_score = 0.f;
};

inline int utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 0x6 ? 2 : (c >> 4) == 0xE ? 3 : (c >> 3) == 0x1E ? 4 : 1; }

// best segmentation of text[0, n) into vocabulary pieces (maximum total score)
void viterbi(const Unigram& u, const std::string& text, std::vector<int>& out) {
  const size_t n = text.size();
  const float NEG = -std::numeric_limits<float>::infinity();
  std::vector<float> best(n + 1, NEG);
  std::vector<int> back_pos(n + 1, -1), back_id(n + 1, -1);
  best[0] = 0.f;
  const float unk_pen = u.min_score - 10.0f;
  for (size_t i = 0; i < n; ++i) {
    if (best[i] == NEG) continue;
    if ((static_cast<unsigned char>(text[i]) & 0xC0) == 0x80) continue;      // not a character boundary
    const size_t lim = std::min(n, i + u.max_len);
    for (size_t j = i + 1; j <= lim; ++j) {
      if (j < n && (static_cast<unsigned char>(text[j]) & 0xC0) == 0x80) continue;
      auto it = u.piece_to_id.find(text.substr(i, j - i));
      if (it == u.piece_to_id.end()) continue;
      const float sc = best[i] + u.scores[it->second];
      if (sc > best[j]) { best[j] = sc; back_pos[j] = (int)i; back_id[j] = it->second; }
    }
    // unknown character: one step over it with a penalty (id -1 = expand to bytes / unk afterwards)
    const size_t j = std::min(n, i + (size_t)utf8_len((unsigned char)text[i]));
    const float sc = best[i] + unk_pen;
    if (sc > best[j]) { best[j] = sc; back_pos[j] = (int)i; back_id[j] = -1; }
  }
  std::vector<std::pair<int, int>> segs;      // (start, id) from the end
  for (int p = (int)n; p > 0;) {
    segs.emplace_back(back_pos[p], back_id[p]);
    p = back_pos[p];
  }
  int prev_unk = 0;
  for (auto it = segs.rbegin(); it != segs.rend(); ++it) {
    const int start = it->first, id = it->second;
    if (id >= 0) { out.push_back(id); prev_unk = 0; continue; }
    const int len = utf8_len((unsigned char)text[start]);
    if (u.has_bytes) {
      for (int k = 0; k < len && start + k < (int)n; ++k) out.push_back(u.byte_ids[(unsigned char)text[start + k]]);
    } else if (!prev_unk) {
      out.push_back(u.unk_id);                 // runs of unknown characters collapse into one unk
    }
    prev_unk = !u.has_bytes;
  }
}

}  // namespace

extern "C" {

void* fbuni_create() { Unigram* u = new Unigram(); for (int i = 0; i < 256; ++i) u->byte_ids[i] = -1; return u; }
void fbuni_destroy(void* h) { delete static_cast<Unigram*>(h); }

void fbuni_add_piece(void* h, const char* s, int len, float score) {
  Unigram* u = static_cast<Unigram*>(h);
  std::string p(s, len);
  const int id = (int)u->pieces.size();
  u->pieces.push_back(p);
  u->scores.push_back(score);
  u->is_special.push_back(0);
  u->piece_to_id.emplace(p, id);
  if (p.size() > u->max_len) u->max_len = p.size();
  if (score < u->min_score) u->min_score = score;
  if (len == 6 && p[0] == '<' && p[1] == '0' && p[2] == 'x' && p[5] == '>') {
    const int b = (int)std::strtol(p.substr(3, 2).c_str(), nullptr, 16);
    u->byte_ids[b & 255] = id;
  }
}

void fbuni_finish(void* h, int unk_id, int byte_fallback) {
  Unigram* u = static_cast<Unigram*>(h);
  u->unk_id = unk_id;
  bool all = byte_fallback != 0;
  for (int i = 0; i < 256 && all; ++i) all = u->byte_ids[i] >= 0;
  u->has_bytes = all;
  if (all)                                      // byte pieces are reachable only through the fallback, never by matching "<0x41>" in text
    for (int i = 0; i < 256; ++i) u->piece_to_id.erase(u->pieces[u->byte_ids[i]]);
}

void fbuni_add_special(void* h, const char* s, int len, int id) {
  Unigram* u = static_cast<Unigram*>(h);
  u->specials[std::string(s, len)] = id;
  if (id >= (int)u->pieces.size()) {
    u->pieces.resize(id + 1);
    u->scores.resize(id + 1, 0.f);
    u->is_special.resize(id + 1, 0);
  }
  u->pieces[id] = std::string(s, len);
  u->is_special[id] = 1;
  u->piece_to_id.erase(std::string(s, len));
}

int fbuni_vocab_size(void* h) { return (int)static_cast<Unigram*>(h)->pieces.size(); }

// text is already normalised (spaces replaced by U+2581 where the model wants it).  Special tokens are split out first.
// Returns the number of ids, or -needed when cap is too small.
int fbuni_encode(void* h, const char* text, int len, int* out, int cap) {
  Unigram* u = static_cast<Unigram*>(h);
  std::string s(text, len);
  std::vector<int> ids;
  size_t pos = 0;
  while (pos < s.size()) {
    size_t best_at = std::string::npos, best_len = 0;
    int best_id = -1;
    for (const auto& kv : u->specials) {
      const size_t at = s.find(kv.first, pos);
      if (at != std::string::npos && (at < best_at || (at == best_at && kv.first.size() > best_len))) {
        best_at = at; best_len = kv.first.size(); best_id = kv.second;
      }
    }
    const size_t end = best_at == std::string::npos ? s.size() : best_at;
    if (end > pos) viterbi(*u, s.substr(pos, end - pos), ids);
    if (best_at == std::string::npos) break;
    ids.push_back(best_id);
    pos = best_at + best_len;
  }
  if ((int)ids.size() > cap) return -(int)ids.size();
  for (size_t i = 0; i < ids.size(); ++i) out[i] = ids[i];
  return (int)ids.size();
}

// Concatenated piece bytes (byte pieces become their byte; U+2581 is left in place for the caller to turn into spaces).
int fbuni_decode(void* h, const int* ids, int n, char* out, int cap, int skip_special) {
  Unigram* u = static_cast<Unigram*>(h);
  std::string s;
  for (int i = 0; i < n; ++i) {
    const int id = ids[i];
    if (id < 0 || id >= (int)u->pieces.size()) continue;
    if (u->is_special[id]) { if (!skip_special) s += u->pieces[id]; continue; }
    bool byte_piece = false;
    if (u->has_bytes)
      for (int b = 0; b < 256; ++b) if (u->byte_ids[b] == id) { s.push_back((char)b); byte_piece = true; break; }
    if (!byte_piece) s += u->pieces[id];
  }
  if ((int)s.size() > cap) return -(int)s.size();
  std::memcpy(out, s.data(), s.size());
  return (int)s.size();
}

}  // extern "C"
