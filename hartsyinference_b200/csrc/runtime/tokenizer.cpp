// BPE tokenizer cores (host side).
//
// Two merge procedures over a vocabulary of raw byte strings:
//   * rank BPE  (GPT-2 / Llama-3 / Qwen byte-level BPE): a pre-tokenised piece starts as single
//     bytes; the adjacent pair with the lowest merge rank is merged until none is left;
//   * score BPE (SentencePiece-style vocabularies as stored in GGUF: Llama-2, Gemma, Mistral):
//     a piece starts as UTF-8 characters; the adjacent pair whose concatenation is a vocabulary
//     entry with the highest score is merged; leftovers fall back to <0xXX> byte tokens.
// Pre-tokenisation (regex splitting, special tokens, normalisation) is done by the Python front
// end; this file is the hot loop. Decoding is a table lookup with byte-fallback handling.
//
// Reference counterparts: the BPE / SentencePiece / GGUF-embedded tokenizers under
// src/HartsyInference.ModelAssets/Tokenizers/ (27 implementations sharing these two cores).
#include <cstdint>
#include <cstring>
#include <limits>
#include <string>
#include <unordered_map>
#include <vector>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

struct PairHash {
  size_t operator()(const std::pair<int32_t, int32_t>& p) const {
    return std::hash<uint64_t>()((static_cast<uint64_t>(static_cast<uint32_t>(p.first)) << 32) |
                                 static_cast<uint32_t>(p.second));
  }
};

struct Tok {
  std::vector<std::string> vocab;                       // id -> bytes
  std::unordered_map<std::string, int32_t> index;       // bytes -> id
  std::vector<float> scores;                            // score BPE
  std::unordered_map<std::pair<int32_t, int32_t>, std::pair<int32_t, int32_t>, PairHash> merges;  // (a,b) -> (rank, merged id)
  int32_t byte_token[256];                              // id of the single-byte token (rank BPE) or <0xXX> (score BPE)
  int32_t unk = -1;
};

size_t utf8_len(unsigned char c) {
  if (c < 0x80) return 1;
  if ((c >> 5) == 0x6) return 2;
  if ((c >> 4) == 0xE) return 3;
  if ((c >> 3) == 0x1E) return 4;
  return 1;
}

}  // namespace

// tokens: concatenated bytes of all vocabulary entries, lens[i] bytes each.
B200_API void* b200_tok_create(const uint8_t* tokens, const int32_t* lens, int32_t n, const float* scores,
                               int32_t unk_id) {
  auto* t = new Tok();
  t->vocab.reserve(static_cast<size_t>(n));
  size_t off = 0;
  for (int i = 0; i < 256; ++i) t->byte_token[i] = -1;
  for (int32_t i = 0; i < n; ++i) {
    std::string s(reinterpret_cast<const char*>(tokens + off), static_cast<size_t>(lens[i]));
    off += static_cast<size_t>(lens[i]);
    t->index.emplace(s, i);   // first id wins on duplicates
    t->vocab.push_back(std::move(s));
  }
  if (scores) t->scores.assign(scores, scores + n);
  t->unk = unk_id;
  return t;
}
B200_API void b200_tok_destroy(void* h) { delete static_cast<Tok*>(h); }

// Registers merge `rank`: tokens a + b -> merged (ids). Pairs whose parts or result are missing
// from the vocabulary are ignored.
B200_API void b200_tok_add_merge(void* h, int32_t a, int32_t b, int32_t rank) {
  auto* t = static_cast<Tok*>(h);
  if (a < 0 || b < 0 || a >= static_cast<int32_t>(t->vocab.size()) || b >= static_cast<int32_t>(t->vocab.size())) return;
  auto it = t->index.find(t->vocab[static_cast<size_t>(a)] + t->vocab[static_cast<size_t>(b)]);
  if (it == t->index.end()) return;
  t->merges.emplace(std::make_pair(a, b), std::make_pair(rank, it->second));
}
B200_API void b200_tok_set_byte_token(void* h, int32_t byte, int32_t id) {
  if (byte >= 0 && byte < 256) static_cast<Tok*>(h)->byte_token[byte] = id;
}
B200_API int32_t b200_tok_lookup(void* h, const uint8_t* s, int32_t n) {
  auto* t = static_cast<Tok*>(h);
  auto it = t->index.find(std::string(reinterpret_cast<const char*>(s), static_cast<size_t>(n)));
  return it == t->index.end() ? -1 : it->second;
}

// Rank BPE of one pre-tokenised piece. Returns the number of ids written (<= cap) or -1.
B200_API int32_t b200_tok_encode_rank(void* h, const uint8_t* s, int32_t n, int32_t* out, int32_t cap) {
  auto* t = static_cast<Tok*>(h);
  if (n <= 0) return 0;
  // whole piece in the vocabulary: common fast path
  auto whole = t->index.find(std::string(reinterpret_cast<const char*>(s), static_cast<size_t>(n)));
  if (whole != t->index.end()) { if (cap < 1) return -1; out[0] = whole->second; return 1; }
  std::vector<int32_t> sym(static_cast<size_t>(n));
  for (int32_t i = 0; i < n; ++i) {
    int32_t id = t->byte_token[s[i]];
    if (id < 0) id = t->unk;
    sym[static_cast<size_t>(i)] = id;
  }
  while (sym.size() > 1) {
    int32_t best_rank = std::numeric_limits<int32_t>::max(), best_pos = -1, best_id = -1;
    for (size_t i = 0; i + 1 < sym.size(); ++i) {
      auto it = t->merges.find(std::make_pair(sym[i], sym[i + 1]));
      if (it != t->merges.end() && it->second.first < best_rank) {
        best_rank = it->second.first;
        best_pos = static_cast<int32_t>(i);
        best_id = it->second.second;
      }
    }
    if (best_pos < 0) break;
    sym[static_cast<size_t>(best_pos)] = best_id;
    sym.erase(sym.begin() + best_pos + 1);
  }
  if (static_cast<int32_t>(sym.size()) > cap) return -1;
  for (size_t i = 0; i < sym.size(); ++i) out[i] = sym[i];
  return static_cast<int32_t>(sym.size());
}

// Score BPE of one piece of UTF-8 text (already normalised, spaces replaced by U+2581).
B200_API int32_t b200_tok_encode_score(void* h, const uint8_t* s, int32_t n, int32_t* out, int32_t cap) {
  auto* t = static_cast<Tok*>(h);
  std::vector<std::string> sym;
  for (int32_t i = 0; i < n;) {
    size_t l = utf8_len(s[i]);
    if (i + static_cast<int32_t>(l) > n) l = static_cast<size_t>(n - i);
    sym.emplace_back(reinterpret_cast<const char*>(s + i), l);
    i += static_cast<int32_t>(l);
  }
  while (sym.size() > 1) {
    float best = -std::numeric_limits<float>::infinity();
    int32_t pos = -1;
    for (size_t i = 0; i + 1 < sym.size(); ++i) {
      auto it = t->index.find(sym[i] + sym[i + 1]);
      if (it == t->index.end()) continue;
      const float sc = t->scores.empty() ? 0.f : t->scores[static_cast<size_t>(it->second)];
      if (sc > best) { best = sc; pos = static_cast<int32_t>(i); }
    }
    if (pos < 0) break;
    sym[static_cast<size_t>(pos)] += sym[static_cast<size_t>(pos) + 1];
    sym.erase(sym.begin() + pos + 1);
  }
  int32_t w = 0;
  for (const auto& piece : sym) {
    auto it = t->index.find(piece);
    if (it != t->index.end()) {
      if (w >= cap) return -1;
      out[w++] = it->second;
    } else {
      for (unsigned char c : piece) {
        int32_t id = t->byte_token[c];
        if (id < 0) id = t->unk;
        if (id < 0) continue;
        if (w >= cap) return -1;
        out[w++] = id;
      }
    }
  }
  return w;
}

// Bytes of token `id` (empty for out-of-range ids). Returns the length; copies at most cap bytes.
B200_API int32_t b200_tok_bytes(void* h, int32_t id, uint8_t* out, int32_t cap) {
  auto* t = static_cast<Tok*>(h);
  if (id < 0 || id >= static_cast<int32_t>(t->vocab.size())) return 0;
  const std::string& s = t->vocab[static_cast<size_t>(id)];
  const int32_t n = static_cast<int32_t>(s.size());
  memcpy(out, s.data(), static_cast<size_t>(n < cap ? n : cap));
  return n;
}
B200_API int32_t b200_tok_size(void* h) { return static_cast<int32_t>(static_cast<Tok*>(h)->vocab.size()); }
