// Byte-pair-encoding tokenizer compatible with tiktoken for the reference's vocabulary.
//
// Loads ``tokenizer.json`` ({"pattern", "mergeable_ranks": [[base64, rank]..], "special_tokens":
// [[name, rank]..]}) or ``tokenizer.tiktoken`` + ``tokenizer_config.txt``
// (brain/src/feeder/tokenizer.rs:36-228).  The GPT-4 style split pattern
//   '(?i:[sdmt]|ll|ve|re)|[^\r\n\p{L}\p{N}]?+\p{L}+|\p{N}{1,2}| ?[^\s\p{L}\p{N}]++[\r\n]*|\s*[\r\n]|\s+(?!\S)|\s+
// (original/prepare.py:48) is implemented as a hand-written scanner over code points (ordered
// alternation, possessive quantifiers, the negative look-ahead) with generated Unicode tables
// instead of a regex engine; the merge loop is tiktoken's lowest-rank-pair-first rule
// (brain/src/feeder/tokenizer.rs:268-341).
#include "ar_native.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

namespace arn {
extern const uint32_t kLetterRanges[][2];
extern const int kLetterRanges_count;
extern const uint32_t kNumberRanges[][2];
extern const int kNumberRanges_count;
extern const uint32_t kSpaceRanges[][2];
extern const int kSpaceRanges_count;

static bool in_ranges(const uint32_t (*r)[2], int n, uint32_t cp) {
  int lo = 0, hi = n - 1;
  while (lo <= hi) {
    int mid = (lo + hi) >> 1;
    if (cp < r[mid][0]) hi = mid - 1;
    else if (cp > r[mid][1]) lo = mid + 1;
    else return true;
  }
  return false;
}
static inline bool is_letter(uint32_t cp) {
  if (cp < 128) return (cp >= 'a' && cp <= 'z') || (cp >= 'A' && cp <= 'Z');
  return in_ranges(kLetterRanges, kLetterRanges_count, cp);
}
static inline bool is_number(uint32_t cp) {
  if (cp < 128) return cp >= '0' && cp <= '9';
  return in_ranges(kNumberRanges, kNumberRanges_count, cp);
}
static inline bool is_space(uint32_t cp) {
  if (cp < 128) return (cp >= 9 && cp <= 13) || cp == 32;
  return in_ranges(kSpaceRanges, kSpaceRanges_count, cp);
}

// Decode one UTF-8 code point at s[i]; invalid bytes decode as themselves (length 1) so that the
// scanner always advances and every byte ends up in some piece.
static inline uint32_t decode(const unsigned char* s, int64_t n, int64_t i, int* len) {
  unsigned char c = s[i];
  if (c < 0x80) { *len = 1; return c; }
  int need = (c >= 0xF0 && c < 0xF8) ? 3 : (c >= 0xE0) ? 2 : (c >= 0xC0) ? 1 : -1;
  if (need < 0 || i + need >= n) { *len = 1; return 0xFFFD0000u | c; }
  uint32_t cp = (need == 3) ? (c & 0x07) : (need == 2) ? (c & 0x0F) : (c & 0x1F);
  for (int k = 1; k <= need; ++k) {
    unsigned char cc = s[i + k];
    if ((cc & 0xC0) != 0x80) { *len = 1; return 0xFFFD0000u | c; }
    cp = (cp << 6) | (cc & 0x3F);
  }
  *len = need + 1;
  return cp;
}

struct Tokenizer {
  std::unordered_map<std::string, int32_t> ranks;
  std::vector<std::string> vocab;          // id -> bytes
  std::vector<std::pair<std::string, int32_t>> specials;
  std::string pattern;
  int32_t bos = -1;
  int32_t n_vocab = 0;

  // ---- pre-tokenisation: returns the end offset of the piece that starts at i ----
  int64_t next_piece(const unsigned char* s, int64_t n, int64_t i) const {
    int l0;
    const uint32_t c0 = decode(s, n, i, &l0);
    // 1. '(?i:[sdmt]|ll|ve|re)
    if (c0 == '\'' && i + 1 < n) {
      unsigned char a = s[i + 1] | 0x20;
      if (s[i + 1] < 0x80 && (a == 's' || a == 'd' || a == 'm' || a == 't')) return i + 2;
      if (i + 2 < n && s[i + 1] < 0x80 && s[i + 2] < 0x80) {
        unsigned char b = s[i + 2] | 0x20;
        if ((a == 'l' && b == 'l') || (a == 'v' && b == 'e') || (a == 'r' && b == 'e')) return i + 3;
      }
    }
    // 2. [^\r\n\p{L}\p{N}]?+\p{L}+
    {
      int64_t j = i;
      if (c0 != '\r' && c0 != '\n' && !is_letter(c0) && !is_number(c0)) j = i + l0;
      int64_t k = j;
      while (k < n) {
        int l;
        uint32_t c = decode(s, n, k, &l);
        if (!is_letter(c)) break;
        k += l;
      }
      if (k > j) return k;
    }
    // 3. \p{N}{1,2}
    if (is_number(c0)) {
      int64_t k = i + l0;
      if (k < n) {
        int l;
        uint32_t c = decode(s, n, k, &l);
        if (is_number(c)) k += l;
      }
      return k;
    }
    // 4.  ?[^\s\p{L}\p{N}]++[\r\n]*
    {
      int64_t j = i;
      if (c0 == ' ') j = i + 1;
      for (int attempt = 0; attempt < 2; ++attempt) {
        int64_t k = j;
        while (k < n) {
          int l;
          uint32_t c = decode(s, n, k, &l);
          if (is_space(c) || is_letter(c) || is_number(c)) break;
          k += l;
        }
        if (k > j) {
          while (k < n && (s[k] == '\r' || s[k] == '\n')) ++k;
          return k;
        }
        if (j == i) break;   // no optional space was taken: nothing to back off
        j = i;               // retry without the space (a space never matches the class, so this fails)
      }
    }
    // whitespace run starting at i
    if (is_space(c0)) {
      int64_t e = i;
      int64_t last_nl_end = -1;
      int64_t prev_start = i;
      while (e < n) {
        int l;
        uint32_t c = decode(s, n, e, &l);
        if (!is_space(c)) break;
        prev_start = e;
        e += l;
        if (c == '\r' || c == '\n') last_nl_end = e;
      }
      // 5. \s*[\r\n]
      if (last_nl_end >= 0) return last_nl_end;
      // 6. \s+(?!\S)
      if (e == n) return e;
      if (prev_start > i) return prev_start;
      // 7. \s+
      return e;
    }
    // unreachable for valid input; never stall
    return i + l0;
  }

  void bpe(const unsigned char* p, int64_t len, std::vector<int32_t>& out) const {
    if (len == 0) return;
    {
      auto it = ranks.find(std::string(reinterpret_cast<const char*>(p), size_t(len)));
      if (it != ranks.end()) { out.push_back(it->second); return; }
    }
    // boundaries of the current parts; rank[i] = rank of merging parts i and i+1
    std::vector<int32_t> start(size_t(len) + 1);
    for (int64_t i = 0; i <= len; ++i) start[size_t(i)] = int32_t(i);
    auto pair_rank = [&](size_t i) -> int32_t {   // parts i, i+1 -> bytes [start[i], start[i+2])
      if (i + 2 >= start.size()) return INT32_MAX;
      auto it = ranks.find(std::string(reinterpret_cast<const char*>(p) + start[i], size_t(start[i + 2] - start[i])));
      return it == ranks.end() ? INT32_MAX : it->second;
    };
    std::vector<int32_t> rk(start.size(), INT32_MAX);
    for (size_t i = 0; i + 2 < start.size(); ++i) rk[i] = pair_rank(i);
    for (;;) {
      int32_t best = INT32_MAX;
      size_t bi = 0;
      for (size_t i = 0; i + 2 < start.size(); ++i)
        if (rk[i] < best) { best = rk[i]; bi = i; }
      if (best == INT32_MAX) break;
      start.erase(start.begin() + long(bi) + 1);
      rk.erase(rk.begin() + long(bi) + 1);
      rk[bi] = pair_rank(bi);
      if (bi > 0) rk[bi - 1] = pair_rank(bi - 1);
    }
    for (size_t i = 0; i + 1 < start.size(); ++i) {
      auto it = ranks.find(std::string(reinterpret_cast<const char*>(p) + start[i], size_t(start[i + 1] - start[i])));
      out.push_back(it == ranks.end() ? 0 : it->second);   // single bytes are always in the vocabulary
    }
  }

  void finish() {
    int32_t mx = -1;
    for (auto& kv : ranks) mx = std::max(mx, kv.second);
    for (auto& sp : specials) mx = std::max(mx, sp.second);
    n_vocab = mx + 1;
    vocab.assign(size_t(n_vocab), std::string());
    for (auto& kv : ranks) vocab[size_t(kv.second)] = kv.first;
    for (auto& sp : specials) {
      if (sp.first.find("reserved_0") != std::string::npos && bos < 0) bos = sp.second;
    }
  }
};

static int b64val(char c) {
  if (c >= 'A' && c <= 'Z') return c - 'A';
  if (c >= 'a' && c <= 'z') return c - 'a' + 26;
  if (c >= '0' && c <= '9') return c - '0' + 52;
  if (c == '+') return 62;
  if (c == '/') return 63;
  return -1;
}
static bool b64decode(const std::string& in, std::string& out) {
  out.clear();
  uint32_t acc = 0;
  int bits = 0;
  for (char c : in) {
    if (c == '=') break;
    int v = b64val(c);
    if (v < 0) return false;
    acc = (acc << 6) | uint32_t(v);
    bits += 6;
    if (bits >= 8) { bits -= 8; out.push_back(char((acc >> bits) & 0xFF)); }
  }
  return true;
}

// Minimal JSON reader for this file's fixed structure.
struct J {
  const char* p; const char* e; bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  bool peek(char c) { ws(); return p < e && *p == c; }
  std::string str() {
    ws(); std::string o;
    if (p >= e || *p != '"') { ok = false; return o; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        switch (*p) {
          case 'n': o += '\n'; break; case 't': o += '\t'; break; case 'r': o += '\r'; break;
          case 'b': o += '\b'; break; case 'f': o += '\f'; break;
          case 'u': {
            unsigned v = 0;
            for (int i = 0; i < 4 && p + 1 < e; ++i) { ++p; char h = *p; v = v * 16 + unsigned(h <= '9' ? h - '0' : (h | 0x20) - 'a' + 10); }
            if (v < 0x80) o += char(v);
            else if (v < 0x800) { o += char(0xC0 | (v >> 6)); o += char(0x80 | (v & 0x3F)); }
            else { o += char(0xE0 | (v >> 12)); o += char(0x80 | ((v >> 6) & 0x3F)); o += char(0x80 | (v & 0x3F)); }
            break;
          }
          default: o += *p;
        }
        ++p;
      } else o += *p++;
    }
    if (p >= e) { ok = false; return o; }
    ++p;
    return o;
  }
  long long num() { ws(); char* end = nullptr; long long v = std::strtoll(p, &end, 10); if (end == p) ok = false; p = end; return v; }
  void skip() {
    ws();
    if (p >= e) { ok = false; return; }
    if (*p == '"') { str(); return; }
    if (*p == '{' || *p == '[') {
      int depth = 0;
      while (p < e) {
        if (*p == '"') { str(); continue; }
        if (*p == '{' || *p == '[') ++depth;
        else if (*p == '}' || *p == ']') { --depth; if (depth == 0) { ++p; return; } }
        ++p;
      }
      ok = false; return;
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
  }
};

static bool read_file(const char* path, std::string& out) {
  std::ifstream f(path, std::ios::binary);
  if (!f) return false;
  std::ostringstream ss;
  ss << f.rdbuf();
  out = ss.str();
  return true;
}

}  // namespace arn

using namespace arn;

static void* fail(char* err, int32_t n, const char* msg) {
  if (err && n > 0) std::snprintf(err, size_t(n), "%s", msg);
  return nullptr;
}

extern "C" {

void* ar_tok_load_json(const char* path, char* err, int32_t errlen) {
  std::string data;
  if (!read_file(path, data)) return fail(err, errlen, "cannot read tokenizer.json");
  J j{data.data(), data.data() + data.size()};
  Tokenizer* t = new Tokenizer;
  if (!j.eat('{')) { delete t; return fail(err, errlen, "tokenizer.json is not a JSON object"); }
  while (j.ok && !j.peek('}')) {
    std::string key = j.str();
    if (!j.eat(':')) { j.ok = false; break; }
    if (key == "pattern") t->pattern = j.str();
    else if (key == "mergeable_ranks" || key == "special_tokens") {
      const bool special = key == "special_tokens";
      if (!j.eat('[')) { j.ok = false; break; }
      while (j.ok && !j.peek(']')) {
        if (!j.eat('[')) { j.ok = false; break; }
        std::string name = j.str();
        if (!j.eat(',')) { j.ok = false; break; }
        long long rank = j.num();
        if (!j.eat(']')) { j.ok = false; break; }
        if (special) t->specials.emplace_back(name, int32_t(rank));
        else {
          std::string bytes;
          if (!b64decode(name, bytes)) { j.ok = false; break; }
          t->ranks.emplace(std::move(bytes), int32_t(rank));
        }
        j.eat(',');
      }
      if (!j.eat(']')) j.ok = false;
    } else j.skip();
    j.eat(',');
  }
  if (!j.ok || t->ranks.empty()) { delete t; return fail(err, errlen, "malformed tokenizer.json"); }
  t->finish();
  if (t->bos < 0) { delete t; return fail(err, errlen, "no reserved_0 special token (BOS) in tokenizer.json"); }
  return t;
}

void* ar_tok_load_tiktoken(const char* tiktoken_path, const char* config_path, char* err, int32_t errlen) {
  std::string data, cfg;
  if (!read_file(tiktoken_path, data)) return fail(err, errlen, "cannot read tokenizer.tiktoken");
  if (!read_file(config_path, cfg)) return fail(err, errlen, "cannot read tokenizer_config.txt");
  Tokenizer* t = new Tokenizer;
  std::istringstream ls(data);
  std::string line;
  while (std::getline(ls, line)) {
    if (line.empty()) continue;
    size_t sp = line.find(' ');
    if (sp == std::string::npos) { delete t; return fail(err, errlen, "tokenizer.tiktoken: missing rank"); }
    std::string bytes;
    if (!b64decode(line.substr(0, sp), bytes)) { delete t; return fail(err, errlen, "tokenizer.tiktoken: invalid base64"); }
    t->ranks.emplace(std::move(bytes), int32_t(std::strtol(line.c_str() + sp + 1, nullptr, 10)));
  }
  std::istringstream cs(cfg);
  while (std::getline(cs, line)) {
    if (line.rfind("pat_str:", 0) == 0) t->pattern = line.substr(8);
    else if (line.rfind("bos_id:", 0) == 0) t->bos = int32_t(std::strtol(line.c_str() + 7, nullptr, 10));
    else if (line.rfind("special:", 0) == 0) {
      size_t sp = line.rfind(' ');
      if (sp != std::string::npos && sp > 8)
        t->specials.emplace_back(line.substr(8, sp - 8), int32_t(std::strtol(line.c_str() + sp + 1, nullptr, 10)));
    }
  }
  if (t->pattern.empty()) { delete t; return fail(err, errlen, "pat_str not found in tokenizer_config.txt"); }
  if (t->bos < 0) { delete t; return fail(err, errlen, "bos_id not found in tokenizer_config.txt"); }
  int32_t bos = t->bos;
  t->finish();
  t->bos = bos;
  if (t->n_vocab <= bos) t->n_vocab = bos + 1;
  return t;
}

int32_t ar_tok_vocab(void* t) { return static_cast<Tokenizer*>(t)->n_vocab; }
int32_t ar_tok_bos(void* t) { return static_cast<Tokenizer*>(t)->bos; }

int64_t ar_tok_split(void* tv, const char* text, int64_t len, int64_t* ends, int64_t cap) {
  Tokenizer* t = static_cast<Tokenizer*>(tv);
  const unsigned char* s = reinterpret_cast<const unsigned char*>(text);
  int64_t i = 0, n = 0;
  while (i < len) {
    int64_t e = t->next_piece(s, len, i);
    if (e <= i) e = i + 1;
    if (ends && n < cap) ends[n] = e;
    ++n;
    i = e;
  }
  return n;
}

int64_t ar_tok_encode(void* tv, const char* text, int64_t len, int add_bos, int32_t* out, int64_t cap) {
  Tokenizer* t = static_cast<Tokenizer*>(tv);
  const unsigned char* s = reinterpret_cast<const unsigned char*>(text);
  std::vector<int32_t> ids;
  if (add_bos) ids.push_back(t->bos);
  int64_t i = 0;
  while (i < len) {
    int64_t e = t->next_piece(s, len, i);
    if (e <= i) e = i + 1;
    t->bpe(s + i, e - i, ids);
    i = e;
  }
  if (out) {
    int64_t m = std::min<int64_t>(cap, int64_t(ids.size()));
    std::memcpy(out, ids.data(), size_t(m) * 4);
  }
  return int64_t(ids.size());
}

int64_t ar_tok_decode(void* tv, const int32_t* ids, int64_t n, char* out, int64_t cap) {
  Tokenizer* t = static_cast<Tokenizer*>(tv);
  std::string s;
  for (int64_t i = 0; i < n; ++i)
    if (ids[i] >= 0 && ids[i] < t->n_vocab) s += t->vocab[size_t(ids[i])];
  if (out) std::memcpy(out, s.data(), size_t(std::min<int64_t>(cap, int64_t(s.size()))));
  return int64_t(s.size());
}

void ar_tok_destroy(void* t) { delete static_cast<Tokenizer*>(t); }

}  // extern "C"
