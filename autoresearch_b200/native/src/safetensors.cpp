// Minimal safetensors reader / writer.
// File = u64 little-endian header length | JSON header | raw tensor bytes.  The reference
// writes BF16 tensors with sorted names and no metadata through the safetensors crate
// (brain/src/train.rs:2733-2743); this writer produces the same layout: entries ordered
// by name, compact JSON, header padded with spaces to a multiple of 8 bytes.
#include "ar_native.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

struct Entry {
  std::string name, dtype;
  std::vector<int64_t> shape;
  const void* data = nullptr;
  int64_t nbytes = 0;
  int64_t begin = 0, end = 0;
};

struct Writer { std::vector<Entry> entries; };

struct Reader {
  void* map = nullptr;
  size_t len = 0;
  const uint8_t* data_base = nullptr;
  std::vector<Entry> entries;
};

std::string json_escape(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') { o += '\\'; o += c; }
    else if (static_cast<unsigned char>(c) < 0x20) {
      char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o += b;
    } else o += c;
  }
  return o;
}

// ---- tiny JSON scanner sufficient for safetensors headers ----
struct Scan {
  const char* p; const char* e; bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
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
            for (int i = 0; i < 4 && p + 1 < e; ++i) { ++p; v = v * 16 + unsigned(std::strtol(std::string(1, *p).c_str(), nullptr, 16)); }
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
  int64_t num() {
    ws(); char* end = nullptr;
    long long v = std::strtoll(p, &end, 10);
    if (end == p) ok = false;
    p = end; return v;
  }
  void skip_value() {
    ws();
    if (p >= e) { ok = false; return; }
    if (*p == '"') { str(); return; }
    if (*p == '{' || *p == '[') {
      char open = *p, close = (open == '{') ? '}' : ']';
      int depth = 0;
      while (p < e) {
        if (*p == '"') { str(); continue; }
        if (*p == open) ++depth;
        else if (*p == close) { --depth; if (depth == 0) { ++p; return; } }
        ++p;
      }
      ok = false; return;
    }
    while (p < e && *p != ',' && *p != '}' && *p != ']') ++p;
  }
};

}  // namespace

extern "C" {

void* ar_st_writer_create(void) { return new Writer; }

void ar_st_writer_add(void* w, const char* name, const char* dtype, const int64_t* shape,
                      int32_t ndim, const void* data, int64_t nbytes) {
  Entry e;
  e.name = name; e.dtype = dtype;
  e.shape.assign(shape, shape + ndim);
  e.data = data; e.nbytes = nbytes;
  static_cast<Writer*>(w)->entries.push_back(std::move(e));
}

int ar_st_writer_finish(void* wv, const char* path) {
  Writer* w = static_cast<Writer*>(wv);
  std::sort(w->entries.begin(), w->entries.end(),
            [](const Entry& a, const Entry& b) { return a.name < b.name; });
  std::string hdr = "{";
  int64_t off = 0;
  bool first = true;
  for (auto& e : w->entries) {
    if (!first) hdr += ",";
    first = false;
    hdr += "\"" + json_escape(e.name) + "\":{\"dtype\":\"" + e.dtype + "\",\"shape\":[";
    for (size_t i = 0; i < e.shape.size(); ++i) {
      if (i) hdr += ",";
      hdr += std::to_string(e.shape[i]);
    }
    hdr += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + e.nbytes) + "]}";
    off += e.nbytes;
  }
  hdr += "}";
  while (hdr.size() % 8) hdr += ' ';
  std::string tmp = std::string(path) + ".tmp";
  FILE* f = std::fopen(tmp.c_str(), "wb");
  int rc = 0;
  if (!f) { delete w; return -1; }
  uint64_t n = hdr.size();
  if (std::fwrite(&n, 8, 1, f) != 1) rc = -1;
  if (std::fwrite(hdr.data(), 1, hdr.size(), f) != hdr.size()) rc = -1;
  for (auto& e : w->entries)
    if (e.nbytes && std::fwrite(e.data, 1, size_t(e.nbytes), f) != size_t(e.nbytes)) rc = -1;
  if (std::fclose(f) != 0) rc = -1;
  if (rc == 0 && std::rename(tmp.c_str(), path) != 0) rc = -1;
  delete w;
  return rc;
}

void* ar_st_open(const char* path, char* err, int32_t errlen) {
  auto fail = [&](const char* m) -> void* { if (err && errlen > 0) std::snprintf(err, size_t(errlen), "%s", m); return nullptr; };
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return fail("cannot open file");
  struct stat st;
  if (fstat(fd, &st) != 0) { ::close(fd); return fail("cannot stat file"); }
  size_t len = size_t(st.st_size);
  if (len < 8) { ::close(fd); return fail("file shorter than the 8-byte header length"); }
  void* m = mmap(nullptr, len, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (m == MAP_FAILED) return fail("mmap failed");
  uint64_t n;
  std::memcpy(&n, m, 8);
  if (n > len - 8) { munmap(m, len); return fail("header length exceeds file size"); }
  Reader* r = new Reader;
  r->map = m; r->len = len;
  r->data_base = static_cast<const uint8_t*>(m) + 8 + n;
  const size_t data_len = len - 8 - size_t(n);
  Scan s{static_cast<const char*>(m) + 8, static_cast<const char*>(m) + 8 + n};
  if (!s.eat('{')) { munmap(m, len); delete r; return fail("header is not a JSON object"); }
  if (!s.eat('}')) {
    for (;;) {
      std::string key = s.str();
      if (!s.ok || !s.eat(':')) break;
      if (key == "__metadata__") { s.skip_value(); }
      else {
        Entry e; e.name = key;
        if (!s.eat('{')) { s.ok = false; break; }
        for (;;) {
          std::string k = s.str();
          if (!s.ok || !s.eat(':')) { s.ok = false; break; }
          if (k == "dtype") e.dtype = s.str();
          else if (k == "shape") {
            if (!s.eat('[')) { s.ok = false; break; }
            if (!s.eat(']')) { for (;;) { e.shape.push_back(s.num()); if (s.eat(']')) break; if (!s.eat(',')) { s.ok = false; break; } } }
          } else if (k == "data_offsets") {
            if (!s.eat('[')) { s.ok = false; break; }
            e.begin = s.num(); if (!s.eat(',')) { s.ok = false; break; }
            e.end = s.num(); if (!s.eat(']')) { s.ok = false; break; }
          } else s.skip_value();
          if (!s.ok) break;
          if (s.eat('}')) break;
          if (!s.eat(',')) { s.ok = false; break; }
        }
        if (!s.ok) break;
        if (e.begin < 0 || e.end < e.begin || size_t(e.end) > data_len) { munmap(m, len); delete r; return fail("tensor data offsets outside the file"); }
        e.nbytes = e.end - e.begin;
        e.data = r->data_base + e.begin;
        r->entries.push_back(std::move(e));
      }
      if (s.eat('}')) break;
      if (!s.eat(',')) { s.ok = false; break; }
    }
  }
  if (!s.ok) { munmap(m, len); delete r; return fail("malformed JSON header"); }
  return r;
}

int32_t ar_st_count(void* r) { return int32_t(static_cast<Reader*>(r)->entries.size()); }
const char* ar_st_name(void* r, int32_t i) { return static_cast<Reader*>(r)->entries[size_t(i)].name.c_str(); }
const char* ar_st_dtype(void* r, int32_t i) { return static_cast<Reader*>(r)->entries[size_t(i)].dtype.c_str(); }
int32_t ar_st_ndim(void* r, int32_t i) { return int32_t(static_cast<Reader*>(r)->entries[size_t(i)].shape.size()); }
int64_t ar_st_dim(void* r, int32_t i, int32_t d) { return static_cast<Reader*>(r)->entries[size_t(i)].shape[size_t(d)]; }
const void* ar_st_data(void* r, int32_t i, int64_t* nbytes) {
  auto& e = static_cast<Reader*>(r)->entries[size_t(i)];
  *nbytes = e.nbytes;
  return e.data;
}
void ar_st_close(void* rv) {
  Reader* r = static_cast<Reader*>(rv);
  if (!r) return;
  munmap(r->map, r->len);
  delete r;
}

}  // extern "C"
