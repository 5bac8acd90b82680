// Stand-alone data feeder: documents -> BPE tokens (+BOS) -> best-fit packed rows of SEQ+1
// little-endian u16 on stdout, the stream the trainer's --stream-input mode consumes.
//
// Pipeline and flags follow the reference feeder (brain/src/bin/feeder.rs:18-129,
// brain/feeder.py:303-425): --input DIR | --jsonl FILE|-  --tokenizer-dir DIR  --seq-len N
// --prefetch N (documents per tokenisation batch)  --workers N  --max-rows N  --no-bos.
// Documents come from JSONL (fields "text", or "messages"/"turns" lists with "content") or
// plain .txt files (one document per file).  Parquet shards and HTTP download are handled by
// the Python side-car (autoresearch_b200/data/feeder.py), which pipes JSONL into this binary.
// Progress goes to stderr every 10000 rows; a closed pipe ends the program quietly.
#include "ar_native.h"

#include <dirent.h>
#include <signal.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

namespace {

// --- tiny JSON extractor: pulls the document text out of one JSONL record ---
struct JP {
  const char* p; const char* e; bool ok = true;
  void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < e && *p == c) { ++p; return true; } return false; }
  bool peek(char c) { ws(); return p < e && *p == c; }
  void utf8(unsigned v, std::string& o) {
    if (v < 0x80) o += char(v);
    else if (v < 0x800) { o += char(0xC0 | (v >> 6)); o += char(0x80 | (v & 0x3F)); }
    else if (v < 0x10000) { o += char(0xE0 | (v >> 12)); o += char(0x80 | ((v >> 6) & 0x3F)); o += char(0x80 | (v & 0x3F)); }
    else { o += char(0xF0 | (v >> 18)); o += char(0x80 | ((v >> 12) & 0x3F)); o += char(0x80 | ((v >> 6) & 0x3F)); o += char(0x80 | (v & 0x3F)); }
  }
  unsigned hex4() {
    unsigned v = 0;
    for (int i = 0; i < 4 && p < e; ++i, ++p) { char h = *p; v = v * 16 + unsigned(h <= '9' ? h - '0' : (h | 0x20) - 'a' + 10); }
    return v;
  }
  std::string str() {
    ws(); std::string o;
    if (p >= e || *p != '"') { ok = false; return o; }
    ++p;
    while (p < e && *p != '"') {
      if (*p == '\\' && p + 1 < e) {
        ++p;
        char c = *p++;
        switch (c) {
          case 'n': o += '\n'; break; case 't': o += '\t'; break; case 'r': o += '\r'; break;
          case 'b': o += '\b'; break; case 'f': o += '\f'; break;
          case 'u': {
            unsigned v = hex4();
            if (v >= 0xD800 && v < 0xDC00 && p + 1 < e && p[0] == '\\' && p[1] == 'u') {
              p += 2;
              unsigned lo = hex4();
              v = 0x10000 + ((v - 0xD800) << 10) + (lo - 0xDC00);
            }
            utf8(v, o);
            break;
          }
          default: o += c;
        }
      } else o += *p++;
    }
    if (p >= e) { ok = false; return o; }
    ++p;
    return o;
  }
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
  // list of objects: concatenate their "content" strings with newlines
  std::string contents() {
    std::string out;
    if (!eat('[')) { skip(); return out; }
    while (ok && !peek(']')) {
      if (eat('{')) {
        while (ok && !peek('}')) {
          std::string k = str();
          if (!eat(':')) { ok = false; break; }
          if (k == "content" && peek('"')) { if (!out.empty()) out += '\n'; out += str(); }
          else skip();
          eat(',');
        }
        eat('}');
      } else skip();
      eat(',');
    }
    eat(']');
    return out;
  }
};

bool extract_text(const std::string& line, std::string& text) {
  JP j{line.data(), line.data() + line.size()};
  if (!j.eat('{')) return false;
  std::string alt;
  text.clear();
  while (j.ok && !j.peek('}')) {
    std::string k = j.str();
    if (!j.eat(':')) return false;
    if (k == "text" && j.peek('"')) text = j.str();
    else if (k == "messages" || k == "turns") alt = j.contents();
    else j.skip();
    j.eat(',');
  }
  if (text.empty()) text = alt;
  return j.ok && !text.empty();
}

volatile sig_atomic_t g_pipe_closed = 0;
void on_sigpipe(int) { g_pipe_closed = 1; }

bool write_all(const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n > 0) {
    ssize_t w = ::write(1, p, n);
    if (w < 0) { if (errno == EINTR) continue; return false; }
    p += w; n -= size_t(w);
  }
  return true;
}

}  // namespace

int main(int argc, char** argv) {
  std::string input_dir, jsonl, tok_dir;
  int seq_len = 2048, prefetch = 128, workers = int(std::max(1u, std::thread::hardware_concurrency()));
  long long max_rows = -1;
  bool add_bos = true;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto val = [&]() -> std::string { if (i + 1 >= argc) { std::fprintf(stderr, "%s expects a value\n", a.c_str()); std::exit(2); } return argv[++i]; };
    if (a == "--input") input_dir = val();
    else if (a == "--jsonl") jsonl = val();
    else if (a == "--tokenizer-dir") tok_dir = val();
    else if (a == "--seq-len") seq_len = std::atoi(val().c_str());
    else if (a == "--prefetch") prefetch = std::max(1, std::atoi(val().c_str()));
    else if (a == "--workers") workers = std::max(1, std::atoi(val().c_str()));
    else if (a == "--max-rows") max_rows = std::atoll(val().c_str());
    else if (a == "--no-bos") add_bos = false;
    else if (a == "--stream" || a == "--cache-dir") { if (a == "--cache-dir") val(); }
  }
  if (tok_dir.empty() || (input_dir.empty() && jsonl.empty())) {
    std::fprintf(stderr, "usage: feeder --tokenizer-dir DIR (--input DIR | --jsonl FILE|-) [--seq-len N] [--prefetch N] "
                         "[--workers N] [--max-rows N] [--no-bos]\n");
    return 2;
  }
  signal(SIGPIPE, on_sigpipe);
  char err[256] = {0};
  void* tok = ar_tok_load_json((tok_dir + "/tokenizer.json").c_str(), err, sizeof err);
  if (!tok) tok = ar_tok_load_tiktoken((tok_dir + "/tokenizer.tiktoken").c_str(), (tok_dir + "/tokenizer_config.txt").c_str(), err, sizeof err);
  if (!tok) { std::fprintf(stderr, "[feeder] cannot load tokenizer from %s: %s\n", tok_dir.c_str(), err); return 1; }
  if (ar_tok_vocab(tok) > 65536) { std::fprintf(stderr, "[feeder] vocabulary does not fit u16 rows\n"); return 1; }
  std::fprintf(stderr, "[feeder] tokenizer: %d ids, bos %d; rows of %d tokens\n", ar_tok_vocab(tok), ar_tok_bos(tok), seq_len + 1);

  // document sources
  std::vector<std::string> files;
  if (!jsonl.empty()) files.push_back(jsonl);
  else {
    DIR* d = opendir(input_dir.c_str());
    if (!d) { std::fprintf(stderr, "[feeder] cannot open %s\n", input_dir.c_str()); return 1; }
    while (dirent* e = readdir(d)) {
      std::string n = e->d_name;
      if (n.size() > 6 && n.substr(n.size() - 6) == ".jsonl") files.push_back(input_dir + "/" + n);
      else if (n.size() > 4 && n.substr(n.size() - 4) == ".txt") files.push_back(input_dir + "/" + n);
    }
    closedir(d);
    std::sort(files.begin(), files.end());
  }
  void* packer = ar_packer_create(seq_len + 1, 1000);
  std::vector<uint16_t> row(size_t(seq_len) + 1);
  long long rows = 0, docs = 0;
  double t_tok = 0, t_pack = 0, t_write = 0;
  auto now = [] { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); };
  bool stop = false;

  auto flush_rows = [&](int exhausted) {
    double t0 = now();
    while (!stop && ar_packer_next_row(packer, exhausted, row.data())) {
      double t1 = now();
      t_pack += t1 - t0;
      if (!write_all(row.data(), row.size() * 2) || g_pipe_closed) { stop = true; break; }
      t0 = now();
      t_write += t0 - t1;
      if (++rows % 10000 == 0)
        std::fprintf(stderr, "[feeder] rows=%lld docs=%lld tokenize=%.1fs pack=%.1fs write=%.1fs\n", rows, docs, t_tok, t_pack, t_write);
      if (max_rows >= 0 && rows >= max_rows) { stop = true; break; }
    }
  };
  auto process_batch = [&](std::vector<std::string>& batch) {
    if (batch.empty()) return;
    double t0 = now();
    std::vector<std::vector<int32_t>> out(batch.size());
    std::vector<std::thread> th;
    const int nw = std::min<int>(workers, int(batch.size()));
    for (int w = 0; w < nw; ++w)
      th.emplace_back([&, w] {
        for (size_t i = size_t(w); i < batch.size(); i += size_t(nw)) {
          const std::string& s = batch[i];
          int64_t n = ar_tok_encode(tok, s.data(), int64_t(s.size()), add_bos ? 1 : 0, nullptr, 0);
          out[i].resize(size_t(n));
          ar_tok_encode(tok, s.data(), int64_t(s.size()), add_bos ? 1 : 0, out[i].data(), n);
        }
      });
    for (auto& t : th) t.join();
    t_tok += now() - t0;
    for (auto& d : out) { ar_packer_add_doc(packer, d.data(), int32_t(d.size())); ++docs; }
    batch.clear();
    flush_rows(0);
  };

  std::vector<std::string> batch;
  for (const auto& f : files) {
    if (stop) break;
    const bool is_txt = f.size() > 4 && f.substr(f.size() - 4) == ".txt";
    std::istream* in = &std::cin;
    std::ifstream fs;
    if (f != "-") { fs.open(f, std::ios::binary); if (!fs) { std::fprintf(stderr, "[feeder] skipping unreadable %s\n", f.c_str()); continue; } in = &fs; }
    if (is_txt) {
      std::ostringstream ss; ss << in->rdbuf();
      batch.push_back(ss.str());
      if (int(batch.size()) >= prefetch) process_batch(batch);
      continue;
    }
    std::string line, text;
    while (!stop && std::getline(*in, line)) {
      if (line.empty()) continue;
      if (!extract_text(line, text)) continue;   // malformed records are skipped, like corrupt parquet rows
      batch.push_back(text);
      if (int(batch.size()) >= prefetch) process_batch(batch);
    }
  }
  if (!stop) process_batch(batch);
  if (!stop) flush_rows(1);
  std::fprintf(stderr, "[feeder] done: rows=%lld docs=%lld tokenize=%.1fs pack=%.1fs write=%.1fs\n", rows, docs, t_tok, t_pack, t_write);
  ar_packer_destroy(packer);
  ar_tok_destroy(tok);
  return 0;
}
