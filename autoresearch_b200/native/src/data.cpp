// TKNS shard files and the stdin row stream.
// Formats: brain/src/train.rs:247-271 (20-byte header "TKNS" | version=1 | vocab | seq_len
// | num_rows, then u16 rows) and brain/src/train.rs:348-409 (rows of SEQ+1 little-endian
// u16 on a pipe, read by a background thread into a bounded queue).
#include "ar_native.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstring>
#include <deque>
#include <mutex>
#include <thread>
#include <vector>

namespace {

struct Shard {
  void* map = nullptr;
  size_t len = 0;
  uint32_t vocab = 0, seq_len = 0, num_rows = 0;
};

inline uint32_t rd32(const uint8_t* p) {
  return uint32_t(p[0]) | uint32_t(p[1]) << 8 | uint32_t(p[2]) << 16 | uint32_t(p[3]) << 24;
}

struct RowStream {
  int fd;
  int32_t row_len, batch_rows, depth;
  std::thread th;
  std::mutex mu;
  std::condition_variable cv_data, cv_space;
  std::deque<std::vector<uint16_t>> q;
  bool eof = false, failed = false, stop = false;
  std::atomic<int64_t> rows{0};

  void run() {
    const size_t row_bytes = size_t(row_len) * 2;
    const size_t batch_bytes = row_bytes * size_t(batch_rows);
    for (;;) {
      std::vector<uint16_t> buf(static_cast<size_t>(row_len) * static_cast<size_t>(batch_rows), uint16_t(0));
      size_t got = 0;
      uint8_t* dst = reinterpret_cast<uint8_t*>(buf.data());
      while (got < batch_bytes) {
        ssize_t r = ::read(fd, dst + got, batch_bytes - got);
        if (r < 0) {
          if (errno == EINTR) continue;
          std::lock_guard<std::mutex> l(mu);
          failed = true;
          eof = true;
          cv_data.notify_all();
          return;
        }
        if (r == 0) break;
        got += size_t(r);
        {
          std::lock_guard<std::mutex> l(mu);
          if (stop) return;
        }
      }
      if (got < batch_bytes) {
        std::lock_guard<std::mutex> l(mu);
        // A partial batch is dropped; a stream that stops inside a row is an error.
        if (got % row_bytes != 0) failed = true;
        eof = true;
        cv_data.notify_all();
        return;
      }
      rows += batch_rows;
      std::unique_lock<std::mutex> l(mu);
      cv_space.wait(l, [&] { return stop || int32_t(q.size()) < depth; });
      if (stop) return;
      q.emplace_back(std::move(buf));
      cv_data.notify_one();
    }
  }
};

}  // namespace

extern "C" {

int ar_shard_open(const char* path, void** handle, uint32_t* vocab, uint32_t* seq_len,
                  uint32_t* num_rows) {
  *handle = nullptr;
  int fd = ::open(path, O_RDONLY);
  if (fd < 0) return -1;
  struct stat st;
  if (fstat(fd, &st) != 0) { ::close(fd); return -1; }
  size_t len = size_t(st.st_size);
  if (len < 20) { ::close(fd); return -2; }
  void* m = mmap(nullptr, len, PROT_READ, MAP_PRIVATE, fd, 0);
  ::close(fd);
  if (m == MAP_FAILED) return -1;
  const uint8_t* p = static_cast<const uint8_t*>(m);
  if (std::memcmp(p, "TKNS", 4) != 0) { munmap(m, len); return -3; }
  if (rd32(p + 4) != 1) { munmap(m, len); return -4; }
  Shard* s = new Shard;
  s->map = m;
  s->len = len;
  s->vocab = rd32(p + 8);
  s->seq_len = rd32(p + 12);
  s->num_rows = rd32(p + 16);
  size_t expect = 20 + size_t(s->num_rows) * size_t(s->seq_len) * 2;
  if (len < expect) { munmap(m, len); delete s; return -5; }
  *vocab = s->vocab; *seq_len = s->seq_len; *num_rows = s->num_rows;
  *handle = s;
  return 0;
}

const uint16_t* ar_shard_row(void* handle, uint32_t idx) {
  Shard* s = static_cast<Shard*>(handle);
  if (idx >= s->num_rows) return nullptr;
  const uint8_t* p = static_cast<const uint8_t*>(s->map) + 20 + size_t(idx) * s->seq_len * 2;
  return reinterpret_cast<const uint16_t*>(p);
}

void ar_shard_close(void* handle) {
  Shard* s = static_cast<Shard*>(handle);
  if (!s) return;
  munmap(s->map, s->len);
  delete s;
}

int ar_shard_write(const char* path, uint32_t vocab, uint32_t seq_len, uint32_t num_rows,
                   const uint16_t* rows) {
  FILE* f = std::fopen(path, "wb");
  if (!f) return -1;
  uint32_t hdr[4] = {1u, vocab, seq_len, num_rows};
  bool ok = std::fwrite("TKNS", 1, 4, f) == 4 && std::fwrite(hdr, 4, 4, f) == 4;
  size_t n = size_t(seq_len) * num_rows;
  ok = ok && std::fwrite(rows, 2, n, f) == n;
  ok = (std::fclose(f) == 0) && ok;
  return ok ? 0 : -1;
}

void* ar_rowstream_open(int fd, int32_t row_len, int32_t batch_rows, int32_t depth) {
  if (row_len < 2 || batch_rows < 1 || depth < 1) return nullptr;
  RowStream* r = new RowStream;
  r->fd = fd; r->row_len = row_len; r->batch_rows = batch_rows; r->depth = depth;
  r->th = std::thread([r] { r->run(); });
  return r;
}

int ar_rowstream_next(void* h, int32_t* ids, int32_t* targets, int32_t timeout_ms) {
  RowStream* r = static_cast<RowStream*>(h);
  std::vector<uint16_t> buf;
  {
    std::unique_lock<std::mutex> l(r->mu);
    auto ready = [&] { return !r->q.empty() || r->eof; };
    if (timeout_ms < 0) {
      r->cv_data.wait(l, ready);
    } else if (!r->cv_data.wait_for(l, std::chrono::milliseconds(timeout_ms), ready)) {
      return -2;
    }
    if (r->q.empty()) return r->failed ? -1 : 0;
    buf = std::move(r->q.front());
    r->q.pop_front();
    r->cv_space.notify_one();
  }
  const int32_t T = r->row_len - 1;
  for (int32_t b = 0; b < r->batch_rows; ++b) {
    const uint16_t* row = buf.data() + size_t(b) * r->row_len;
    int32_t* di = ids + size_t(b) * T;
    int32_t* dt = targets + size_t(b) * T;
    for (int32_t t = 0; t < T; ++t) { di[t] = row[t]; dt[t] = row[t + 1]; }
  }
  return 1;
}

int64_t ar_rowstream_rows_read(void* h) { return static_cast<RowStream*>(h)->rows.load(); }

void ar_rowstream_close(void* h) {
  RowStream* r = static_cast<RowStream*>(h);
  if (!r) return;
  {
    std::lock_guard<std::mutex> l(r->mu);
    r->stop = true;
    r->cv_space.notify_all();
  }
  // The reader may be blocked in read(); closing our end of the descriptor unblocks a
  // pipe whose writer is gone, otherwise detach and let process exit reap it.
  if (r->th.joinable()) {
    bool done;
    {
      std::lock_guard<std::mutex> l(r->mu);
      done = r->eof;
    }
    if (done) { r->th.join(); delete r; }
    else { r->th.detach(); /* leaked on purpose: thread still references *r */ }
  }
}

}  // extern "C"
