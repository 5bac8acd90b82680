// Best-fit document packer.
// Behaviour (brain/src/feeder/packing.rs:13-108, brain/feeder.py pack_rows): keep a buffer
// of at least `buffer_docs` tokenised documents; for each output row repeatedly take the
// LARGEST buffered document that fits the remaining space; if none fits take the SHORTEST
// one and crop it to the remaining space (its tail is discarded); zero-pad only when the
// source is exhausted in the middle of a row.
#include "ar_native.h"

#include <algorithm>
#include <cstring>
#include <vector>

namespace {
struct Packer {
  int32_t cap, buffer_docs;
  std::vector<std::vector<uint16_t>> docs;
  std::vector<uint16_t> row;
  int32_t pos = 0;
};
}  // namespace

extern "C" {

void* ar_packer_create(int32_t row_capacity, int32_t buffer_docs) {
  if (row_capacity < 1) return nullptr;
  Packer* p = new Packer;
  p->cap = row_capacity;
  p->buffer_docs = buffer_docs;
  p->row.assign(size_t(row_capacity), 0);
  return p;
}

void ar_packer_add_doc(void* h, const int32_t* tokens, int32_t n) {
  Packer* p = static_cast<Packer*>(h);
  if (n <= 0) return;  // an empty document can never advance a row
  std::vector<uint16_t> d(static_cast<size_t>(n), uint16_t(0));
  for (int32_t i = 0; i < n; ++i) d[size_t(i)] = uint16_t(tokens[i]);
  p->docs.emplace_back(std::move(d));
}

int32_t ar_packer_buffered(void* h) { return int32_t(static_cast<Packer*>(h)->docs.size()); }

int ar_packer_next_row(void* h, int exhausted, uint16_t* out_row) {
  Packer* p = static_cast<Packer*>(h);
  while (p->pos < p->cap) {
    if (!exhausted && int32_t(p->docs.size()) < p->buffer_docs) return 0;  // refill first
    if (p->docs.empty()) {
      if (p->pos > 0) break;  // pad the tail with zeros
      return 0;
    }
    const int32_t remaining = p->cap - p->pos;
    int64_t best = -1, shortest = 0;
    size_t best_len = 0;
    for (size_t i = 0; i < p->docs.size(); ++i) {
      size_t L = p->docs[i].size();
      if (L <= size_t(remaining) && L > best_len) { best = int64_t(i); best_len = L; }
      if (L < p->docs[size_t(shortest)].size()) shortest = int64_t(i);
    }
    if (best >= 0) {
      auto& d = p->docs[size_t(best)];
      std::memcpy(p->row.data() + p->pos, d.data(), d.size() * 2);
      p->pos += int32_t(d.size());
      p->docs.erase(p->docs.begin() + best);
    } else {
      auto& d = p->docs[size_t(shortest)];
      std::memcpy(p->row.data() + p->pos, d.data(), size_t(remaining) * 2);
      p->pos += remaining;
      p->docs.erase(p->docs.begin() + shortest);
    }
  }
  std::memcpy(out_row, p->row.data(), size_t(p->cap) * 2);
  std::fill(p->row.begin(), p->row.end(), uint16_t(0));
  p->pos = 0;
  return 1;
}

void ar_packer_destroy(void* h) { delete static_cast<Packer*>(h); }

}  // extern "C"
