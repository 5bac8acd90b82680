// Byte-pair-encoding trainer over pre-split words with counts (role of the one-time vocabulary
// training in original/prepare.py:88-140, which calls the rustbpe crate).  Classic algorithm with
// incremental pair statistics: the most frequent adjacent pair (ties: the smaller pair of ids) is
// merged into a new id until `vocab_size` ids exist; ids 0..255 are the bytes.
#include "ar_native.h"

#include <algorithm>
#include <cstring>
#include <queue>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

using Pair = std::pair<int32_t, int32_t>;
struct PairHash {
  size_t operator()(const Pair& p) const { return (uint64_t(uint32_t(p.first)) << 32 | uint32_t(p.second)) * 0x9E3779B97F4A7C15ull >> 7; }
};
struct Word {
  std::vector<int32_t> ids;
  int64_t count;
};
struct HeapItem {
  int64_t count;
  Pair pair;
  bool operator<(const HeapItem& o) const {   // max-heap on count, then smaller pair first
    if (count != o.count) return count < o.count;
    return pair > o.pair;
  }
};

}  // namespace

extern "C" int32_t ar_bpe_train(const uint8_t* bytes, const int64_t* offsets, const int64_t* counts, int64_t n_words,
                                int32_t vocab_size, int32_t* merges_out) {
  if (n_words < 0 || vocab_size < 256) return -1;
  std::vector<Word> words(static_cast<size_t>(n_words));
  for (int64_t w = 0; w < n_words; ++w) {
    const int64_t a = offsets[w], b = offsets[w + 1];
    words[w].ids.assign(bytes + a, bytes + b);
    words[w].count = counts[w];
  }
  std::unordered_map<Pair, int64_t, PairHash> stat;
  std::unordered_map<Pair, std::unordered_set<int64_t>, PairHash> where;
  for (int64_t w = 0; w < n_words; ++w) {
    const auto& v = words[w].ids;
    for (size_t i = 0; i + 1 < v.size(); ++i) {
      const Pair p{v[i], v[i + 1]};
      stat[p] += words[w].count;
      where[p].insert(w);
    }
  }
  std::priority_queue<HeapItem> heap;
  for (const auto& kv : stat) heap.push({kv.second, kv.first});
  int32_t n_merges = 0;
  for (int32_t new_id = 256; new_id < vocab_size; ++new_id) {
    Pair best{-1, -1};
    while (!heap.empty()) {                       // lazy deletion: skip entries whose count is stale
      const HeapItem top = heap.top();
      heap.pop();
      auto it = stat.find(top.pair);
      if (it != stat.end() && it->second == top.count && top.count > 0) { best = top.pair; break; }
    }
    if (best.first < 0) break;
    merges_out[2 * n_merges] = best.first;
    merges_out[2 * n_merges + 1] = best.second;
    ++n_merges;
    // Every word that may contain the pair: subtract its old pairs from the statistics, merge, add its new
    // pairs.  `where` may hold stale entries (words that lost the pair earlier); they merge nothing.
    std::unordered_set<Pair, PairHash> touched;
    const std::vector<int64_t> ws(where[best].begin(), where[best].end());
    for (int64_t w : ws) {
      auto& v = words[w].ids;
      const int64_t c = words[w].count;
      std::vector<int32_t> out;
      out.reserve(v.size());
      bool merged = false;
      for (size_t i = 0; i < v.size();) {
        if (i + 1 < v.size() && v[i] == best.first && v[i + 1] == best.second) {
          out.push_back(new_id);
          i += 2;
          merged = true;
        } else {
          out.push_back(v[i]);
          ++i;
        }
      }
      if (!merged) continue;
      for (size_t i = 0; i + 1 < v.size(); ++i) { const Pair p{v[i], v[i + 1]}; stat[p] -= c; touched.insert(p); }
      for (size_t i = 0; i + 1 < out.size(); ++i) {
        const Pair p{out[i], out[i + 1]};
        stat[p] += c;
        touched.insert(p);
        where[p].insert(w);
      }
      v.swap(out);
    }
    stat.erase(best);
    where.erase(best);
    for (const Pair& p : touched) {
      if (p == best) continue;
      auto it = stat.find(p);
      if (it == stat.end()) continue;
      if (it->second > 0) heap.push({it->second, p});
      else stat.erase(it);
    }
  }
  return n_merges;
}
