// Host RNG used for weight initialisation and synthetic token streams.
// Math spec: xorshift64 (13, 7, 17) seeded 42, Box-Muller normals, uniform(-b, b)
// (brain/src/train.rs:2424-2483); LCG token stream (brain/src/train.rs:419-430).
#include "ar_native.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <vector>

namespace {

inline uint64_t xs64(uint64_t& s) {
  s ^= s << 13;
  s ^= s >> 7;
  s ^= s << 17;
  return s;
}

inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return uint16_t((u >> 16) | 0x40);  // NaN
  uint32_t r = 0x7fffu + ((u >> 16) & 1u);
  return uint16_t((u + r) >> 16);
}

// u64 -> f32 in the way a `as f32` conversion rounds (round-to-nearest-even), divided by
// u64::MAX as f32 (= 2^64).
inline float u64_unit_f32(uint64_t v) { return float(v) / 18446744073709551616.0f; }
inline double u64_unit_f64(uint64_t v) { return double(v) / 18446744073709551616.0; }

struct Zipf {
  std::vector<double> cdf;
  uint64_t state;
  uint32_t vocab;
};

inline uint64_t splitmix(uint64_t& s) {
  uint64_t z = (s += 0x9e3779b97f4a7c15ull);
  z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
  z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
  return z ^ (z >> 31);
}

}  // namespace

extern "C" {

void ar_uniform_bf16(uint64_t* state, int64_t n, double bound, uint16_t* out) {
  uint64_t s = *state;
  for (int64_t i = 0; i < n; ++i) {
    double u = u64_unit_f64(xs64(s));
    out[i] = f32_to_bf16(float(2.0 * bound * u - bound));
  }
  *state = s;
}

void ar_uniform_f32(uint64_t* state, int64_t n, double bound, float* out) {
  uint64_t s = *state;
  for (int64_t i = 0; i < n; ++i) {
    double u = u64_unit_f64(xs64(s));
    out[i] = float(2.0 * bound * u - bound);
  }
  *state = s;
}

void ar_randn_f32(uint64_t* state, int64_t n, float scale, float* out) {
  uint64_t s = *state;
  const float two_pi = 2.0f * 3.14159265358979323846f;
  int64_t pairs = (n + 1) / 2;
  for (int64_t p = 0; p < pairs; ++p) {
    float u1 = std::max(u64_unit_f32(xs64(s)), std::numeric_limits<float>::min());
    float u2 = u64_unit_f32(xs64(s));
    float r = std::sqrt(-2.0f * std::log(u1));
    float a = r * std::cos(two_pi * u2), b = r * std::sin(two_pi * u2);
    out[2 * p] = a * scale;
    if (2 * p + 1 < n) out[2 * p + 1] = b * scale;
  }
  *state = s;
}

void ar_randn_bf16(uint64_t* state, int64_t n, float scale, uint16_t* out) {
  std::vector<float> tmp(static_cast<size_t>(std::min<int64_t>(n, 1 << 20)), 0.0f);
  int64_t done = 0;
  // Box-Muller consumes two draws per pair; chunk on even boundaries to keep the stream
  // identical to a single call.
  while (done < n) {
    int64_t c = std::min<int64_t>(n - done, int64_t(tmp.size()) & ~int64_t(1));
    if (c == 0) c = n - done;
    ar_randn_f32(state, c, scale, tmp.data());
    for (int64_t i = 0; i < c; ++i) out[done + i] = f32_to_bf16(tmp[size_t(i)]);
    done += c;
  }
}

void ar_shuffle_order(int64_t* order, int64_t n, uint64_t seed) {
  for (int64_t i = 0; i < n; ++i) order[i] = i;
  if (n <= 1) return;
  uint64_t s = seed;
  for (int64_t i = n - 1; i >= 1; --i) {
    int64_t j = int64_t(xs64(s) % uint64_t(i + 1));
    std::swap(order[i], order[j]);
  }
}

void ar_lcg_tokens(uint64_t* state, int64_t n, uint32_t vocab, int32_t* out) {
  uint64_t s = *state;
  for (int64_t i = 0; i < n; ++i) {
    s = s * 6364136223846793005ull + 1442695040888963407ull;
    out[i] = int32_t(uint32_t(s >> 33) % (vocab - 1)) + 1;
  }
  *state = s;
}

void* ar_zipf_create(uint32_t vocab, double sexp, uint64_t seed) {
  Zipf* z = new Zipf;
  z->vocab = vocab;
  z->state = seed;
  z->cdf.resize(vocab);
  double acc = 0;
  for (uint32_t k = 0; k < vocab; ++k) {
    acc += std::pow(double(k + 1), -sexp);
    z->cdf[k] = acc;
  }
  for (auto& c : z->cdf) c /= acc;
  z->cdf[vocab - 1] = 1.0;
  return z;
}

void ar_zipf_seek(void* h, uint64_t seed, uint64_t draws) {
  Zipf* z = static_cast<Zipf*>(h);
  z->state = seed + draws * 0x9e3779b97f4a7c15ull;  // splitmix64 is counter based
}

void ar_zipf_fill(void* h, int64_t n, int32_t* out) {
  Zipf* z = static_cast<Zipf*>(h);
  for (int64_t i = 0; i < n; ++i) {
    double u = double(splitmix(z->state) >> 11) * (1.0 / 9007199254740992.0);
    auto it = std::lower_bound(z->cdf.begin(), z->cdf.end(), u);
    size_t k = size_t(it - z->cdf.begin());
    if (k >= z->vocab) k = z->vocab - 1;
    out[i] = int32_t(k);
  }
}

void ar_zipf_destroy(void* h) { delete static_cast<Zipf*>(h); }

}  // extern "C"
