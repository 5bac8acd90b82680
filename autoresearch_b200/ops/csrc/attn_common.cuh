// Shared pieces of the attention kernels (attn_sm100.cu, attn_wide_sm100.cu).
#pragma once
#include "api.h"
#include "ptx.cuh"
#include "tmap.h"

namespace arb {

constexpr int HD = 128;
constexpr int ATT_THREADS = 192;        // producer warp, MMA warp, 4 softmax warps
constexpr int ATT_WIDE_THREADS = 320;   // producer warp, MMA warp, 8 softmax warps
constexpr float LOG2E = 1.4426950408889634f;

struct AttnArgs {
  int B, T, H, window;
  float scale;
  // forward / dq
  void* o; long long ldo;            // forward: O [B,T,H,128] bf16 ; dq kernel: dQ
  float* lse;                        // [B,H,T]
  const float* delta;                // [B,H,T] (backward)
  // dkv
  void* dk; void* dv; long long lddk, lddv;
  int* err;
};

// Optional per-role cycle accounting (compile with -DARB_ATTN_PROF): each role of the CTA with
// blockIdx == (0,0,0) sums clock64() deltas between PROF_TOC marks and stores eight counters at
// arb_attn_prof_buffer[role * 8 ..]; counter 0 is the role's total.  Compiled out by default.
#ifdef ARB_ATTN_PROF
__device__ long long* arb_attn_prof_buffer;
#define PROF_DECL() long long prof_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long prof_t0 = clock64(); const long long prof_begin = prof_t0
#define PROF_TIC() prof_t0 = clock64()
#define PROF_TOC(i) do { const long long prof_t1 = clock64(); prof_acc[i] += prof_t1 - prof_t0; prof_t0 = prof_t1; } while (0)
#define PROF_DUMP(role)                                                                                   \
  do {                                                                                                    \
    prof_acc[0] = clock64() - prof_begin;                                                                 \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && arb_attn_prof_buffer)                    \
      for (int prof_i = 0; prof_i < 8; ++prof_i) arb_attn_prof_buffer[(role) * 8 + prof_i] = prof_acc[prof_i]; \
  } while (0)
#else
#define PROF_DECL() do { } while (0)
#define PROF_TIC() do { } while (0)
#define PROF_TOC(i) do { } while (0)
#define PROF_DUMP(role) do { } while (0)
#endif

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#ifndef ARB_FWD2_POLY
#define ARB_FWD2_POLY 0
#endif
#ifndef ARB_FWD_POLY_OF_8
#define ARB_FWD_POLY_OF_8 0
#endif
// 2^x on the FMA pipe for x <= ~1: round-to-nearest split x = n + f, |f| <= 0.5, cubic for 2^f (max relative
// error 7.5e-5; the results are rounded to bf16, 3.9e-3), n added to the exponent field.  Very negative
// arguments (masked scores) give 2^-126, i.e. zero for every purpose here.
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -126.f);
  const float t = __fadd_rn(x, 12582912.f);             // 1.5 * 2^23: n sits in the low mantissa bits of t
  const float f = __fsub_rn(x, __fsub_rn(t, 12582912.f));
  float r = fmaf(f, 0.05517164617776871f, 0.2426111251115799f);
  r = fmaf(r, f, 0.6932609677314758f);
  r = fmaf(r, f, 0.9999280571937561f);
  return __int_as_float(__float_as_int(r) + (__float_as_int(t) << 23));
}

// row maximum of 64 scores, columns [col0, col0 + 64) of a tile whose visible columns are [mlo, mlo + span]
template <bool MASK>
__device__ __forceinline__ void max64(const uint32_t (&a)[32], const uint32_t (&b)[32], int col0, int mlo, unsigned span,
                                      float (&mxa)[4]) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    float x = __uint_as_float(a[j]), y = __uint_as_float(b[j]);
    if constexpr (MASK) {
      x = (unsigned(col0 + j - mlo) <= span) ? x : -INFINITY;
      y = (unsigned(col0 + 32 + j - mlo) <= span) ? y : -INFINITY;
    }
    mxa[j & 3] = fmaxf(mxa[j & 3], fmaxf(x, y));
  }
}

// Exponentials of the 64 scores of columns [col0, col0 + 64) of one row (two 32-column loads), written to
// `tm_dst` as 32 columns of bf16 pairs; row sums into four chains.
template <bool MASK>
__device__ __forceinline__ void exp64_store(const uint32_t (&s0)[32], const uint32_t (&s1)[32], uint32_t tm_dst, float c,
                                            float mc, int col0, int mlo, unsigned span, float (&rsa)[4]) {
  uint32_t pk[32];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    float e[4];
    // ARB_FWD2_POLY of every four exponentials go to the FMA pipe as a cubic instead of the ex2 unit (measured on the
    // two-query-tile forward, full causal T=32768: 0 -> 9.25 ms, 1 -> 10.65 ms, 2 -> 11.54 ms: the softmax warps are
    // short of issue slots, not of ex2 throughput, so the default is 0)
    e[0] = fast_exp2(__uint_as_float(s0[2 * j]) * c - mc);
    e[1] = (ARB_FWD2_POLY >= 2) ? poly_exp2(__uint_as_float(s0[2 * j + 1]) * c - mc) : fast_exp2(__uint_as_float(s0[2 * j + 1]) * c - mc);
    e[2] = fast_exp2(__uint_as_float(s1[2 * j]) * c - mc);
    e[3] = (ARB_FWD2_POLY >= 1) ? poly_exp2(__uint_as_float(s1[2 * j + 1]) * c - mc) : fast_exp2(__uint_as_float(s1[2 * j + 1]) * c - mc);
    if constexpr (MASK) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int col = col0 + (u >> 1) * 32 + 2 * j + (u & 1);
        e[u] = (unsigned(col - mlo) <= span) ? e[u] : 0.f;
      }
    }
    rsa[j & 3] += (e[0] + e[1]) + (e[2] + e[3]);
    pk[j] = pack_bf16(e[0], e[1]);
    pk[16 + j] = pack_bf16(e[2], e[3]);
  }
  tmem_st32(tm_dst, pk);
}

__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// [B, T, H, 128] bf16 view with token stride ld: dims {128, H, T, B}; box {64, 1, rows, 1}
inline int make_qkv_tmap(CUtensorMap* m, const void* base, int B, int T, int H, long long ld, int box_rows) {
  uint64_t dims[4] = {128, uint64_t(H), uint64_t(T), uint64_t(B)};
  uint64_t str[3] = {256, uint64_t(ld) * 2, uint64_t(ld) * 2 * uint64_t(T)};
  uint32_t box[4] = {64, 1, uint32_t(box_rows), 1};
  return make_tmap_bf16(m, base, 4, dims, str, box);
}

inline bool bad_ptr(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

template <typename Kern>
inline int set_smem(Kern k, int bytes) {
  return int(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}


// attn_wide_sm100.cu
int attn_wide_bwd_launch(const void* q, const void* k, const void* v, const void* d_o, void* dq, void* dk, void* dv,
                         long long ldq, long long ldk, long long ldv, long long lddo, long long lddq, long long lddk,
                         long long lddv, AttnArgs a, cudaStream_t stream);


// attn_fwd2_sm100.cu
int attn_fwd2_launch(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv, AttnArgs a,
                     cudaStream_t stream);


// attn_fwd3_sm100.cu
int attn_fwd3_launch(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv, AttnArgs a,
                     cudaStream_t stream);

}  // namespace arb
