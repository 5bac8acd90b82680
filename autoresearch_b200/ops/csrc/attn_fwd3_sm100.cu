// Flash attention forward for head_dim = 128, two 128-query tiles per CTA, with the register file split between the
// roles: the third forward kernel of this package, used for long key ranges (full-causal layers).
//
// Same data flow as attn_fwd2_sm100.cu (S0 | S1 | O0 | O1 in TMEM, one softmax warp group per query tile, the
// single MMA-issuing thread interleaves  ... PV0(t) S0(t+1) PV1(t) S1(t+1) ...,  P written over the score tile).
// What is different is the softmax, which bounds that kernel (its role counters show the score pass at ~1900 clk per
// tile and group against ~1000 clk of tensor work):
//   * registers: the CTA has twelve warps = three warp groups; after start-up the group that only moves data and
//     issues MMAs gives registers back (setmaxnreg.dec to 56) and the two softmax groups take them (setmaxnreg.inc
//     to 224), so a thread holds its whole 128-column score row in registers: ONE tcgen05.ld pass per tile instead of
//     two (row maximum, then exponentials), and no TMEM traffic between them;
//   * arithmetic: scale-and-shift, row sums and the polynomial below run as packed fp32 pairs (fma.rn.f32x2 /
//     add.f32x2: two results per issue slot);
//   * the ex2 unit does 16 results per clock and SM, i.e. 1024 clk per 128 x 128 tile - as long as the tensor work of
//     the tile.  One exponential in four is therefore evaluated on the FMA pipe instead (round-to-nearest split,
//     cubic for 2^f, exponent add; relative error 7.5e-5 before the bf16 rounding of P).
//
// Mask semantics: key j is visible to query i iff i - window <= j <= i (brain/src/forward.rs:1134-1138); the
// reference calls a Hopper-only FlashAttention-3 build here (brain/src/forward.rs:1124-1177).
#include "attn_common.cuh"

namespace arb {

constexpr int ATT_FWD3_THREADS = 384;   // softmax group 0 (warps 0-3), softmax group 1 (4-7), warp 8 TMA, warp 9 MMA, 10-11 idle

__device__ __forceinline__ void reg_alloc_224() { asm volatile("setmaxnreg.inc.sync.aligned.u32 224;"); }
__device__ __forceinline__ void reg_dealloc_56() { asm volatile("setmaxnreg.dec.sync.aligned.u32 56;"); }

// packed fp32 pairs in one 64-bit register
__device__ __forceinline__ unsigned long long pk2(float a, float b) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpk2(unsigned long long v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ unsigned long long sub2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// 2^x for a pair, x <= ~1, on the FMA pipe (see poly_exp2 in attn_common.cuh for the scalar form)
__device__ __forceinline__ void poly_exp2_pair(unsigned long long x, float& e0, float& e1) {
  float x0, x1;
  unpk2(x, x0, x1);
  x = pk2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const unsigned long long magic = pk2(12582912.f, 12582912.f);
  const unsigned long long t = add2(x, magic);                 // n in the low mantissa bits
  const unsigned long long f = sub2(x, sub2(t, magic));
  unsigned long long r = fma2(f, pk2(0.05517164617776871f, 0.05517164617776871f), pk2(0.2426111251115799f, 0.2426111251115799f));
  r = fma2(r, f, pk2(0.6932609677314758f, 0.6932609677314758f));
  r = fma2(r, f, pk2(0.9999280571937561f, 0.9999280571937561f));
  float r0, r1, t0, t1;
  unpk2(r, r0, r1);
  unpk2(t, t0, t1);
  e0 = __int_as_float(__float_as_int(r0) + (__float_as_int(t0) << 23));
  e1 = __int_as_float(__float_as_int(r1) + (__float_as_int(t1) << 23));
}

// Exponentials of 32 scores (one tcgen05.ld chunk) of a row: e = 2^(s*c - mc); bf16 pairs into pk[16]; row sum into
// the packed accumulator.  Pairs 3, 7, 11, 15 of the chunk (one in four) take the polynomial.
template <bool MASK>
__device__ __forceinline__ void exp32(const uint32_t (&s)[32], uint32_t* pk, unsigned long long c2, unsigned long long nmc2,
                                      int col0, int mlo, unsigned span, unsigned long long& rs2) {
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const unsigned long long x = fma2(pk2(__uint_as_float(s[2 * j]), __uint_as_float(s[2 * j + 1])), c2, nmc2);
    float e0, e1;
    if ((j & 3) == 3) {
      poly_exp2_pair(x, e0, e1);
    } else {
      float x0, x1;
      unpk2(x, x0, x1);
      e0 = fast_exp2(x0);
      e1 = fast_exp2(x1);
    }
    if constexpr (MASK) {
      e0 = (unsigned(col0 + 2 * j - mlo) <= span) ? e0 : 0.f;
      e1 = (unsigned(col0 + 2 * j + 1 - mlo) <= span) ? e1 : 0.f;
    }
    rs2 = add2(rs2, pk2(e0, e1));
    pk[j] = pack_bf16(e0, e1);
  }
}

template <bool MASK>
__device__ __forceinline__ float max32(const uint32_t (&s)[32], int col0, int mlo, unsigned span, float m) {
  float a = m, b = m;
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      v[u] = __uint_as_float(s[j + u]);
      if constexpr (MASK) v[u] = (unsigned(col0 + j + u - mlo) <= span) ? v[u] : -INFINITY;
    }
    a = fmaxf(a, fmaxf(v[0], v[1]));      // three-input maximum: one instruction each
    b = fmaxf(b, fmaxf(v[2], v[3]));
  }
  return fmaxf(a, b);
}

struct Fwd3Smem {
  static constexpr int Q = 0;                       // 2 x 32 KB
  static constexpr int K0 = 65536;                  // 3 x 32 KB
  static constexpr int V0 = K0 + 3 * 32768;         // 2 x 32 KB
  static constexpr int BAR = V0 + 2 * 32768;
  static constexpr int TOTAL = BAR + 512;
};
static_assert(Fwd3Smem::TOTAL <= 232448, "exceeds the 227 KB shared memory of one CTA");

__global__ void __launch_bounds__(ATT_FWD3_THREADS, 1)
attn_fwd3_k(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
            const __grid_constant__ CUtensorMap tmV, const AttnArgs p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, ERR_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Fwd3Smem::BAR);
  uint64_t* q_full = bars;          // both query tiles landed
  uint64_t* k_full = bars + 1;      // [3]
  uint64_t* k_empty = bars + 4;     // [3] every S MMA that reads the slot has been issued and is complete
  uint64_t* v_full = bars + 7;      // [2]
  uint64_t* v_empty = bars + 9;     // [2]
  uint64_t* s_full = bars + 11;     // [2] per query tile: S_i of its n-th key tile complete
  uint64_t* p_full = bars + 13;     // [2] per query tile: P_i written (4 arrivals)
  uint64_t* o_done = bars + 15;     // [2] per query tile: last PV_i complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_pair = (p.T + 255) / 256;
  const int mp = n_pair - 1 - int(blockIdx.x);     // later queries see more keys: schedule them first
  const int h = blockIdx.y, b = blockIdx.z;
  const int m0 = mp * 256;
  // key-tile range of each query tile; tile 1 is empty when the sequence ends inside tile 0
  int lo_i[2], hi_i[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int mi = m0 + 128 * i;
    lo_i[i] = (p.window >= p.T) ? 0 : max(0, (mi - p.window) / 128);
    hi_i[i] = (mi < p.T) ? min((p.T - 1) / 128, (mi + 127) / 128) : -1;
    if (hi_i[i] < 0) lo_i[i] = 1 << 30;
  }
  const int lo = min(lo_i[0], lo_i[1]), hi = max(hi_i[0], hi_i[1]);
  auto uses = [&](int i, int t) { return t >= lo_i[i] && t <= hi_i[i]; };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&o_done[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // The data-movement warp group hands registers to the two softmax groups; each setmaxnreg is the first
  // instruction of its group's branch (executed by all four warps of the group) and dominates the group's code.
  if (warp >= 8) {
  reg_dealloc_56();
  if (warp == 8) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 65536);                 // rows past the end of the sequence are zero-filled
      for (int i = 0; i < 2; ++i) {
        tma_load_4d(smem + Fwd3Smem::Q + i * 32768, &tmQ, q_full, 0, h, m0 + 128 * i, b);
        tma_load_4d(smem + Fwd3Smem::Q + i * 32768 + 16384, &tmQ, q_full, 64, h, m0 + 128 * i, b);
      }
      for (int t = lo; t <= hi; ++t) {
        const int kt = t - lo, n0 = t * 128;
        if (!mbar_wait(&k_empty[kt % 3], (uint32_t(kt / 3) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* ks = smem + Fwd3Smem::K0 + (kt % 3) * 32768;
        mbar_expect_tx(&k_full[kt % 3], 32768);
        tma_load_4d(ks, &tmK, &k_full[kt % 3], 0, h, n0, b);
        tma_load_4d(ks + 16384, &tmK, &k_full[kt % 3], 64, h, n0, b);
        if (!mbar_wait(&v_empty[kt & 1], (uint32_t(kt >> 1) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* vs = smem + Fwd3Smem::V0 + (kt & 1) * 32768;
        mbar_expect_tx(&v_full[kt & 1], 32768);
        tma_load_4d(vs, &tmV, &v_full[kt & 1], 0, h, n0, b);
        tma_load_4d(vs + 16384, &tmV, &v_full[kt & 1], 64, h, n0, b);
      }
    }
  } else if (warp == 9) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      const uint32_t sq = smem_u32(smem + Fwd3Smem::Q);
      const uint32_t sk0 = smem_u32(smem + Fwd3Smem::K0), sv0 = smem_u32(smem + Fwd3Smem::V0);
      int cnt[2] = {0, 0};                           // key tiles of each query tile whose PV has been issued
      // descriptor words computed once: low word = start address >> 4 (+ the leading-dimension offset for V), high word
      // constant; a K slice or a ring slot is a 32-bit add on the low word.  The thread issues from a warp whose scheduler
      // also serves two softmax warps, so every instruction between two MMAs counts.
      const uint32_t hi_k = uint32_t(make_smem_desc(0, 0, 1024) >> 32), hi_v = uint32_t(make_smem_desc(0, 16384, 1024) >> 32);
      const uint32_t q_lo = uint32_t(make_smem_desc(sq, 0, 1024)), k_lo = uint32_t(make_smem_desc(sk0, 0, 1024));
      const uint32_t v_lo = uint32_t(make_smem_desc(sv0, 16384, 1024));
      auto issue_s = [&](int i, int t) {             // S_i = Q_i K(t)^T ; K(t) has been waited for by the caller
        const uint32_t kb = k_lo + uint32_t((t - lo) % 3) * 2048u, qa = q_lo + uint32_t(i) * 2048u;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = uint32_t(k >> 2) * 1024u + uint32_t(k & 3) * 2u;     // (16 KB half, 32 B slice) >> 4
          tc_mma_ss_lh(tmem + uint32_t(i) * 128u, qa + off, hi_k, kb + off, hi_k, idesc_s, k > 0);
        }
        tc_commit(&s_full[i]);
      };
      auto wait_p = [&](int i) -> bool {
        if (!mbar_wait(&p_full[i], uint32_t(cnt[i]) & 1u, abort_flag)) return false;
        tc_fence_after();
        return true;
      };
      auto issue_pv = [&](int i, int t) {            // O_i += P_i V(t)
        const uint32_t vb = v_lo + uint32_t((t - lo) & 1) * 2048u;
        const uint32_t to = tmem + 256u + uint32_t(i) * 128u, tp = tmem + uint32_t(i) * 128u;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_ts_lh(to, tp + uint32_t(k) * 8u, vb + uint32_t(k) * 128u, hi_v, idesc_o, (cnt[i] > 0 || k > 0) ? 1u : 0u);
        ++cnt[i];
        if (t == hi_i[i]) tc_commit(&o_done[i]);
      };
      PROF_DECL();                                   // total only: marks inside the loop cost this thread registers it does not have
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        if (uses(0, lo)) issue_s(0, lo);
        if (uses(1, lo)) issue_s(1, lo);
        tc_commit(&k_empty[0]);
      }
      for (int t = lo; t <= hi && ok; ++t) {
        const int kt = t - lo;
        const bool nxt = t + 1 <= hi;
        if (!mbar_wait(&v_full[kt & 1], uint32_t(kt >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (uses(0, t)) {
          if (!wait_p(0)) { ok = false; break; }
          issue_pv(0, t);
        }
        if (nxt) {
          if (!mbar_wait(&k_full[(kt + 1) % 3], uint32_t((kt + 1) / 3) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if (uses(0, t + 1)) issue_s(0, t + 1);     // after PV0(t): it overwrites the tile P0(t) lives in
        }
        if (uses(1, t)) {
          if (!wait_p(1)) { ok = false; break; }
          issue_pv(1, t);
        }
        tc_commit(&v_empty[kt & 1]);
        if (nxt) {
          if (uses(1, t + 1)) issue_s(1, t + 1);
          tc_commit(&k_empty[(kt + 1) % 3]);
        }
      }
      PROF_DUMP(0);
    }
  }
  } else {
    reg_alloc_224();
    // ---------------- softmax / epilogue: warp group i <-> query tile i, thread <-> query row ----------------
    const int sw = warp;
    const int i = sw >> 2;
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int row = m0 + 128 * i + r;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const uint32_t TM_S = tmem + uint32_t(i) * 128u, TM_O = tmem + 256u + uint32_t(i) * 128u;
    const float c = p.scale * LOG2E;
    const int mi = m0 + 128 * i;
    const int my_lo = i ? lo_i[1] : lo_i[0], my_hi = i ? hi_i[1] : hi_i[0];
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    int n = 0;
    PROF_DECL();
    for (int t = my_lo; t <= my_hi && ok; ++t, ++n) {
      const int n0 = t * 128;
      PROF_TIC();
      if (!mbar_wait(&s_full[i], uint32_t(n) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      PROF_TOC(1);
      const bool need_mask = (n0 + 127 > mi) || (p.window < p.T && n0 < mi + 127 - p.window) || (n0 + 127 >= p.T);
      // visible keys of this row inside the tile: column indices [mlo, mlo + span]
      const int mlo = (row < p.T) ? row - p.window - n0 : 128;
      const unsigned span = (row < p.T) ? unsigned(p.window) : 0u;
      // ---- the whole score row into registers: one TMEM pass ----
      uint32_t sa[32], sb[32], sc[32], sd[32];
      tmem_ld32(TM_S + lane_addr, sa);
      tmem_ld32(TM_S + lane_addr + 32u, sb);
      tmem_ld32(TM_S + lane_addr + 64u, sc);
      tmem_ld32(TM_S + lane_addr + 96u, sd);
      tmem_wait_ld();
      float mx;
      if (need_mask) {
        mx = max32<true>(sa, 0, mlo, span, -INFINITY);
        mx = max32<true>(sb, 32, mlo, span, mx);
        mx = max32<true>(sc, 64, mlo, span, mx);
        mx = max32<true>(sd, 96, mlo, span, mx);
      } else {
        mx = max32<false>(sa, 0, mlo, span, -INFINITY);
        mx = max32<false>(sb, 32, mlo, span, mx);
        mx = max32<false>(sc, 64, mlo, span, mx);
        mx = max32<false>(sd, 96, mlo, span, mx);
      }
      const float m_new = fmaxf(m_used, mx);
      PROF_TOC(2);
      bool resc = false;
      if (m_used == -INFINITY) m_used = m_new;            // nothing accumulated for this row yet
      else resc = (m_new - m_used) * c > 8.f;
      if (n > 0 && __any_sync(0xffffffffu, resc)) {
        // S_i(t) complete implies PV_i(t-1) complete: O_i is not in flight
        const float alpha = resc ? fast_exp2((m_used - m_new) * c) : 1.f;
        if (resc) { l *= alpha; m_used = m_new; }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t v[32];
          tmem_ld32(TM_O + lane_addr + uint32_t(cc * 32), v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
          tmem_st32(TM_O + lane_addr + uint32_t(cc * 32), v);
        }
        tmem_wait_st();
      }
      const float mc = (m_used == -INFINITY) ? 0.f : m_used * c;
      PROF_TOC(3);
      // ---- exponentials from registers; P (bf16 pairs) over the first 64 columns of the tile ----
      const unsigned long long c2 = pk2(c, c), nmc2 = pk2(-mc, -mc);
      unsigned long long rs2 = pk2(0.f, 0.f);
      uint32_t p0[32], p1[32];
      if (need_mask) {
        exp32<true>(sa, p0, c2, nmc2, 0, mlo, span, rs2);
        exp32<true>(sb, p0 + 16, c2, nmc2, 32, mlo, span, rs2);
        exp32<true>(sc, p1, c2, nmc2, 64, mlo, span, rs2);
        exp32<true>(sd, p1 + 16, c2, nmc2, 96, mlo, span, rs2);
      } else {
        exp32<false>(sa, p0, c2, nmc2, 0, mlo, span, rs2);
        exp32<false>(sb, p0 + 16, c2, nmc2, 32, mlo, span, rs2);
        exp32<false>(sc, p1, c2, nmc2, 64, mlo, span, rs2);
        exp32<false>(sd, p1 + 16, c2, nmc2, 96, mlo, span, rs2);
      }
      tmem_st32(TM_S + lane_addr, p0);
      tmem_st32(TM_S + lane_addr + 32u, p1);
      {
        float r0, r1;
        unpk2(rs2, r0, r1);
        l += r0 + r1;
      }
      PROF_TOC(4);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i]);
      PROF_TOC(5);
    }
    if (lane == 0 && (sw == 0 || sw == 4)) PROF_DUMP(sw == 0 ? 2 : 3);
    if (ok && my_hi >= my_lo && mbar_wait(&o_done[i], 0, abort_flag)) {
      tc_fence_after();
      const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + ((long long)b * p.T + row) * p.ldo + h * HD;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t v[32];
        tmem_ld32(TM_O + lane_addr + uint32_t(cc * 32), v);
        tmem_wait_ld();
        if (row < p.T) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 u;
            u.x = pack_bf16(__uint_as_float(v[j]) * inv_l, __uint_as_float(v[j + 1]) * inv_l);
            u.y = pack_bf16(__uint_as_float(v[j + 2]) * inv_l, __uint_as_float(v[j + 3]) * inv_l);
            u.z = pack_bf16(__uint_as_float(v[j + 4]) * inv_l, __uint_as_float(v[j + 5]) * inv_l);
            u.w = pack_bf16(__uint_as_float(v[j + 6]) * inv_l, __uint_as_float(v[j + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + cc * 32 + j) = u;
          }
        }
      }
      if (row < p.T) p.lse[((long long)b * p.H + h) * p.T + row] = (l > 0.f) ? (m_used * p.scale + __logf(l)) : -INFINITY;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, ERR_ATTN_TIMEOUT);
  if (warp == 9) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 512); }
}

int attn_fwd3_launch(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv, AttnArgs a,
                     cudaStream_t stream) {
  static PerDeviceOnce cfg;
  int r;
  if (cfg.first()) { if ((r = set_smem(attn_fwd3_k, Fwd3Smem::TOTAL))) return r; }
  CUtensorMap tq, tk, tv;
  if ((r = make_qkv_tmap(&tq, q, a.B, a.T, a.H, ldq, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tk, k, a.B, a.T, a.H, ldk, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tv, v, a.B, a.T, a.H, ldv, 128))) return 1000 + r;
  dim3 grid((a.T + 255) / 256, a.H, a.B);
  attn_fwd3_k<<<grid, ATT_FWD3_THREADS, Fwd3Smem::TOTAL, stream>>>(tq, tk, tv, a);
  return int(cudaGetLastError());
}

}  // namespace arb

#ifdef ARB_ATTN_PROF
// Entry point of the profiling build (bench/attn_roles.py --kernel fwd2): runs the forward once and leaves the
// per-role cycle counters of CTA (0,0,0) in `prof` (device, 64 x int64).
extern "C" int arb_attn_prof_fwd3(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int H,
                                  long long ld, long long ldo, int window, float scale, int* err, long long* prof) {
  cudaMemcpyToSymbol(arb::arb_attn_prof_buffer, &prof, sizeof(prof));
  arb::AttnArgs a{};
  a.B = B; a.T = T; a.H = H; a.window = window > T ? T : window; a.scale = scale;
  a.o = o; a.ldo = ldo; a.lse = lse; a.err = err;
  return arb::attn_fwd3_launch(q, k, v, ld, ld, ld, a, 0);
}
#endif
