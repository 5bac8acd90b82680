// Flash attention forward for head_dim = 128 with TWO 128-query tiles per CTA in ping-pong.
//
// The one-tile kernel (attn_sm100.cu) alternates between its softmax warps and its MMAs: while the
// four softmax warps work on a score tile the tensor pipe has little to do, and vice versa.  Here a
// CTA owns 256 queries as two tiles with their own score / output accumulators in TMEM
// (S0 | S1 | O0 | O1 = 4 x 128 columns) and one softmax warp group each; the single MMA-issuing
// thread interleaves them,
//
//     ... PV0(t)  S0(t+1)  PV1(t)  S1(t+1)  PV0(t+1) ...
//
// so that group 0 computes its softmax of tile t+1 while the pipe runs PV1(t) and S1(t+1), and the
// K / V tiles are loaded once for both query tiles.  P (bf16) overwrites the first 64 columns of the
// score tile it was computed from: every thread owns one row, reads 64 score columns, converts them
// and writes 32 packed columns front to back, never ahead of its own reads; the next S MMA into that
// tile is issued after the PV MMA that reads P (MMAs of one thread execute in order), which also
// means that "S(t+1) complete" implies "PV(t) complete" and the rare rescale of O needs no barrier
// of its own.  The scores are read from TMEM twice (row maximum, then exponentials) instead of being
// held in 128 registers.
//
// Measured (B=4, H=8, T=32768, B200 under its power cap): 3-5 % faster than the one-tile kernel (full causal 9.79 ->
// 9.42 ms, window 4096 2.61 -> 2.50 ms, window 256 0.51 -> 0.47 ms); slower on grids of few waves, so the dispatcher
// uses it on large grids only.  Two findings from the role counters (bench/attn_roles.py --kernel fwd2): (1) a mask
// test inside the unrolled loops, even on tiles that need none, doubled both softmax passes (full causal 13.05 ms
// with it), so the masked variants are selected per tile outside the loops; (2) with that fixed the MMA-issuing
// thread is the bound: the 32 MMAs of a key tile take about 3000 clk to issue (94 each, 66 in isolation), and each
// softmax group waits for scores half of the time.
//
// Mask semantics: key j is visible to query i iff i - window <= j <= i
// (brain/src/forward.rs:1134-1138); the reference calls a Hopper-only FlashAttention-3 build here
// (brain/src/forward.rs:1124-1177).
#include "attn_common.cuh"

namespace arb {

struct Fwd2Smem {
  static constexpr int Q = 0;                       // 2 x 32 KB
  static constexpr int K0 = 65536;                  // 3 x 32 KB
  static constexpr int V0 = K0 + 3 * 32768;         // 2 x 32 KB
  static constexpr int BAR = V0 + 2 * 32768;
  static constexpr int TOTAL = BAR + 512;
};
static_assert(Fwd2Smem::TOTAL <= 232448, "exceeds the 227 KB shared memory of one CTA");

__global__ void __launch_bounds__(ATT_WIDE_THREADS, 1)
attn_fwd2_k(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
            const __grid_constant__ CUtensorMap tmV, const AttnArgs p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, ERR_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Fwd2Smem::BAR);
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
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 65536);                 // rows past the end of the sequence are zero-filled
      for (int i = 0; i < 2; ++i) {
        tma_load_4d(smem + Fwd2Smem::Q + i * 32768, &tmQ, q_full, 0, h, m0 + 128 * i, b);
        tma_load_4d(smem + Fwd2Smem::Q + i * 32768 + 16384, &tmQ, q_full, 64, h, m0 + 128 * i, b);
      }
      for (int t = lo; t <= hi; ++t) {
        const int kt = t - lo, n0 = t * 128;
        if (!mbar_wait(&k_empty[kt % 3], (uint32_t(kt / 3) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* ks = smem + Fwd2Smem::K0 + (kt % 3) * 32768;
        mbar_expect_tx(&k_full[kt % 3], 32768);
        tma_load_4d(ks, &tmK, &k_full[kt % 3], 0, h, n0, b);
        tma_load_4d(ks + 16384, &tmK, &k_full[kt % 3], 64, h, n0, b);
        if (!mbar_wait(&v_empty[kt & 1], (uint32_t(kt >> 1) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* vs = smem + Fwd2Smem::V0 + (kt & 1) * 32768;
        mbar_expect_tx(&v_full[kt & 1], 32768);
        tma_load_4d(vs, &tmV, &v_full[kt & 1], 0, h, n0, b);
        tma_load_4d(vs + 16384, &tmV, &v_full[kt & 1], 64, h, n0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      const uint32_t sq = smem_u32(smem + Fwd2Smem::Q);
      const uint32_t sk0 = smem_u32(smem + Fwd2Smem::K0), sv0 = smem_u32(smem + Fwd2Smem::V0);
      int cnt[2] = {0, 0};                           // key tiles of each query tile whose PV has been issued
      // descriptor words computed once; a K slice or a ring slot is an add on the low word (start address >> 4)
      const uint32_t hi_k = uint32_t(make_smem_desc(0, 0, 1024) >> 32), hi_v = uint32_t(make_smem_desc(0, 16384, 1024) >> 32);
      const uint32_t q_lo = uint32_t(make_smem_desc(sq, 0, 1024)), k_lo = uint32_t(make_smem_desc(sk0, 0, 1024));
      const uint32_t v_lo = uint32_t(make_smem_desc(sv0, 16384, 1024));
      auto issue_s = [&](int i, int t) {             // S_i = Q_i K(t)^T ; K(t) has been waited for by the caller
        const uint32_t kb = k_lo + uint32_t((t - lo) % 3) * 2048u, qa = q_lo + uint32_t(i) * 2048u;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = uint32_t(k >> 2) * 1024u + uint32_t(k & 3) * 2u;
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
#pragma unroll
        for (int k = 0; k < 8; ++k)
          tc_mma_ts_lh(tmem + 256u + uint32_t(i) * 128u, tmem + uint32_t(i) * 128u + uint32_t(k) * 8u, vb + uint32_t(k) * 128u, hi_v,
                       idesc_o, (cnt[i] > 0 || k > 0) ? 1u : 0u);
        ++cnt[i];
        if (t == hi_i[i]) tc_commit(&o_done[i]);
      };
      PROF_DECL();
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
        PROF_TIC();
        if (!mbar_wait(&v_full[kt & 1], uint32_t(kt >> 1) & 1u, abort_flag)) { ok = false; break; }
        PROF_TOC(1);
        if (uses(0, t)) {
          if (!wait_p(0)) { ok = false; break; }
          PROF_TOC(2);
          issue_pv(0, t);
        }
        PROF_TOC(3);
        if (nxt) {
          if (!mbar_wait(&k_full[(kt + 1) % 3], uint32_t((kt + 1) / 3) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          PROF_TOC(4);
          if (uses(0, t + 1)) issue_s(0, t + 1);     // after PV0(t): it overwrites the tile P0(t) lives in
        }
        PROF_TOC(5);
        if (uses(1, t)) {
          if (!wait_p(1)) { ok = false; break; }
          PROF_TOC(6);
          issue_pv(1, t);
        }
        tc_commit(&v_empty[kt & 1]);
        if (nxt) {
          if (uses(1, t + 1)) issue_s(1, t + 1);
          tc_commit(&k_empty[(kt + 1) % 3]);
        }
        PROF_TOC(7);
      }
      PROF_DUMP(0);
    }
  } else {
    // ---------------- softmax / epilogue: warp group i <-> query tile i, thread <-> query row ----------------
    const int sw = warp - 2;
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
      // ---- pass 1: row maximum ----
      float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      // the masked variants are selected per tile, outside the unrolled loops: a compare / select per element in the
      // common path doubled the time of both passes
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t s0[32], s1[32];
        tmem_ld32(TM_S + lane_addr + uint32_t(hf * 64), s0);
        tmem_ld32(TM_S + lane_addr + uint32_t(hf * 64 + 32), s1);
        tmem_wait_ld();
        if (need_mask) max64<true>(s0, s1, hf * 64, mlo, span, mxa);
        else max64<false>(s0, s1, hf * 64, mlo, span, mxa);
      }
      const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3]));
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
      // ---- pass 2: exponentials; P (bf16 pairs) overwrites the tile front to back, behind the reads ----
      float rsa[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t s0[32], s1[32];
        tmem_ld32(TM_S + lane_addr + uint32_t(hf * 64), s0);
        tmem_ld32(TM_S + lane_addr + uint32_t(hf * 64 + 32), s1);
        tmem_wait_ld();
        // columns [32 hf, 32 hf + 32) <= scores already read
        if (need_mask) exp64_store<true>(s0, s1, TM_S + lane_addr + uint32_t(hf * 32), c, mc, hf * 64, mlo, span, rsa);
        else exp64_store<false>(s0, s1, TM_S + lane_addr + uint32_t(hf * 32), c, mc, hf * 64, mlo, span, rsa);
      }
      l += (rsa[0] + rsa[1]) + (rsa[2] + rsa[3]);
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
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 512); }
}

int attn_fwd2_launch(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv, AttnArgs a,
                     cudaStream_t stream) {
  static PerDeviceOnce cfg;
  int r;
  if (cfg.first()) { if ((r = set_smem(attn_fwd2_k, Fwd2Smem::TOTAL))) return r; }
  CUtensorMap tq, tk, tv;
  if ((r = make_qkv_tmap(&tq, q, a.B, a.T, a.H, ldq, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tk, k, a.B, a.T, a.H, ldk, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tv, v, a.B, a.T, a.H, ldv, 128))) return 1000 + r;
  dim3 grid((a.T + 255) / 256, a.H, a.B);
  attn_fwd2_k<<<grid, ATT_WIDE_THREADS, Fwd2Smem::TOTAL, stream>>>(tq, tk, tv, a);
  return int(cudaGetLastError());
}

}  // namespace arb

#ifdef ARB_ATTN_PROF
// Entry point of the profiling build (bench/attn_roles.py --kernel fwd2): runs the forward once and leaves the
// per-role cycle counters of CTA (0,0,0) in `prof` (device, 64 x int64).
extern "C" int arb_attn_prof_fwd2(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int H,
                                  long long ld, long long ldo, int window, float scale, int* err, long long* prof) {
  cudaMemcpyToSymbol(arb::arb_attn_prof_buffer, &prof, sizeof(prof));
  arb::AttnArgs a{};
  a.B = B; a.T = T; a.H = H; a.window = window > T ? T : window; a.scale = scale;
  a.o = o; a.ldo = ldo; a.lse = lse; a.err = err;
  return arb::attn_fwd2_launch(q, k, v, ld, ld, ld, a, 0);
}
#endif
