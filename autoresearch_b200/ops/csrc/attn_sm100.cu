// Causal / sliding-window flash attention for head_dim = 128 on tcgen05 tensor cores with
// TMEM accumulators.  Three kernels share one structure (TMA producer warp, single-thread MMA
// issuer, four softmax/epilogue warps that own one TMEM lane = one row each):
//
//   attn_fwd_k   : per 128-query tile, loop over visible 128-key tiles:
//                  S = Q K^T (TMEM, double buffered) -> online softmax in registers (exp2,
//                  lazy rescale of O only when the row maximum grows by more than 2^8) ->
//                  P (bf16, swizzled smem) -> O += P V (TMEM).
//   attn_bwd_dq_k: per 128-query tile: S = Q K^T, dP = dO V^T -> dS = P o (dP - delta) * scale
//                  -> dQ += dS K.
//   attn_bwd_dkv_k: per 128-key tile, loop over visible 64-query tiles, transposed scores:
//                  S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T -> dV += P^T dO, dK += dS^T Q.
//
// Fully masked key tiles are never visited (causal upper triangle, keys older than the
// window).  Mask semantics: key j is visible to query i iff i - window <= j <= i
// (brain/src/forward.rs:1134-1138, brain/fa3/flash3_api.cu:124-133).  The reference calls a
// Hopper-only FlashAttention-3 build here (brain/src/forward.rs:1124-1177,
// brain/src/backward.rs:613-659); the two-kernel backward is deterministic (no atomics into
// dQ, unlike the FA3 semaphore/atomic accumulation).
#include "api.h"
#include "ptx.cuh"
#include "tmap.h"
#include "attn_common.cuh"

namespace arb {

// ===============================================================================================
// Forward
// ===============================================================================================
// TS = the bf16 probabilities are handed to the P*V MMA through TMEM (A operand from tensor
// memory) instead of swizzled shared memory.  Shared-memory bandwidth (128 B/clk) is what bounds
// these kernels: an SS MMA of M=128, N=128, K=16 reads 8 KB of operands for 64 clk of math, so every
// operand that stays out of shared memory counts.  The freed 64 KB hold a third K/V stage.
template <bool TS>
struct FwdSmemT {
  static constexpr int STAGES = TS ? 3 : 2;
  static constexpr int Q = 0;
  static constexpr int K0 = 32768;                 // STAGES x 32 KB
  static constexpr int V0 = K0 + STAGES * 32768;   // STAGES x 32 KB
  static constexpr int P0 = V0 + STAGES * 32768;   // SS only: 2 buffers of 32 KB
  static constexpr int BAR = P0 + (TS ? 0 : 2 * 32768);
  static constexpr int TOTAL = BAR + 256 + 1024;
};

template <bool TS>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_k(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
           const __grid_constant__ CUtensorMap tmV, const AttnArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using FwdSmem = FwdSmemT<TS>;
  constexpr int ST = FwdSmem::STAGES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + FwdSmem::BAR);
  uint64_t* q_full = bars;             // 1
  uint64_t* k_full = bars + 1;         // ST
  uint64_t* k_empty = k_full + ST;     // ST
  uint64_t* v_full = k_empty + ST;     // ST
  uint64_t* v_empty = v_full + ST;     // ST
  uint64_t* s_full = v_empty + ST;     // 2
  uint64_t* s_empty = s_full + 2;      // 2
  uint64_t* p_full = s_empty + 2;      // 2
  uint64_t* p_empty = p_full + 2;      // 2
  uint64_t* o_done = p_empty + 2;      // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Heavier (later) query tiles are scheduled first.
  const int n_mt = (p.T + 127) / 128;
  const int mt = n_mt - 1 - int(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int m0 = mt * 128;
  const int j_lo = (p.window >= p.T) ? 0 : max(0, (m0 - p.window) / 128);
  const int j_hi = min((p.T - 1) / 128, (m0 + 127) / 128);
  const int n_tiles = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < ST; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4);
      mbar_init(&p_full[i], 4); mbar_init(&p_empty[i], 1);
    }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t TM_S = tmem, TM_O = tmem + 256, TM_P = tmem + 384;   // S[2] x 128, O 128, P[2] x 64 (TS)

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, 32768);
      tma_load_4d(smem + FwdSmem::Q, &tmQ, q_full, 0, h, m0, b);
      tma_load_4d(smem + FwdSmem::Q + 16384, &tmQ, q_full, 64, h, m0, b);
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % ST;
        const uint32_t ph = (t / ST) & 1;
        const int n0 = (j_lo + t) * 128;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&k_full[s], 32768);
        tma_load_4d(smem + FwdSmem::K0 + s * 32768, &tmK, &k_full[s], 0, h, n0, b);
        tma_load_4d(smem + FwdSmem::K0 + s * 32768 + 16384, &tmK, &k_full[s], 64, h, n0, b);
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&v_full[s], 32768);
        tma_load_4d(smem + FwdSmem::V0 + s * 32768, &tmV, &v_full[s], 0, h, n0, b);
        tma_load_4d(smem + FwdSmem::V0 + s * 32768 + 16384, &tmV, &v_full[s], 64, h, n0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      const uint32_t sq = smem_u32(smem + FwdSmem::Q);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_s = [&](int t) -> bool {
        const int s = t % ST, sb = t & 1;
        if (!mbar_wait(&k_full[s], (t / ST) & 1, abort_flag)) return false;
        if (!mbar_wait(&s_empty[sb], ((t >> 1) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + FwdSmem::K0 + s * 32768);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = uint32_t(k >> 2) * 16384u + uint32_t(k & 3) * 32u;
          tc_mma_ss(TM_S + sb * 128, make_smem_desc(sq + off, 0, 1024), make_smem_desc(sk + off, 0, 1024), idesc_s, k > 0);
        }
        tc_commit(&k_empty[s]);
        tc_commit(&s_full[sb]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) { ok = issue_s(t + 1); if (!ok) break; }
        const int s = t % ST, pb = t & 1;
        if (!mbar_wait(&p_full[pb], (t >> 1) & 1, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&v_full[s], (t / ST) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sv = smem_u32(smem + FwdSmem::V0 + s * 32768);
        if constexpr (TS) {
#pragma unroll
          for (int k = 0; k < 8; ++k)
            tc_mma_ts(TM_O, TM_P + uint32_t(pb * 64 + k * 8), make_smem_desc(sv + k * 2048, 16384, 1024), idesc_o,
                      (t > 0 || k > 0) ? 1u : 0u);
        } else {
          const uint32_t sp = smem_u32(smem + FwdSmem::P0 + pb * 32768);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t aoff = uint32_t(k >> 2) * 16384u + uint32_t(k & 3) * 32u;
            tc_mma_ss(TM_O, make_smem_desc(sp + aoff, 0, 1024), make_smem_desc(sv + k * 2048, 16384, 1024), idesc_o,
                      (t > 0 || k > 0) ? 1u : 0u);
          }
        }
        tc_commit(&v_empty[s]);
        tc_commit(&p_empty[pb]);
      }
      if (ok) tc_commit(o_done);
    }
  } else {
    // ---------------- softmax / correction / epilogue: thread <-> query row ----------------
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int row = m0 + r;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const float c = p.scale * LOG2E;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int s = t & 1;
      const uint32_t ph = (t >> 1) & 1;
      const int n0 = (j_lo + t) * 128;
      if (!mbar_wait(&s_full[s], ph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      float sc[128];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t v[32];
        tmem_ld32(TM_S + lane_addr + uint32_t(s * 128 + cc * 32), v);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) sc[cc * 32 + j] = __uint_as_float(v[j]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[s]);
      // masks are needed only on tiles that touch the diagonal, the window edge or the tail
      const bool need_mask = (n0 + 127 > m0) || (p.window < p.T && n0 < m0 + 127 - p.window) || (n0 + 127 >= p.T);
      if (need_mask) {
        // the visible keys of a row are one interval [lo, hi] of column indices: one unsigned compare per element
        const int lo = (row < p.T) ? row - p.window - n0 : 128;     // rows past the end see nothing
        const unsigned span = (row < p.T) ? unsigned(p.window) : 0u;  // hi - lo = min(row, T-1) - row + window
#pragma unroll
        for (int j = 0; j < 128; ++j) sc[j] = (unsigned(j - lo) <= span) ? sc[j] : -INFINITY;
      }
      // eight independent chains: one chain of 127 dependent max operations cost 400 clk per tile
#ifndef ARB_FWD_MAX_CHAINS
#define ARB_FWD_MAX_CHAINS 8
#endif
      float mxa[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) mxa[j] = sc[j];
#pragma unroll
      for (int j = 8; j < 128; ++j) mxa[j % ARB_FWD_MAX_CHAINS] = fmaxf(mxa[j % ARB_FWD_MAX_CHAINS], sc[j]);
      const float mx = fmaxf(fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])), fmaxf(fmaxf(mxa[4], mxa[5]), fmaxf(mxa[6], mxa[7])));
      const float m_new = fmaxf(m_used, mx);
      bool resc = false;
      if (m_used == -INFINITY) m_used = m_new;            // nothing accumulated for this row yet
      else resc = (m_new - m_used) * c > 8.f;
      if (t > 0 && __any_sync(0xffffffffu, resc)) {
        // O must not be in flight: PV of the previous tile has to be complete.
        const int sp = (t - 1) & 1;
        if (!mbar_wait(&p_empty[sp], ((t - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
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
        tc_fence_before();
      }
      const float mc = (m_used == -INFINITY) ? 0.f : m_used * c;
      // P buffer s was last read by the PV MMA of tile t-2
      if (t >= 2 && !mbar_wait(&p_empty[s], ((t - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
      float rs = 0.f;
      float rsa[4] = {0.f, 0.f, 0.f, 0.f};
      if constexpr (TS) {
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {   // 64 keys -> 32 packed columns
          uint32_t pk[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            // the ex2 unit (4 lanes per clock and scheduler) is the bound of this loop: ARB_FWD_POLY_OF_8 of every
            // eight exponentials are evaluated as a cubic on the FMA pipe instead
            const float x0 = sc[hf * 64 + 2 * j] * c - mc, x1 = sc[hf * 64 + 2 * j + 1] * c - mc;
            const float e0 = ((2 * j) & 7) < ARB_FWD_POLY_OF_8 ? poly_exp2(x0) : fast_exp2(x0);
            const float e1 = ((2 * j + 1) & 7) < ARB_FWD_POLY_OF_8 ? poly_exp2(x1) : fast_exp2(x1);
            rsa[j & 3] += e0 + e1;
            pk[j] = pack_bf16(e0, e1);
          }
          tmem_st32(TM_P + lane_addr + uint32_t(s * 64 + hf * 32), pk);
        }
        rs = (rsa[0] + rsa[1]) + (rsa[2] + rsa[3]);
        tmem_wait_st();
        tc_fence_before();
      } else {
        const uint32_t pbase = smem_u32(smem + FwdSmem::P0 + s * 32768);
#pragma unroll
        for (int j = 0; j < 128; j += 8) {
          float e[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) { e[u] = fast_exp2(sc[j + u] * c - mc); rs += e[u]; }
          uint4 pk;
          pk.x = pack_bf16(e[0], e[1]); pk.y = pack_bf16(e[2], e[3]); pk.z = pack_bf16(e[4], e[5]); pk.w = pack_bf16(e[6], e[7]);
          st_sw128(pbase, 128, r, j, pk);
        }
        fence_proxy_async_smem();
      }
      l += rs;
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[s]);
    }
    if (ok && mbar_wait(o_done, 0, abort_flag)) {
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

// ===============================================================================================
// Backward.  Both kernels stream 64-row sub-tiles through a 4-stage TMA ring, keep two TMEM
// buffers for the score / dP accumulators (the MMAs of sub-tile t+1 run while the softmax warps
// work on sub-tile t) and stage the bf16 P / dS operands of the output MMAs in swizzled smem.
// ===============================================================================================
constexpr int BWD_STAGES = 4;

// p = exp2(s*c - lse2), ds = p * (dp - delta) for 32 columns of one row; results packed
// to bf16 pairs.  ROWSTAT: lse2/delta are per-row scalars (dQ kernel); otherwise per-column
// arrays (dK/dV kernel, transposed scores).
template <bool MASK, bool ROWSTAT, bool WANT_P>
__device__ __forceinline__ void bwd_chunk(const uint32_t (&sv)[32], const uint32_t (&dv)[32], float c, float scale,
                                          float row_lse2, float row_dl, const float* col_lse2, const float* col_dl,
                                          int row_idx, int col0, int window, int T, bool row_is_query,
                                          uint32_t* p_pk, uint32_t* ds_pk) {
  float pr[32], ds[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float l2 = ROWSTAT ? row_lse2 : col_lse2[j];
    const float dl = ROWSTAT ? row_dl : col_dl[j];
    float e = fast_exp2(__uint_as_float(sv[j]) * c - l2);
    if (MASK) {
      const int qi = row_is_query ? row_idx : col0 + j;
      const int ki = row_is_query ? col0 + j : row_idx;
      const bool vis = (ki <= qi) && (ki >= qi - window) && (qi < T) && (ki < T);
      e = vis ? e : 0.f;
    }
    pr[j] = e;
    ds[j] = e * (__uint_as_float(dv[j]) - dl);   // the 1/sqrt(hd) factor is applied once, to dQ / dK
  }
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    if (WANT_P) p_pk[j >> 1] = pack_bf16(pr[j], pr[j + 1]);
    ds_pk[j >> 1] = pack_bf16(ds[j], ds[j + 1]);
  }
}

struct DqSmem {
  static constexpr int Q = 0, DO = 32768;
  static constexpr int KV0 = 65536;                          // BWD_STAGES x (K_sub 16 KB + V_sub 16 KB)
  static constexpr int DS = KV0 + BWD_STAGES * 32768;        // 16 KB  dS [128 q x 64 keys]
  static constexpr int BAR = DS + 16384;
  static constexpr int TOTAL = BAR + 256 + 1024;
};

template <bool TS>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dq_k(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const AttnArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DqSmem::BAR);
  uint64_t* q_full = bars;                          // Q + dO
  uint64_t* kv_full = bars + 1;                     // [4]
  uint64_t* k_empty = kv_full + BWD_STAGES;         // [4] released by the dQ MMA
  uint64_t* v_empty = k_empty + BWD_STAGES;         // [4] released by the dP MMA
  uint64_t* sd_full = v_empty + BWD_STAGES;         // [2]
  uint64_t* sd_empty = sd_full + 2;                 // [2]
  uint64_t* ds_full = sd_empty + 2;                 // [2] (SS uses [0] only)
  uint64_t* ds_empty = ds_full + 2;                 // [2]
  uint64_t* done = ds_empty + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_mt = (p.T + 127) / 128;
  const int mt = n_mt - 1 - int(blockIdx.x);
  const int h = blockIdx.y, b = blockIdx.z;
  const int m0 = mt * 128;
  const int j_lo = (p.window >= p.T) ? 0 : max(0, (m0 - p.window) / 64);
  const int j_hi = min((p.T - 1) / 64, (m0 + 127) / 64);
  const int n_sub = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < BWD_STAGES; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sd_full[i], 1); mbar_init(&sd_empty[i], 4); }
    for (int i = 0; i < 2; ++i) { mbar_init(&ds_full[i], 4); mbar_init(&ds_empty[i], 1); }
    mbar_init(done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // S[2] x 64, dP[2] x 64, dQ 128, dS[2] x 32 (bf16 pairs; TS only)
  const uint32_t TM_S = tmem, TM_DP = tmem + 128, TM_DQ = tmem + 256, TM_DS = tmem + 384;
  // dS hand-off: TS double-buffers it in TMEM, SS has one shared-memory buffer
  auto ds_buf = [](int t) { return TS ? (t & 1) : 0; };
  auto ds_phase = [](int t) -> uint32_t { return TS ? uint32_t((t >> 1) & 1) : uint32_t(t & 1); };
  constexpr int DS_BUFS = TS ? 2 : 1;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
      mbar_expect_tx(q_full, 65536);
      tma_load_4d(smem + DqSmem::Q, &tmQ, q_full, 0, h, m0, b);
      tma_load_4d(smem + DqSmem::Q + 16384, &tmQ, q_full, 64, h, m0, b);
      tma_load_4d(smem + DqSmem::DO, &tmDO, q_full, 0, h, m0, b);
      tma_load_4d(smem + DqSmem::DO + 16384, &tmDO, q_full, 64, h, m0, b);
      for (int t = 0; t < n_sub; ++t) {
        const int s = t % BWD_STAGES;
        const uint32_t ph = (t / BWD_STAGES) & 1;
        const int n0 = (j_lo + t) * 64;
        if (!mbar_wait(&k_empty[s], ph ^ 1, abort_flag)) break;
        if (!mbar_wait(&v_empty[s], ph ^ 1, abort_flag)) break;
        uint8_t* st = smem + DqSmem::KV0 + s * 32768;
        mbar_expect_tx(&kv_full[s], 32768);
        tma_load_4d(st, &tmK, &kv_full[s], 0, h, n0, b);
        tma_load_4d(st + 8192, &tmK, &kv_full[s], 64, h, n0, b);
        tma_load_4d(st + 16384, &tmV, &kv_full[s], 0, h, n0, b);
        tma_load_4d(st + 24576, &tmV, &kv_full[s], 64, h, n0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      const uint32_t sq = smem_u32(smem + DqSmem::Q), sdo = smem_u32(smem + DqSmem::DO);
      const uint32_t sds = smem_u32(smem + DqSmem::DS);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_sd = [&](int t) -> bool {
        const int s = t % BWD_STAGES, buf = t & 1;
        if (!mbar_wait(&kv_full[s], (t / BWD_STAGES) & 1, abort_flag)) return false;
        if (!mbar_wait(&sd_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + DqSmem::KV0 + s * 32768), sv = sk + 16384;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t aoff = uint32_t(k >> 2) * 16384u + uint32_t(k & 3) * 32u;
          const uint32_t boff = uint32_t(k >> 2) * 8192u + uint32_t(k & 3) * 32u;
          tc_mma_ss(TM_S + buf * 64, make_smem_desc(sq + aoff, 0, 1024), make_smem_desc(sk + boff, 0, 1024), idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t aoff = uint32_t(k >> 2) * 16384u + uint32_t(k & 3) * 32u;
          const uint32_t boff = uint32_t(k >> 2) * 8192u + uint32_t(k & 3) * 32u;
          tc_mma_ss(TM_DP + buf * 64, make_smem_desc(sdo + aoff, 0, 1024), make_smem_desc(sv + boff, 0, 1024), idesc_s, k > 0);
        }
        tc_commit(&v_empty[s]);
        tc_commit(&sd_full[buf]);
        return true;
      };
      if (ok) ok = issue_sd(0);
      for (int t = 0; t < n_sub && ok; ++t) {
        if (t + 1 < n_sub) { ok = issue_sd(t + 1); if (!ok) break; }
        const int s = t % BWD_STAGES;
        if (!mbar_wait(&ds_full[ds_buf(t)], ds_phase(t), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sk = smem_u32(smem + DqSmem::KV0 + s * 32768);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if constexpr (TS)
            tc_mma_ts(TM_DQ, TM_DS + uint32_t(ds_buf(t) * 32 + k * 8), make_smem_desc(sk + k * 2048, 8192, 1024), idesc_o,
                      (t > 0 || k > 0) ? 1u : 0u);
          else
            tc_mma_ss(TM_DQ, make_smem_desc(sds + k * 32, 0, 1024), make_smem_desc(sk + k * 2048, 8192, 1024), idesc_o,
                      (t > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&k_empty[s]);
        tc_commit(&ds_empty[ds_buf(t)]);
      }
      if (ok) tc_commit(done);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int row = m0 + r;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const float c = p.scale * LOG2E;
    const long long stat = ((long long)b * p.H + h) * p.T + row;
    const float lse2 = (row < p.T) ? p.lse[stat] * LOG2E : INFINITY;
    const float dlt = (row < p.T) ? p.delta[stat] : 0.f;
    const uint32_t dsbase = smem_u32(smem + DqSmem::DS);
    bool ok = true;
    for (int t = 0; t < n_sub && ok; ++t) {
      const int n0 = (j_lo + t) * 64;
      const int buf = t & 1;
      if (!mbar_wait(&sd_full[buf], (t >> 1) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = (n0 + 63 > m0) || (p.window < p.T && n0 < m0 + 127 - p.window) || (n0 + 63 >= p.T) || (m0 + 127 >= p.T);
      uint32_t ds_pk[32];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t sv[32], dv[32];
        tmem_ld32(TM_S + lane_addr + uint32_t(buf * 64 + cc * 32), sv);
        tmem_ld32(TM_DP + lane_addr + uint32_t(buf * 64 + cc * 32), dv);
        tmem_wait_ld();
        if (need_mask) bwd_chunk<true, true, false>(sv, dv, c, p.scale, lse2, dlt, nullptr, nullptr, row, n0 + cc * 32, p.window, p.T, true, nullptr, ds_pk + cc * 16);
        else bwd_chunk<false, true, false>(sv, dv, c, p.scale, lse2, dlt, nullptr, nullptr, row, n0 + cc * 32, p.window, p.T, true, nullptr, ds_pk + cc * 16);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sd_empty[buf]);
      // the dQ MMA that last read this dS buffer (sub-tile t - DS_BUFS) has to be complete
      if (t >= DS_BUFS && !mbar_wait(&ds_empty[ds_buf(t)], ds_phase(t - DS_BUFS), abort_flag)) { ok = false; break; }
      if constexpr (TS) {
        tmem_st32(TM_DS + lane_addr + uint32_t(buf * 32), ds_pk);
        tmem_wait_st();
        tc_fence_before();
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          st_sw128(dsbase, 128, r, j * 8, make_uint4(ds_pk[j * 4], ds_pk[j * 4 + 1], ds_pk[j * 4 + 2], ds_pk[j * 4 + 3]));
        fence_proxy_async_smem();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[ds_buf(t)]);
    }
    if (ok && mbar_wait(done, 0, abort_flag)) {
      tc_fence_after();
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + ((long long)b * p.T + row) * p.ldo + h * HD;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t v[32];
        tmem_ld32(TM_DQ + lane_addr + uint32_t(cc * 32), v);
        tmem_wait_ld();
        if (row < p.T) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 u;
            const float sc = p.scale;
            u.x = pack_bf16(__uint_as_float(v[j]) * sc, __uint_as_float(v[j + 1]) * sc);
            u.y = pack_bf16(__uint_as_float(v[j + 2]) * sc, __uint_as_float(v[j + 3]) * sc);
            u.z = pack_bf16(__uint_as_float(v[j + 4]) * sc, __uint_as_float(v[j + 5]) * sc);
            u.w = pack_bf16(__uint_as_float(v[j + 6]) * sc, __uint_as_float(v[j + 7]) * sc);
            *reinterpret_cast<uint4*>(orow + cc * 32 + j) = u;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, ERR_ATTN_TIMEOUT);
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// -----------------------------------------------------------------------------------------------
// dK / dV: key-stationary, transposed scores (TMEM lane = key, column = query).
// -----------------------------------------------------------------------------------------------
struct DkvSmem {
  static constexpr int K = 0, V = 32768;
  static constexpr int QD0 = 65536;                          // BWD_STAGES x (Q_sub 16 KB + dO_sub 16 KB)
  static constexpr int PT = QD0 + BWD_STAGES * 32768;        // 16 KB  P^T  [128 keys x 64 q]
  static constexpr int DST = PT + 16384;                     // 16 KB  dS^T
  static constexpr int STAT = DST + 16384;                   // lse2[2][64], delta[2][64]
  static constexpr int BAR = STAT + 1024;
  static constexpr int TOTAL = BAR + 256 + 1024;
};

// TS: P^T and dS^T (bf16 pairs, 32 columns each) overwrite the first half of the S^T / dP^T
// buffer they were computed from; every thread overwrites only its own lane after reading it.  The
// S^T / dP^T MMAs of sub-tile t+2 reuse those columns and are issued after the dV / dK MMAs of
// sub-tile t (MMAs of one thread execute in issue order), which in turn are issued only after the
// softmax warps have signalled pd_full(t); no separate "empty" barriers are needed.
template <bool TS>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dkv_k(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const AttnArgs p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DkvSmem::BAR);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;                      // [4]
  uint64_t* q_empty = q_full + BWD_STAGES;          // [4] released by the dV/dK MMAs
  uint64_t* sd_full = q_empty + BWD_STAGES;         // [2]
  uint64_t* sd_empty = sd_full + 2;                 // [2]
  uint64_t* pd_full = sd_empty + 2;                 // [2] (SS uses [0] only)
  uint64_t* pd_empty = pd_full + 2;
  uint64_t* done = pd_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat_lse = reinterpret_cast<float*>(smem + DkvSmem::STAT);   // [2][64]
  float* stat_dl = stat_lse + 128;                                     // [2][64]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int n0 = int(blockIdx.x) * 128;
  const int i_lo = n0 / 64;
  const long long last_q = (p.window >= p.T) ? (long long)(p.T - 1) : min((long long)(p.T - 1), (long long)n0 + 127 + p.window);
  const int i_hi = int(last_q / 64);
  const int n_sub = i_hi - i_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < BWD_STAGES; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sd_full[i], 1); mbar_init(&sd_empty[i], 4); }
    mbar_init(&pd_full[0], 4); mbar_init(&pd_full[1], 4); mbar_init(pd_empty, 1); mbar_init(done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t TM_S = tmem, TM_DP = tmem + 128, TM_DV = tmem + 256, TM_DK = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
      mbar_expect_tx(kv_full, 65536);
      tma_load_4d(smem + DkvSmem::K, &tmK, kv_full, 0, h, n0, b);
      tma_load_4d(smem + DkvSmem::K + 16384, &tmK, kv_full, 64, h, n0, b);
      tma_load_4d(smem + DkvSmem::V, &tmV, kv_full, 0, h, n0, b);
      tma_load_4d(smem + DkvSmem::V + 16384, &tmV, kv_full, 64, h, n0, b);
      for (int t = 0; t < n_sub; ++t) {
        const int s = t % BWD_STAGES;
        const uint32_t ph = (t / BWD_STAGES) & 1;
        const int q0 = (i_lo + t) * 64;
        if (!mbar_wait(&q_empty[s], ph ^ 1, abort_flag)) break;
        uint8_t* st = smem + DkvSmem::QD0 + s * 32768;
        mbar_expect_tx(&q_full[s], 32768);
        tma_load_4d(st, &tmQ, &q_full[s], 0, h, q0, b);
        tma_load_4d(st + 8192, &tmQ, &q_full[s], 64, h, q0, b);
        tma_load_4d(st + 16384, &tmDO, &q_full[s], 0, h, q0, b);
        tma_load_4d(st + 24576, &tmDO, &q_full[s], 64, h, q0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, 128, false, true);
      const uint32_t sk = smem_u32(smem + DkvSmem::K), sv = smem_u32(smem + DkvSmem::V);
      const uint32_t spt = smem_u32(smem + DkvSmem::PT), sdst = smem_u32(smem + DkvSmem::DST);
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      auto issue_sd = [&](int t) -> bool {
        const int s = t % BWD_STAGES, buf = t & 1;
        if (!mbar_wait(&q_full[s], (t / BWD_STAGES) & 1, abort_flag)) return false;
        if (!TS && !mbar_wait(&sd_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sq = smem_u32(smem + DkvSmem::QD0 + s * 32768), sdo = sq + 16384;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t aoff = uint32_t(k >> 2) * 16384u + uint32_t(k & 3) * 32u;
          const uint32_t boff = uint32_t(k >> 2) * 8192u + uint32_t(k & 3) * 32u;
          tc_mma_ss(TM_S + buf * 64, make_smem_desc(sk + aoff, 0, 1024), make_smem_desc(sq + boff, 0, 1024), idesc_s, k > 0);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t aoff = uint32_t(k >> 2) * 16384u + uint32_t(k & 3) * 32u;
          const uint32_t boff = uint32_t(k >> 2) * 8192u + uint32_t(k & 3) * 32u;
          tc_mma_ss(TM_DP + buf * 64, make_smem_desc(sv + aoff, 0, 1024), make_smem_desc(sdo + boff, 0, 1024), idesc_s, k > 0);
        }
        tc_commit(&sd_full[buf]);
        return true;
      };
      if (ok) ok = issue_sd(0);
      for (int t = 0; t < n_sub && ok; ++t) {
        if (t + 1 < n_sub) { ok = issue_sd(t + 1); if (!ok) break; }
        const int s = t % BWD_STAGES;
        if (!mbar_wait(&pd_full[TS ? (t & 1) : 0], TS ? uint32_t((t >> 1) & 1) : uint32_t(t & 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sq = smem_u32(smem + DkvSmem::QD0 + s * 32768), sdo = sq + 16384;
        const uint32_t acc = (t > 0) ? 1u : 0u;
        if constexpr (TS) {
          const uint32_t buf = uint32_t(t & 1);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_ts(TM_DV, TM_S + buf * 64 + k * 8, make_smem_desc(sdo + k * 2048, 8192, 1024), idesc_o, k > 0 ? 1u : acc);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_ts(TM_DK, TM_DP + buf * 64 + k * 8, make_smem_desc(sq + k * 2048, 8192, 1024), idesc_o, k > 0 ? 1u : acc);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_ss(TM_DV, make_smem_desc(spt + k * 32, 0, 1024), make_smem_desc(sdo + k * 2048, 8192, 1024), idesc_o, k > 0 ? 1u : acc);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma_ss(TM_DK, make_smem_desc(sdst + k * 32, 0, 1024), make_smem_desc(sq + k * 2048, 8192, 1024), idesc_o, k > 0 ? 1u : acc);
        }
        tc_commit(&q_empty[s]);
        if (!TS) tc_commit(pd_empty);
      }
      if (ok) tc_commit(done);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;         // key row inside the tile
    const int key = n0 + r;
    const int tid = threadIdx.x - 64;    // 0..127
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const float c = p.scale * LOG2E;
    const uint32_t ptbase = smem_u32(smem + DkvSmem::PT), dstbase = smem_u32(smem + DkvSmem::DST);
    const long long stat0 = ((long long)b * p.H + h) * p.T;
    auto load_stat = [&](int t) -> float {   // thread tid < 64: lse2 of query tid; else delta of query tid-64
      const int qi = (i_lo + t) * 64 + (tid & 63);
      if (t >= n_sub || qi >= p.T) return (tid < 64) ? INFINITY : 0.f;
      return (tid < 64) ? p.lse[stat0 + qi] * LOG2E : p.delta[stat0 + qi];
    };
    {
      const float v0 = load_stat(0);
      (tid < 64 ? stat_lse : stat_dl)[tid & 63] = v0;
    }
    bool ok = true;
    for (int t = 0; t < n_sub; ++t) {
      const int q0 = (i_lo + t) * 64;
      const int buf = t & 1;
      named_bar_sync(1, 128);                   // statistics of sub-tile t are visible
      const float next_stat = load_stat(t + 1);  // in flight while this sub-tile is processed
      if (ok && !mbar_wait(&sd_full[buf], (t >> 1) & 1, abort_flag)) ok = false;
      if (ok) {
        tc_fence_after();
        const bool need_mask = (q0 < n0 + 127) || (p.window < p.T && q0 + 63 > n0 + p.window) || (q0 + 63 >= p.T) || (n0 + 127 >= p.T);
        uint32_t p_pk[32], ds_pk[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t sv[32], dv[32];
          tmem_ld32(TM_S + lane_addr + uint32_t(buf * 64 + cc * 32), sv);
          tmem_ld32(TM_DP + lane_addr + uint32_t(buf * 64 + cc * 32), dv);
          tmem_wait_ld();
          const float* cl = stat_lse + buf * 64 + cc * 32;
          const float* cd = stat_dl + buf * 64 + cc * 32;
          if (need_mask) bwd_chunk<true, false, true>(sv, dv, c, p.scale, 0.f, 0.f, cl, cd, key, q0 + cc * 32, p.window, p.T, false, p_pk + cc * 16, ds_pk + cc * 16);
          else bwd_chunk<false, false, true>(sv, dv, c, p.scale, 0.f, 0.f, cl, cd, key, q0 + cc * 32, p.window, p.T, false, p_pk + cc * 16, ds_pk + cc * 16);
        }
        if constexpr (TS) {
          tmem_st32(TM_S + lane_addr + uint32_t(buf * 64), p_pk);
          tmem_st32(TM_DP + lane_addr + uint32_t(buf * 64), ds_pk);
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&pd_full[buf]);
        } else {
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sd_empty[buf]);
          if (t >= 1 && !mbar_wait(pd_empty, (t - 1) & 1, abort_flag)) ok = false;
          if (ok) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              st_sw128(ptbase, 128, r, j * 8, make_uint4(p_pk[j * 4], p_pk[j * 4 + 1], p_pk[j * 4 + 2], p_pk[j * 4 + 3]));
              st_sw128(dstbase, 128, r, j * 8, make_uint4(ds_pk[j * 4], ds_pk[j * 4 + 1], ds_pk[j * 4 + 2], ds_pk[j * 4 + 3]));
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(&pd_full[0]);
          }
        }
      }
      (tid < 64 ? stat_lse : stat_dl)[((t + 1) & 1) * 64 + (tid & 63)] = next_stat;
    }
    if (ok && mbar_wait(done, 0, abort_flag)) {
      tc_fence_after();
      __nv_bfloat16* dkrow = reinterpret_cast<__nv_bfloat16*>(p.dk) + ((long long)b * p.T + key) * p.lddk + h * HD;
      __nv_bfloat16* dvrow = reinterpret_cast<__nv_bfloat16*>(p.dv) + ((long long)b * p.T + key) * p.lddv + h * HD;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t v[32];
          tmem_ld32((which ? TM_DK : TM_DV) + lane_addr + uint32_t(cc * 32), v);
          tmem_wait_ld();
          if (key < p.T) {
            __nv_bfloat16* dst = (which ? dkrow : dvrow) + cc * 32;
            const float sc = which ? p.scale : 1.f;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 u;
              u.x = pack_bf16(__uint_as_float(v[j]) * sc, __uint_as_float(v[j + 1]) * sc);
              u.y = pack_bf16(__uint_as_float(v[j + 2]) * sc, __uint_as_float(v[j + 3]) * sc);
              u.z = pack_bf16(__uint_as_float(v[j + 4]) * sc, __uint_as_float(v[j + 5]) * sc);
              u.w = pack_bf16(__uint_as_float(v[j + 6]) * sc, __uint_as_float(v[j + 7]) * sc);
              *reinterpret_cast<uint4*>(dst + j) = u;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, ERR_ATTN_TIMEOUT);
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem, 512); }
}

// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one warp per token, a half-warp per head (16-byte loads, two heads
// per iteration), the token arithmetic done once per warp
__global__ void __launch_bounds__(256) attn_delta_k(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                                    float* __restrict__ delta, int B, int T, int H, long long ldo, long long lddo) {
  const long long bt = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (bt >= (long long)B * T) return;
  const int t = int(bt % T);
  const int b = int(bt / T);
  const int sub = lane >> 4, l16 = lane & 15;
  for (int h0 = 0; h0 < H; h0 += 2) {
    const int h = h0 + sub;
    float acc = 0.f;
    if (h < H) {
      const uint4 a = *reinterpret_cast<const uint4*>(o + bt * ldo + h * HD + l16 * 8);
      const uint4 g = *reinterpret_cast<const uint4*>(d_o + bt * lddo + h * HD + l16 * 8);
      const uint32_t aa[4] = {a.x, a.y, a.z, a.w}, gg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 x = unpack_bf16(aa[k]), y = unpack_bf16(gg[k]);
        acc += x.x * y.x + x.y * y.y;
      }
    }
#pragma unroll
    for (int s = 8; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
    if (l16 == 0 && h < H) delta[((long long)b * H + h) * T + t] = acc;
  }
}

}  // namespace arb

using namespace arb;

// 4: as 2 with the register-split forward (attn_fwd3_sm100.cu) for every shape; 3: as 2 with the two-query-tile forward
// for every shape; 2 (default): wide backward, forward chosen by shape (see arb_attn_fwd); 1: 64-wide sub-tiles with TMEM
// operands; 0: with shared-memory operands
static int g_attn_mode = 2;
static int g_attn_ts = 1;
extern "C" void arb_attn_set_mode(int mode) { g_attn_mode = mode < 0 ? 0 : (mode > 4 ? 4 : mode); g_attn_ts = g_attn_mode ? 1 : 0; }

template <bool TS>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a, dim3 grid,
                      cudaStream_t stream) {
  static PerDeviceOnce cfg;
  int r;
  if (cfg.first()) { if ((r = set_smem(attn_fwd_k<TS>, FwdSmemT<TS>::TOTAL))) return r; }
  attn_fwd_k<TS><<<grid, ATT_THREADS, FwdSmemT<TS>::TOTAL, stream>>>(tq, tk, tv, a);
  return int(cudaGetLastError());
}
template <bool TS>
static int launch_dq(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                     const AttnArgs& a, dim3 grid, cudaStream_t stream) {
  static PerDeviceOnce cfg;
  int r;
  if (cfg.first()) { if ((r = set_smem(attn_bwd_dq_k<TS>, DqSmem::TOTAL))) return r; }
  attn_bwd_dq_k<TS><<<grid, ATT_THREADS, DqSmem::TOTAL, stream>>>(tq, tk, tv, tdo, a);
  return int(cudaGetLastError());
}
template <bool TS>
static int launch_dkv(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                      const AttnArgs& a, dim3 grid, cudaStream_t stream) {
  static PerDeviceOnce cfg;
  int r;
  if (cfg.first()) { if ((r = set_smem(attn_bwd_dkv_k<TS>, DkvSmem::TOTAL))) return r; }
  attn_bwd_dkv_k<TS><<<grid, ATT_THREADS, DkvSmem::TOTAL, stream>>>(tq, tk, tv, tdo, a);
  return int(cudaGetLastError());
}

extern "C" int arb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int H,
                            long long ldq, long long ldk, long long ldv, long long ldo, int window, float scale,
                            int* err_flag, cudaStream_t stream) {
  if (B <= 0 || T <= 0 || H <= 0 || window < 0) return -3;
  if (bad_ptr(q) || bad_ptr(k) || bad_ptr(v) || bad_ptr(o) || (ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8)) return -4;
  if (H > 65535 || B > 65535) return -3;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_qkv_tmap(&tq, q, B, T, H, ldq, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tk, k, B, T, H, ldk, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tv, v, B, T, H, ldv, 128))) return 1000 + r;
  AttnArgs a{};
  a.B = B; a.T = T; a.H = H; a.window = window > T ? T : window; a.scale = scale;
  a.o = o; a.ldo = ldo; a.lse = lse; a.err = err_flag;
  // Two query tiles per CTA pay on grids of several waves (B=4, H=8, T=32768, ms one tile / two tiles: full causal
  // 9.79 / 9.42, window 4096 2.61 / 2.50, window 256 0.51 / 0.47) and lose on small grids, where halving the CTA count
  // costs more than the shared K / V loads save, and on short sequences.  Of the two-tile kernels the register-split
  // one (attn_fwd3) is the default: 4-5 % faster than attn_fwd2 on the same shapes (full causal 8.95 -> 8.54 ms,
  // window 4096 2.13 -> 2.04, window 256 0.471 -> 0.458; B=8, H=16, T=8192 full 2.38 -> 2.27).
  const long long pair_ctas = (long long)((T + 255) / 256) * H * B;
  if (g_attn_mode == 4 || (g_attn_mode == 2 && pair_ctas >= 2048 && T >= 4096))
    return attn_fwd3_launch(q, k, v, ldq, ldk, ldv, a, stream);
  if (g_attn_mode == 3) return attn_fwd2_launch(q, k, v, ldq, ldk, ldv, a, stream);
  dim3 grid((T + 127) / 128, H, B);
  return g_attn_ts ? launch_fwd<true>(tq, tk, tv, a, grid, stream) : launch_fwd<false>(tq, tk, tv, a, grid, stream);
}

extern "C" int arb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                            void* dq, void* dk, void* dv, float* delta, float* dq_accum, int B, int T, int H,
                            long long ldq, long long ldk, long long ldv, long long ldo, long long lddo, long long lddq,
                            long long lddk, long long lddv, int window, float scale, int* err_flag, cudaStream_t stream) {
  (void)dq_accum;  // the two-kernel backward needs no fp32 dQ accumulator
  if (B <= 0 || T <= 0 || H <= 0 || window < 0 || H > 65535 || B > 65535) return -3;
  if (bad_ptr(q) || bad_ptr(k) || bad_ptr(v) || bad_ptr(o) || bad_ptr(d_o) || bad_ptr(dq) || bad_ptr(dk) || bad_ptr(dv)) return -4;
  if ((ldq % 8) || (ldk % 8) || (ldv % 8) || (ldo % 8) || (lddo % 8) || (lddq % 8) || (lddk % 8) || (lddv % 8)) return -4;
  int r;
  attn_delta_k<<<unsigned(((long long)B * T + 7) / 8), 256, 0, stream>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, B, T, H, ldo, lddo);
  if ((r = int(cudaGetLastError()))) return r;
  AttnArgs a{};
  a.B = B; a.T = T; a.H = H; a.window = window > T ? T : window; a.scale = scale;
  a.lse = const_cast<float*>(lse); a.delta = delta; a.err = err_flag;
  if (g_attn_mode >= 2)
    return attn_wide_bwd_launch(q, k, v, d_o, dq, dk, dv, ldq, ldk, ldv, lddo, lddq, lddk, lddv, a, stream);
  {
    CUtensorMap tq, tk, tv, tdo;
    if ((r = make_qkv_tmap(&tq, q, B, T, H, ldq, 128))) return 1000 + r;
    if ((r = make_qkv_tmap(&tk, k, B, T, H, ldk, 64))) return 1000 + r;
    if ((r = make_qkv_tmap(&tv, v, B, T, H, ldv, 64))) return 1000 + r;
    if ((r = make_qkv_tmap(&tdo, d_o, B, T, H, lddo, 128))) return 1000 + r;
    a.o = dq; a.ldo = lddq;
    dim3 grid((T + 127) / 128, H, B);
    if ((r = g_attn_ts ? launch_dq<true>(tq, tk, tv, tdo, a, grid, stream) : launch_dq<false>(tq, tk, tv, tdo, a, grid, stream))) return r;
  }
  {
    CUtensorMap tq, tk, tv, tdo;
    if ((r = make_qkv_tmap(&tq, q, B, T, H, ldq, 64))) return 1000 + r;
    if ((r = make_qkv_tmap(&tk, k, B, T, H, ldk, 128))) return 1000 + r;
    if ((r = make_qkv_tmap(&tv, v, B, T, H, ldv, 128))) return 1000 + r;
    if ((r = make_qkv_tmap(&tdo, d_o, B, T, H, lddo, 64))) return 1000 + r;
    a.dk = dk; a.dv = dv; a.lddk = lddk; a.lddv = lddv;
    dim3 grid((T + 127) / 128, H, B);
    if ((r = g_attn_ts ? launch_dkv<true>(tq, tk, tv, tdo, a, grid, stream) : launch_dkv<false>(tq, tk, tv, tdo, a, grid, stream))) return r;
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the backward (see attn_noalloc.h): the delta scratch is a
// file-scope device array.  In host code the array's name is only a handle; its device address
// comes from cudaGetSymbolAddress, once per device, with that device current.
// ---------------------------------------------------------------------------------------------
#include "attn_noalloc.h"

#include <atomic>

static __device__ __align__(256) float g_attn_noalloc_delta[ARB_ATTN_NOALLOC_MAX_ROWS];

extern "C" int arb_attn_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                    const float* lse, void* dq, void* dk, void* dv, int B, int T, int H,
                                    long long ldq, long long ldk, long long ldv, long long ldo, long long lddo,
                                    long long lddq, long long lddk, long long lddv, int window, float scale,
                                    int* err_flag, cudaStream_t stream) {
  constexpr int MAX_DEVICES = 64;
  // one slot per device; atomic, so that two host threads making their first call on a device at the same
  // time both end up with the (identical) address without a data race
  static std::atomic<float*> scratch_of_device[MAX_DEVICES];
  if (B <= 0 || T <= 0 || H <= 0) return -3;
  if ((long long)B * T * H > (long long)ARB_ATTN_NOALLOC_MAX_ROWS) return ARB_ERR_NOALLOC_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return ARB_ERR_NOALLOC_SYMBOL;
  float* scratch = scratch_of_device[dev].load(std::memory_order_acquire);
  if (scratch == nullptr) {
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&scratch), g_attn_noalloc_delta);
    if (e != cudaSuccess || scratch == nullptr) return ARB_ERR_NOALLOC_SYMBOL;
    scratch_of_device[dev].store(scratch, std::memory_order_release);
  }
  return arb_attn_bwd(q, k, v, o, d_o, lse, dq, dk, dv, scratch, nullptr, B, T, H, ldq, ldk, ldv, ldo,
                      lddo, lddq, lddk, lddv, window, scale, err_flag, stream);
}
