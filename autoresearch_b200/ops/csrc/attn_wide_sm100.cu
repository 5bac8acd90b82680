// Flash attention backward for head_dim = 128 with 128 x 128 score tiles and a two-phase softmax.
//
// What bounds these kernels on sm_100a is not the tensor pipe's arithmetic rate but (a) the cost of
// issuing tcgen05.mma instructions, about 50-65 clk each whatever their size, so every MMA here is
// M=128, N=128, K=16 (64 clk of tensor work), never N=64; and (b) the ex2 unit, 1024 clk per
// 128 x 128 tile, so the exponentials must overlap the MMAs.  Ten warps: TMA producer, MMA issuer, eight
// softmax warps (two per TMEM lane quarter, each owning 64 of the 128 columns of a tile).  Measured dead
// ends, for the record: (1) two issuing threads: the tensor pipe interleaves their instructions and the
// tile the softmax warps wait for finishes later than when one thread queues the work in the order it is
// needed; (2) evaluating part of the exponentials with a polynomial on the FMA pipe: the extra
// instructions take issue slots from the issuing thread, which shares a scheduler with two softmax warps;
// (3) in the dQ kernel, double-buffered scores with dS written over the score tile (one barrier check fewer per
// tile) and, separately, Q and dO held in TMEM as the A operands of S and dP (half the shared-memory operand
// reads): both correct, neither faster, so neither the barrier checks nor shared-memory bandwidth is the bound.
//
// The softmax of a tile is split in two phases so that the score buffer is released early:
//   phase A  needs only S: p = exp2(S*c - lse) is kept in fp32 registers (64 per thread);
//   phase B  needs dP: dS = p * (dP - delta), packed to bf16 and written to TMEM as the A operand
//            of the next MMA.
//
//   attn_bwd_dq_wide_k (query-stationary): per key tile  S = Q K^T, dP = dO V^T, dQ += dS K.
//     MMA order   S(t+1) after phase A(t) has loaded S(t);  dP(t+1), dQ(t) after phase B(t).
//     TMEM        S 128 | dP 128 | dQ 128 | dS[2] x 64 columns.
//   attn_bwd_dkv_wide_k (key-stationary, transposed scores): S^T = K Q^T, dP^T = V dO^T,
//     dV += P^T dO, dK += dS^T Q.
//     MMA order   dV(t), S^T(t+1) after phase A(t);  dK(t), dP^T(t+1) after phase B(t).
//     TMEM        S^T 128 | dP^T 128 | dV 128 | dK 128: full, so P^T / dS^T (bf16 pairs) overwrite
//                 columns of the S^T / dP^T tile they came from.  Each thread overwrites only columns
//                 of its own lane that it has already read, and the MMA that next writes the tile
//                 is issued after the MMA that reads those columns (one thread's MMAs execute in
//                 issue order).
//
// Both are deterministic (no atomics).  Mask semantics as in attn_sm100.cu: key j is visible to
// query i iff i - window <= j <= i (brain/src/forward.rs:1134-1138); the reference runs a
// Hopper-only FlashAttention-3 build for this step (brain/src/backward.rs:613-659).
#include "attn_common.cuh"

namespace arb {

// Shared memory map of both kernels: two resident 32 KB tiles, a three-slot and a two-slot ring of
// 32 KB tiles (every tile is 128 rows x 128 bf16 as two 64-column 128B-swizzled halves).
struct WideSmem {
  static constexpr int RES0 = 0, RES1 = 32768;
  static constexpr int RING3 = 65536;
  static constexpr int RING2 = RING3 + 3 * 32768;
  static constexpr int STAT = RING2 + 2 * 32768;   // lse2[2][128], delta[2][128] (dK/dV kernel)
  static constexpr int BAR = STAT + 4 * 128 * 4;
  static constexpr int TOTAL = BAR + 512;
};
static_assert(WideSmem::TOTAL <= 232448, "exceeds the 227 KB shared memory of one CTA");

// One 128 x 128 x 128 product as eight K=16 MMAs.  A, B K-major tiles (two 16 KB halves).
__device__ __forceinline__ void mma_tile_kk(uint32_t d_tmem, uint32_t sa, uint32_t sb, uint32_t idesc) {
  // one descriptor per operand; a K slice is an add on its low word (start address >> 4)
  const uint32_t hi = uint32_t(make_smem_desc(0, 0, 1024) >> 32);
  const uint32_t al = uint32_t(make_smem_desc(sa, 0, 1024)), bl = uint32_t(make_smem_desc(sb, 0, 1024));
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const uint32_t off = uint32_t(k >> 2) * 1024u + uint32_t(k & 3) * 2u;       // (16 KB half, 32 B slice) >> 4
    tc_mma_ss_lh(d_tmem, al + off, hi, bl + off, hi, idesc, k > 0);
  }
}
// D (+)= A[tmem, 128 x 128 bf16 as two groups of 32 columns] * B[smem tile used MN-major: rows are K]
__device__ __forceinline__ void mma_tile_ts(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t sb, uint32_t idesc,
                                            bool accumulate) {
  const uint32_t hi = uint32_t(make_smem_desc(0, 16384, 1024) >> 32), bl = uint32_t(make_smem_desc(sb, 16384, 1024));
#pragma unroll
  for (int k = 0; k < 8; ++k)
    tc_mma_ts_lh(d_tmem, (k < 4 ? a_lo : a_hi) + uint32_t(k & 3) * 8u, bl + uint32_t(k) * 128u, hi, idesc,
                 (accumulate || k > 0) ? 1u : 0u);
}

// exp2 of 64 scores of one row/lane; the offsets are one per-row value or 64 per-column values
template <bool ROW_STAT>
__device__ __forceinline__ void exp2_64(const uint32_t (&s0)[32], const uint32_t (&s1)[32], float c, float row_off,
                                        const float4* col_off, float (&pr)[64]) {
#pragma unroll
  for (int g = 0; g < 16; ++g) {
    float4 o = make_float4(row_off, row_off, row_off, row_off);
    if (!ROW_STAT) o = col_off[g];
    const float off[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = g * 4 + u;
      const float x = __uint_as_float(j < 32 ? s0[j] : s1[j - 32]) * c - off[u];
      pr[j] = fast_exp2(x);
    }
  }
}

__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&a)[32], uint32_t (&b)[32]) {
  tmem_ld32(taddr, a);
  tmem_ld32(taddr + 32, b);
  tmem_wait_ld();
}

// ===============================================================================================
// dQ
// ===============================================================================================
__global__ void __launch_bounds__(ATT_WIDE_THREADS, 1)
attn_bwd_dq_wide_k(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const AttnArgs p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {   // the swizzled tiles need 1 KB alignment; nothing has been allocated yet
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, ERR_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WideSmem::BAR);
  uint64_t* q_full = bars;            // Q + dO resident
  uint64_t* k_full = bars + 1;        // [3]
  uint64_t* v_full = bars + 4;        // [2]
  uint64_t* s_full = bars + 6;        // S(t) complete
  uint64_t* a_done = bars + 7;        // phase A(t) has read S(t)            (8 arrivals)
  uint64_t* dp_full = bars + 8;       // [2] dP(t) complete; also frees V(t)'s slot
  uint64_t* ds_full = bars + 10;      // [2] phase B(t) wrote dS(t) and has read dP(t) (8 arrivals)
  uint64_t* dq_done = bars + 12;      // [6] dQ(t) MMAs complete: frees K(t)'s slot and dS buffer t&1
  uint64_t* done = bars + 18;         // all dQ MMAs complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_mt = (p.T + 127) / 128;
  const int mt = n_mt - 1 - int(blockIdx.x);   // later query tiles see more keys: schedule them first
  const int h = blockIdx.y, b = blockIdx.z;
  const int m0 = mt * 128;
  const int j_lo = (p.window >= p.T) ? 0 : max(0, (m0 - p.window) / 128);
  const int j_hi = min((p.T - 1) / 128, (m0 + 127) / 128);
  const int n_tiles = j_hi - j_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 3; ++i) mbar_init(&k_full[i], 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&v_full[i], 1); mbar_init(&dp_full[i], 1); mbar_init(&ds_full[i], 8); }
    mbar_init(s_full, 1); mbar_init(a_done, 8);
    for (int i = 0; i < 6; ++i) mbar_init(&dq_done[i], 1);
    mbar_init(done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t TM_S = tmem, TM_DP = tmem + 128, TM_DQ = tmem + 256, TM_DS = tmem + 384;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmDO);
      mbar_expect_tx(q_full, 65536);
      tma_load_4d(smem + WideSmem::RES0, &tmQ, q_full, 0, h, m0, b);
      tma_load_4d(smem + WideSmem::RES0 + 16384, &tmQ, q_full, 64, h, m0, b);
      tma_load_4d(smem + WideSmem::RES1, &tmDO, q_full, 0, h, m0, b);
      tma_load_4d(smem + WideSmem::RES1 + 16384, &tmDO, q_full, 64, h, m0, b);
      // A TMA load takes about 1 us under load, so every tile is requested at least a tile period before its
      // first use: K(t) when dQ(t-3) has released its slot, V(t) when dP(t-2) has.
      for (int t = 0; t < n_tiles; ++t) {
        const int n0 = (j_lo + t) * 128;
        if (t >= 3 && !mbar_wait(&dq_done[(t - 3) % 6], uint32_t((t - 3) / 6) & 1u, abort_flag)) break;
        uint8_t* ks = smem + WideSmem::RING3 + (t % 3) * 32768;
        mbar_expect_tx(&k_full[t % 3], 32768);
        tma_load_4d(ks, &tmK, &k_full[t % 3], 0, h, n0, b);
        tma_load_4d(ks + 16384, &tmK, &k_full[t % 3], 64, h, n0, b);
        if (t >= 2 && !mbar_wait(&dp_full[t & 1], uint32_t((t - 2) >> 1) & 1u, abort_flag)) break;
        uint8_t* vs = smem + WideSmem::RING2 + (t & 1) * 32768;
        mbar_expect_tx(&v_full[t & 1], 32768);
        tma_load_4d(vs, &tmV, &v_full[t & 1], 0, h, n0, b);
        tma_load_4d(vs + 16384, &tmV, &v_full[t & 1], 64, h, n0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_mn = make_idesc_bf16(128, 128, false, true);
      const uint32_t sq = smem_u32(smem + WideSmem::RES0), sdo = smem_u32(smem + WideSmem::RES1);
      const uint32_t sk0 = smem_u32(smem + WideSmem::RING3), sv0 = smem_u32(smem + WideSmem::RING2);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        mma_tile_kk(TM_S, sq, sk0, idesc_kk);
        tc_commit(s_full);
        ok = mbar_wait(&v_full[0], 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        mma_tile_kk(TM_DP, sdo, sv0, idesc_kk);
        tc_commit(&dp_full[0]);
      }
      PROF_DECL();
      for (int t = 0; t < n_tiles && ok; ++t) {
        const bool more = t + 1 < n_tiles;
        PROF_TIC();
        if (more) {
          if (!mbar_wait(a_done, uint32_t(t & 1), abort_flag)) { ok = false; break; }
          if (!mbar_wait(&k_full[(t + 1) % 3], uint32_t((t + 1) / 3) & 1u, abort_flag)) { ok = false; break; }
          PROF_TOC(1);
          tc_fence_after();
          mma_tile_kk(TM_S, sq, sk0 + uint32_t((t + 1) % 3) * 32768u, idesc_kk);
          tc_commit(s_full);
          PROF_TOC(2);
        }
        if (!mbar_wait(&ds_full[t & 1], uint32_t(t >> 1) & 1u, abort_flag)) { ok = false; break; }
        if (more) {
          if (!mbar_wait(&v_full[(t + 1) & 1], uint32_t((t + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
          PROF_TOC(3);
          tc_fence_after();
          mma_tile_kk(TM_DP, sdo, sv0 + uint32_t((t + 1) & 1) * 32768u, idesc_kk);
          tc_commit(&dp_full[(t + 1) & 1]);
          PROF_TOC(4);
        }
        tc_fence_after();
        const uint32_t ds = TM_DS + uint32_t(t & 1) * 64u;
        mma_tile_ts(TM_DQ, ds, ds + 32, sk0 + uint32_t(t % 3) * 32768u, idesc_mn, t > 0);
        tc_commit(&dq_done[t % 6]);
        PROF_TOC(5);
      }
      if (ok) tc_commit(done);
      PROF_DUMP(0);
    }
  } else {
    const int sw = warp - 2;             // 0..7
    const int q = warp & 3;              // TMEM lane quarter this warp may access
    const int hf = sw >> 2;              // column half of the tile owned by this warp
    const int r = q * 32 + lane;
    const int row = m0 + r;
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const float c = p.scale * LOG2E;
    const long long stat = ((long long)b * p.H + h) * p.T + row;
    const float lse2 = (row < p.T) ? p.lse[stat] * LOG2E : INFINITY;
    const float dlt = (row < p.T) ? p.delta[stat] : 0.f;
    bool ok = true;
    PROF_DECL();
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int n0 = (j_lo + t) * 128 + hf * 64;   // first key of this thread's 64 columns
      float pr[64];
      // ---- phase A ----
      PROF_TIC();
      if (!mbar_wait(s_full, uint32_t(t & 1), abort_flag)) { ok = false; break; }
      PROF_TOC(1);
      tc_fence_after();
      {
        uint32_t s0[32], s1[32];
        tmem_ld64(TM_S + lane_addr + uint32_t(hf * 64), s0, s1);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a_done);
        const bool need_mask = (n0 + 63 > m0) || (p.window < p.T && n0 < m0 + 127 - p.window) || (n0 + 63 >= p.T) ||
                               (m0 + 127 >= p.T);
        exp2_64<true>(s0, s1, c, lse2, nullptr, pr);
        if (need_mask) {
          // the visible keys of a row are one interval [lo, hi] of column indices: one unsigned compare per element
          const int lo = row - p.window - n0;
          const unsigned span = (row < p.T) ? unsigned(min(row, p.T - 1) - n0 - lo) : 0u;
          const int lo_eff = (row < p.T) ? lo : 64;          // rows past the end see nothing
#pragma unroll
          for (int j = 0; j < 64; ++j) pr[j] = (unsigned(j - lo_eff) <= span) ? pr[j] : 0.f;
        }
      }
      // ---- phase B ----
      PROF_TOC(2);
      if (!mbar_wait(&dp_full[t & 1], uint32_t(t >> 1) & 1u, abort_flag)) { ok = false; break; }
      PROF_TOC(3);
      tc_fence_after();
      uint32_t pk[32];
      {
        uint32_t d0[32], d1[32];
        tmem_ld64(TM_DP + lane_addr + uint32_t(hf * 64), d0, d1);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          pk[j] = pack_bf16(pr[2 * j] * (__uint_as_float(d0[2 * j]) - dlt), pr[2 * j + 1] * (__uint_as_float(d0[2 * j + 1]) - dlt));
          pk[16 + j] = pack_bf16(pr[32 + 2 * j] * (__uint_as_float(d1[2 * j]) - dlt),
                                 pr[32 + 2 * j + 1] * (__uint_as_float(d1[2 * j + 1]) - dlt));
        }
      }
      // dS buffer t&1 was last read by the dQ MMAs of tile t-2
      PROF_TOC(4);
      if (t >= 2 && !mbar_wait(&dq_done[(t - 2) % 6], uint32_t((t - 2) / 6) & 1u, abort_flag)) { ok = false; break; }
      PROF_TOC(5);
      tc_fence_after();
      tmem_st32(TM_DS + lane_addr + uint32_t((t & 1) * 64 + hf * 32), pk);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[t & 1]);
      PROF_TOC(6);
    }
    if (lane == 0 && (sw == 0 || sw == 5)) PROF_DUMP(sw == 0 ? 2 : 3);
    if (ok && mbar_wait(done, 0, abort_flag)) {
      tc_fence_after();
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + ((long long)b * p.T + row) * p.ldo + h * HD + hf * 64;
      const float sc = p.scale;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        uint32_t v[32];
        tmem_ld32(TM_DQ + lane_addr + uint32_t(hf * 64 + cc * 32), v);
        tmem_wait_ld();
        if (row < p.T) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 u;
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

// ===============================================================================================
// dK / dV
// ===============================================================================================
__global__ void __launch_bounds__(ATT_WIDE_THREADS, 1)
attn_bwd_dkv_wide_k(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO, const AttnArgs p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0 && p.err) atomicExch(p.err, ERR_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WideSmem::BAR);
  uint64_t* kv_full = bars;           // K + V resident
  uint64_t* q_full = bars + 1;        // [3]
  uint64_t* q_empty = bars + 4;       // [3] dK(t) complete
  uint64_t* do_full = bars + 7;       // [2]
  uint64_t* do_empty = bars + 9;      // [2] dV(t) complete
  uint64_t* s_full = bars + 11;       // S^T(t) complete
  uint64_t* p_full = bars + 12;       // phase A(t) wrote P^T(t)              (8 arrivals)
  uint64_t* dp_full = bars + 13;      // dP^T(t) complete
  uint64_t* ds_full = bars + 14;      // phase B(t) wrote dS^T(t)             (8 arrivals)
  uint64_t* done = bars + 15;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat_lse = reinterpret_cast<float*>(smem + WideSmem::STAT);   // [2][128]
  float* stat_dl = stat_lse + 256;                                      // [2][128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y, b = blockIdx.z;
  const int n0 = int(blockIdx.x) * 128;      // earlier key tiles are seen by more queries and come first
  const int i_lo = n0 / 128;
  const long long last_q = (p.window >= p.T) ? (long long)(p.T - 1) : min((long long)(p.T - 1), (long long)n0 + 127 + p.window);
  const int i_hi = int(last_q / 128);
  const int n_tiles = i_hi - i_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&do_full[i], 1); mbar_init(&do_empty[i], 1); }
    mbar_init(s_full, 1); mbar_init(p_full, 8); mbar_init(dp_full, 1); mbar_init(ds_full, 8); mbar_init(done, 1);
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
      tma_load_4d(smem + WideSmem::RES0, &tmK, kv_full, 0, h, n0, b);
      tma_load_4d(smem + WideSmem::RES0 + 16384, &tmK, kv_full, 64, h, n0, b);
      tma_load_4d(smem + WideSmem::RES1, &tmV, kv_full, 0, h, n0, b);
      tma_load_4d(smem + WideSmem::RES1 + 16384, &tmV, kv_full, 64, h, n0, b);
      for (int t = 0; t < n_tiles; ++t) {
        const int q0 = (i_lo + t) * 128;
        if (!mbar_wait(&q_empty[t % 3], (uint32_t(t / 3) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* qs = smem + WideSmem::RING3 + (t % 3) * 32768;
        mbar_expect_tx(&q_full[t % 3], 32768);
        tma_load_4d(qs, &tmQ, &q_full[t % 3], 0, h, q0, b);
        tma_load_4d(qs + 16384, &tmQ, &q_full[t % 3], 64, h, q0, b);
        if (!mbar_wait(&do_empty[t & 1], (uint32_t(t >> 1) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* ds = smem + WideSmem::RING2 + (t & 1) * 32768;
        mbar_expect_tx(&do_full[t & 1], 32768);
        tma_load_4d(ds, &tmDO, &do_full[t & 1], 0, h, q0, b);
        tma_load_4d(ds + 16384, &tmDO, &do_full[t & 1], 64, h, q0, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_kk = make_idesc_bf16(128, 128, false, false);
      constexpr uint32_t idesc_mn = make_idesc_bf16(128, 128, false, true);
      const uint32_t sk = smem_u32(smem + WideSmem::RES0), sv = smem_u32(smem + WideSmem::RES1);
      const uint32_t sq0 = smem_u32(smem + WideSmem::RING3), sdo0 = smem_u32(smem + WideSmem::RING2);
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      if (ok) ok = mbar_wait(&q_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        mma_tile_kk(TM_S, sk, sq0, idesc_kk);
        tc_commit(s_full);
        ok = mbar_wait(&do_full[0], 0, abort_flag);
      }
      if (ok) {
        tc_fence_after();
        mma_tile_kk(TM_DP, sv, sdo0, idesc_kk);
        tc_commit(dp_full);
      }
      PROF_DECL();
      for (int t = 0; t < n_tiles && ok; ++t) {
        const bool more = t + 1 < n_tiles;
        const uint32_t sq = sq0 + uint32_t(t % 3) * 32768u, sdo = sdo0 + uint32_t(t & 1) * 32768u;
        PROF_TIC();
        // dV(t) reads P^T(t) from the S^T tile; S^T(t+1) is issued after it and may then overwrite it
        if (!mbar_wait(p_full, uint32_t(t & 1), abort_flag)) { ok = false; break; }
        PROF_TOC(1);
        tc_fence_after();
        mma_tile_ts(TM_DV, TM_S, TM_S + 64, sdo, idesc_mn, t > 0);
        tc_commit(&do_empty[t & 1]);
        if (more) {
          if (!mbar_wait(&q_full[(t + 1) % 3], uint32_t((t + 1) / 3) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_tile_kk(TM_S, sk, sq0 + uint32_t((t + 1) % 3) * 32768u, idesc_kk);
          tc_commit(s_full);
        }
        PROF_TOC(2);
        if (!mbar_wait(ds_full, uint32_t(t & 1), abort_flag)) { ok = false; break; }
        PROF_TOC(3);
        tc_fence_after();
        mma_tile_ts(TM_DK, TM_DP, TM_DP + 64, sq, idesc_mn, t > 0);
        tc_commit(&q_empty[t % 3]);
        if (more) {
          if (!mbar_wait(&do_full[(t + 1) & 1], uint32_t((t + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_tile_kk(TM_DP, sv, sdo0 + uint32_t((t + 1) & 1) * 32768u, idesc_kk);
          tc_commit(dp_full);
        }
        PROF_TOC(4);
      }
      if (ok) tc_commit(done);
      PROF_DUMP(4);
    }
  } else {
    const int sw = warp - 2;
    const int q = warp & 3;
    const int hf = sw >> 2;              // query-column half of the tile owned by this warp
    const int r = q * 32 + lane;         // key row inside the tile
    const int key = n0 + r;
    const int tid = threadIdx.x - 64;    // 0..255
    const uint32_t lane_addr = uint32_t(q * 32) << 16;
    const float c = p.scale * LOG2E;
    const long long stat0 = ((long long)b * p.H + h) * p.T;
    auto load_stat = [&](int t) -> float {   // tid < 128: lse2 of query tid of tile t; else delta of query tid-128
      const int qi = (i_lo + t) * 128 + (tid & 127);
      if (t >= n_tiles || qi >= p.T) return (tid < 128) ? INFINITY : 0.f;
      return (tid < 128) ? p.lse[stat0 + qi] * LOG2E : p.delta[stat0 + qi];
    };
    (tid < 128 ? stat_lse : stat_dl)[tid & 127] = load_stat(0);
    bool ok = true;
    PROF_DECL();
    for (int t = 0; t < n_tiles; ++t) {
      const int q0 = (i_lo + t) * 128 + hf * 64;   // first query of this thread's 64 columns
      const int buf = t & 1;
      PROF_TIC();
      named_bar_sync(1, 256);                    // statistics of tile t are visible to all softmax warps
      const float next_stat = load_stat(t + 1);  // in flight while this tile is processed
      const float4* cl = reinterpret_cast<const float4*>(stat_lse + buf * 128 + hf * 64);
      const float4* cd = reinterpret_cast<const float4*>(stat_dl + buf * 128 + hf * 64);
      float pr[64];
      // ---- phase A: P^T = exp2(S^T * c - lse2[query]) ----
      PROF_TOC(1);
      if (ok && !mbar_wait(s_full, uint32_t(t & 1), abort_flag)) ok = false;
      PROF_TOC(2);
      if (ok) {
        tc_fence_after();
        uint32_t s0[32], s1[32];
        tmem_ld64(TM_S + lane_addr + uint32_t(hf * 64), s0, s1);
        const bool need_mask = (q0 < n0 + 127) || (p.window < p.T && q0 + 63 > n0 + p.window) || (q0 + 63 >= p.T) ||
                               (n0 + 127 >= p.T);
        exp2_64<false>(s0, s1, c, 0.f, cl, pr);
        if (need_mask) {
          // the queries that see a key are one interval of column indices: key <= q <= min(key + window, T - 1)
          const int lo = (key < p.T) ? key - q0 : 64;
          const unsigned span = (key < p.T) ? unsigned(min((long long)key + p.window, (long long)p.T - 1) - key) : 0u;
#pragma unroll
          for (int j = 0; j < 64; ++j) pr[j] = (unsigned(j - lo) <= span) ? pr[j] : 0.f;
        }
        uint32_t pk[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) pk[j] = pack_bf16(pr[2 * j], pr[2 * j + 1]);
        tmem_st32(TM_S + lane_addr + uint32_t(hf * 64), pk);   // over this thread's own, already read, S^T columns
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
      // ---- phase B: dS^T = P^T * (dP^T - delta[query]) ----
      PROF_TOC(3);
      if (ok && !mbar_wait(dp_full, uint32_t(t & 1), abort_flag)) ok = false;
      PROF_TOC(4);
      if (ok) {
        tc_fence_after();
        uint32_t d0[32], d1[32];
        tmem_ld64(TM_DP + lane_addr + uint32_t(hf * 64), d0, d1);
        uint32_t pk[32];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 e0 = cd[g], e1 = cd[8 + g];
          pk[2 * g] = pack_bf16(pr[4 * g] * (__uint_as_float(d0[4 * g]) - e0.x), pr[4 * g + 1] * (__uint_as_float(d0[4 * g + 1]) - e0.y));
          pk[2 * g + 1] = pack_bf16(pr[4 * g + 2] * (__uint_as_float(d0[4 * g + 2]) - e0.z),
                                    pr[4 * g + 3] * (__uint_as_float(d0[4 * g + 3]) - e0.w));
          pk[16 + 2 * g] = pack_bf16(pr[32 + 4 * g] * (__uint_as_float(d1[4 * g]) - e1.x),
                                     pr[32 + 4 * g + 1] * (__uint_as_float(d1[4 * g + 1]) - e1.y));
          pk[16 + 2 * g + 1] = pack_bf16(pr[32 + 4 * g + 2] * (__uint_as_float(d1[4 * g + 2]) - e1.z),
                                         pr[32 + 4 * g + 3] * (__uint_as_float(d1[4 * g + 3]) - e1.w));
        }
        tmem_st32(TM_DP + lane_addr + uint32_t(hf * 64), pk);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(ds_full);
      }
      PROF_TOC(5);
      (tid < 128 ? stat_lse : stat_dl)[((t + 1) & 1) * 128 + (tid & 127)] = next_stat;
    }
    if (lane == 0 && (sw == 0 || sw == 5)) PROF_DUMP(sw == 0 ? 6 : 7);
    if (ok && mbar_wait(done, 0, abort_flag)) {
      tc_fence_after();
      __nv_bfloat16* dkrow = reinterpret_cast<__nv_bfloat16*>(p.dk) + ((long long)b * p.T + key) * p.lddk + h * HD + hf * 64;
      __nv_bfloat16* dvrow = reinterpret_cast<__nv_bfloat16*>(p.dv) + ((long long)b * p.T + key) * p.lddv + h * HD + hf * 64;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const float sc = which ? p.scale : 1.f;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          uint32_t v[32];
          tmem_ld32((which ? TM_DK : TM_DV) + lane_addr + uint32_t(hf * 64 + cc * 32), v);
          tmem_wait_ld();
          if (key < p.T) {
            __nv_bfloat16* dst = (which ? dkrow : dvrow) + cc * 32;
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


// Launches both kernels of the wide backward; `a` carries sizes, lse, delta and the error flag.
int attn_wide_bwd_launch(const void* q, const void* k, const void* v, const void* d_o, void* dq, void* dk, void* dv,
                         long long ldq, long long ldk, long long ldv, long long lddo, long long lddq, long long lddk,
                         long long lddv, AttnArgs a, cudaStream_t stream) {
  static PerDeviceOnce cfg;
  int r;
  if (cfg.first()) {
    if ((r = set_smem(attn_bwd_dq_wide_k, WideSmem::TOTAL))) return r;
    if ((r = set_smem(attn_bwd_dkv_wide_k, WideSmem::TOTAL))) return r;
  }
  CUtensorMap tq, tk, tv, tdo;
  if ((r = make_qkv_tmap(&tq, q, a.B, a.T, a.H, ldq, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tk, k, a.B, a.T, a.H, ldk, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tv, v, a.B, a.T, a.H, ldv, 128))) return 1000 + r;
  if ((r = make_qkv_tmap(&tdo, d_o, a.B, a.T, a.H, lddo, 128))) return 1000 + r;
  dim3 grid((a.T + 127) / 128, a.H, a.B);
  a.o = dq; a.ldo = lddq;
  attn_bwd_dq_wide_k<<<grid, ATT_WIDE_THREADS, WideSmem::TOTAL, stream>>>(tq, tk, tv, tdo, a);
  if ((r = int(cudaGetLastError()))) return r;
  a.dk = dk; a.dv = dv; a.lddk = lddk; a.lddv = lddv;
  attn_bwd_dkv_wide_k<<<grid, ATT_WIDE_THREADS, WideSmem::TOTAL, stream>>>(tq, tk, tv, tdo, a);
  return int(cudaGetLastError());
}

}  // namespace arb

#ifdef ARB_ATTN_PROF
// Entry point of the profiling build (bench/attn_roles.py): runs the wide backward once and leaves the
// per-role cycle counters of CTA (0,0,0) in `prof` (device, 64 x int64).
extern "C" int arb_attn_prof_wide_bwd(const void* q, const void* k, const void* v, const void* d_o, void* dq, void* dk,
                                      void* dv, const float* lse, const float* delta, int B, int T, int H, long long ld,
                                      long long ldo, int window, float scale, int* err, long long* prof) {
  cudaMemcpyToSymbol(arb::arb_attn_prof_buffer, &prof, sizeof(prof));
  arb::AttnArgs a{};
  a.B = B; a.T = T; a.H = H; a.window = window > T ? T : window; a.scale = scale;
  a.lse = const_cast<float*>(lse); a.delta = delta; a.err = err;
  return arb::attn_wide_bwd_launch(q, k, v, d_o, dq, dk, dv, ld, ld, ld, ldo, ld, ld, ld, a, 0);
}
#endif
