// bf16 GEMM on the 5th-generation tensor cores: persistent, warp-specialised, TMA-fed,
// fp32 accumulators in TMEM (double buffered so the epilogue of one tile overlaps the main
// loop of the next).
//
//   C[b] (op)= A[b] * B[b]        A: M x K, B: K x N (each K-major or MN-major in memory)
//
// Replaces the reference's cuBLAS calls (brain/src/gemm.rs:87-441: matmul = NT,
// matmul_bwd_x = NN, matmul_acc = TN with beta=1, strided-batched forms for Newton-Schulz)
// and fuses what the reference runs as separate kernels into the epilogue: ReLU^2
// (brain/kernels/relu_sq.cu), residual add, the Newton-Schulz combine aI + bA + cA^2
// (brain/kernels/muon.cu:385-415), and fp32 gradient accumulation (split-K partial sums are
// added with red.global so wide-K dW GEMMs fill all SMs).
//
// CTA = 224 threads: warp 0 TMA producer, warp 1 MMA issuer + TMEM owner, warps 2-5 epilogue
// (warp w reads TMEM lanes 32*(w%4)..+31), warp 6 copies another operand from a peer GPU while the
// tiles are computed (GemmArgs::ahead_src; idle otherwise).  Tile 128 x BN x 64 (BN = 256 or 128),
// 128-byte swizzled smem stages.
#include "api.h"
#include "ptx.cuh"
#include "tmap.h"

#include <cstring>

namespace arb {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int GEMM_THREADS = 224;

// EPI_QKV_POST: what the epilogue does to the heads of the packed q|k|v projection (see api.h)
struct QkvPostArgs {
  const __nv_bfloat16* cos_t;
  const __nv_bfloat16* sin_t;
  float* rstd;
  int T, H;
  const __nv_bfloat16* xn;
  long long ld_xn;
  const int* ids;
  const __nv_bfloat16* ve;
  const __nv_bfloat16* gate_w;
  float* gate;
  int gate_ch;
  float eps;
};

struct GemmArgs {
  int M, N, K, batch;
  int m_tiles, n_tiles, kb_total, kb_per_split, splitk;
  void* C;
  const void* aux;
  long long ldc, stride_c;      // elements
  float alpha, beta, gamma;
  int* err;
  // Optional prologue: before any tile is loaded, all CTAs of this (fully resident, persistent) grid copy
  // pull_n16 16-byte units from pull_src (the owner rank's copy of the B operand, NVLink peer loads) to
  // pull_dst (the local operand) and meet at a counter barrier.  Fuses the data-parallel all-gather of an
  // updated weight into the first GEMM that consumes it.
  const uint4* pull_src;
  uint4* pull_dst;
  long long pull_n16;
  unsigned* pull_counter;
  unsigned pull_target;
  // Optional side copy, overlapped with the tile loop: warp 6 of every CTA copies ahead_n16 16-byte units from
  // ahead_src (a peer rank's copy of the operand of a LATER GEMM on this stream) to ahead_dst.  Nothing in this
  // kernel reads ahead_dst; the kernel boundary orders the copy before its consumer, so no barrier is needed.
  const uint4* ahead_src;
  uint4* ahead_dst;
  long long ahead_n16;
  // Ragged batches (grouped expert GEMMs).  All three roles of a CTA evaluate the same predicates, so an item that
  // is skipped touches no barrier and no output.
  //   m_valid[b]   rows of batch item b that hold data: M-tiles that start at or beyond it are skipped.
  //   b_div        the B operand (and nothing else) is indexed by b / b_div: several row slabs share one weight.
  //   k_valid[b * k_nseg + seg]  (fp32-accumulate GEMMs whose K runs over rows) the K range is k_nseg segments of
  //                k_seg_kb 64-row blocks; of segment seg only the blocks below k_valid are multiplied.
  const int* m_valid;
  int b_div;
  const int* k_valid;
  int k_seg_kb, k_nseg;
  QkvPostArgs qp;
};

// K blocks of [kb0, kb1) of batch item b that are multiplied
__device__ __forceinline__ bool kb_live(const GemmArgs& p, int b, int kb) {
  if (!p.k_valid) return true;
  const int seg = kb / p.k_seg_kb;
  return (kb - seg * p.k_seg_kb) * BK < p.k_valid[b * p.k_nseg + seg];
}
__device__ __forceinline__ bool item_live(const GemmArgs& p, int b, int m_start, int kb0, int kb1) {
  if (p.m_valid && m_start >= p.m_valid[b]) return false;
  if (p.k_valid) {
    for (int kb = kb0; kb < kb1; ++kb)
      if (kb_live(p, b, kb)) return true;
    return false;
  }
  return true;
}

__device__ __forceinline__ uint4 ld_peer16(const uint4* a) {
  uint4 v;
  asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(a));
  return v;
}

// Warp 6: grid-strided copy with eight peer loads in flight per thread.
__device__ __forceinline__ void pull_ahead(const GemmArgs& p, int lane) {
  if (p.ahead_n16 <= 0) return;
  const long long stride = (long long)gridDim.x * 32;
  long long i = (long long)blockIdx.x * 32 + lane;
  for (; i + 7 * stride < p.ahead_n16; i += 8 * stride) {
    uint4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = ld_peer16(p.ahead_src + i + u * stride);
#pragma unroll
    for (int u = 0; u < 8; ++u) p.ahead_dst[i + u * stride] = v[u];
  }
  for (; i < p.ahead_n16; i += stride) p.ahead_dst[i] = ld_peer16(p.ahead_src + i);
}

// Runs in every thread of every CTA at kernel start.  The waits are bounded; on expiry the error word is set
// and the kernel goes on (the result is then wrong, the host raises on the error word).
__device__ __forceinline__ void pull_prologue(const GemmArgs& p) {
  if (p.pull_n16 <= 0) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  auto ld = [](const uint4* a) { return ld_peer16(a); };
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < p.pull_n16; i += 4 * stride) {     // four peer loads in flight per thread
    const uint4 a = ld(p.pull_src + i), b = ld(p.pull_src + i + stride), c = ld(p.pull_src + i + 2 * stride),
                d = ld(p.pull_src + i + 3 * stride);
    p.pull_dst[i] = a; p.pull_dst[i + stride] = b; p.pull_dst[i + 2 * stride] = c; p.pull_dst[i + 3 * stride] = d;
  }
  for (; i < p.pull_n16; i += stride) p.pull_dst[i] = ld(p.pull_src + i);
  __threadfence();
  asm volatile("fence.proxy.async;" ::: "memory");   // the copies are read by TMA (async proxy) below
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.pull_counter) : "memory");
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.pull_counter) : "memory");
      if (int(v - p.pull_target) >= 0) break;
      if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
        if (p.err) atomicExch(p.err, ERR_GEMM_TIMEOUT);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  asm volatile("fence.proxy.async;" ::: "memory");
}

template <int BN>
struct SmemLayout {
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // + barriers + alignment slack
};

// One 32-column chunk of one accumulator row -> global memory, with the fused epilogue.
template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&v)[32], const GemmArgs& p, int row, long long row_off, int col0) {
  const bool full = (col0 + 32 <= p.N);
  if (EPI == EPI_ATOMIC_F32) {
    float* dst = reinterpret_cast<float*>(p.C) + row_off + col0;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j), "f"(__uint_as_float(v[j])),
                     "f"(__uint_as_float(v[j + 1])), "f"(__uint_as_float(v[j + 2])), "f"(__uint_as_float(v[j + 3])) : "memory");
    } else {
      for (int j = 0; j < 32 && col0 + j < p.N; ++j) atomicAdd(dst + j, __uint_as_float(v[j]));
    }
  } else if (EPI == EPI_STORE_F32) {
    float* dst = reinterpret_cast<float*>(p.C) + row_off + col0;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(dst + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                          __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
    } else {
      for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = __uint_as_float(v[j]);
    }
  } else {
    float f[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
    if (EPI == EPI_RELU2) {
#pragma unroll
      for (int j = 0; j < 32; ++j) { float r = fmaxf(f[j], 0.f); f[j] = r * r; }
    }
    if (EPI == EPI_NS_COMBINE || EPI == EPI_RELU2_BWD || EPI == EPI_ADD_AUX) {
      const __nv_bfloat16* ax = reinterpret_cast<const __nv_bfloat16*>(p.aux) + row_off + col0;
      float a[32];
      if (full) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          uint4 u = *reinterpret_cast<const uint4*>(ax + j);
          float2 t0 = unpack_bf16(u.x), t1 = unpack_bf16(u.y), t2 = unpack_bf16(u.z), t3 = unpack_bf16(u.w);
          a[j] = t0.x; a[j + 1] = t0.y; a[j + 2] = t1.x; a[j + 3] = t1.y;
          a[j + 4] = t2.x; a[j + 5] = t2.y; a[j + 6] = t3.x; a[j + 7] = t3.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) a[j] = (col0 + j < p.N) ? __bfloat162float(ax[j]) : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        if (EPI == EPI_NS_COMBINE) f[j] = p.beta * a[j] + p.gamma * f[j] + ((row == col0 + j) ? p.alpha : 0.f);
        else if (EPI == EPI_RELU2_BWD) f[j] = f[j] * 2.f * sqrtf(fmaxf(a[j], 0.f));
        else f[j] = f[j] + a[j];
      }
    }
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + row_off + col0;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 u;
        u.x = pack_bf16(f[j], f[j + 1]); u.y = pack_bf16(f[j + 2], f[j + 3]);
        u.z = pack_bf16(f[j + 4], f[j + 5]); u.w = pack_bf16(f[j + 6], f[j + 7]);
        *reinterpret_cast<uint4*>(dst + j) = u;
      }
    } else {
      for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = __float2bfloat16(f[j]);
    }
  }
      }

template <bool A_MN, bool B_MN, int EPI, int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs p) {
  using L = SmemLayout<BN>;
  constexpr int STAGES = L::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int items = p.batch * p.m_tiles * p.n_tiles * p.splitk;
  pull_prologue(p);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 4); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 2 * BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < items && ok; w += gridDim.x) {
        int t = w;
        const int nt = t % p.n_tiles; t /= p.n_tiles;
        const int mt = t % p.m_tiles; t /= p.m_tiles;
        const int ks = t % p.splitk;
        const int b = t / p.splitk;
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        if (!item_live(p, b, mt * BM, kb0, kb1)) continue;
        const int bB = b / p.b_div;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!kb_live(p, b, kb)) continue;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ++it;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_3d(sa + c * 8192, &tmA, &full_bar[s], mt * BM + c * 64, kb * BK, b);
          } else {
            tma_load_3d(sa, &tmA, &full_bar[s], kb * BK, mt * BM, b);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_3d(sb + c * 8192, &tmB, &full_bar[s], nt * BN + c * 64, kb * BK, bB);
          } else {
            tma_load_3d(sb, &tmB, &full_bar[s], kb * BK, nt * BN, bB);
          }
        }
      }
      if (!ok) {
        // give loads already in flight a bounded chance to land before the CTA exits
        for (int s = 0; s < STAGES; ++s)
          for (uint32_t i = 0; i < 4096 && !mbar_try_wait(&full_bar[s], 0) && !mbar_try_wait(&full_bar[s], 1); ++i) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < items && ok; w += gridDim.x) {
        int t = w / p.n_tiles;
        const int mt = t % p.m_tiles; t /= p.m_tiles;
        const int ks = t % p.splitk;
        const int b = t / p.splitk;
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        if (!item_live(p, b, mt * BM, kb0, kb1)) continue;
        const int acc = tile_it & 1;
        const uint32_t aph = (tile_it >> 1) & 1;
        ++tile_it;
        if (!mbar_wait(&tempty_bar[acc], aph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool first = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!kb_live(p, b, kb)) continue;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ++it;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 0, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 0, 1024);
            tc_mma_ss(d_tmem, ad, bd, idesc, (!first || k > 0) ? 1u : 0u);
          }
          first = false;
          tc_commit(&empty_bar[s]);
        }
        if (ok) tc_commit(&tfull_bar[acc]);
      }
    }
  } else if (warp == 6) {
    pull_ahead(p, lane);
  } else {
    // ---------------- epilogue (4 warps) ----------------
    const int q = warp & 3;
    uint32_t tile_it = 0;
    bool ok = true;
    for (int w = blockIdx.x; w < items && ok; w += gridDim.x) {
      int t = w;
      const int nt = t % p.n_tiles; t /= p.n_tiles;
      const int mt = t % p.m_tiles; t /= p.m_tiles;
      const int ks = t % p.splitk;
      const int b = t / p.splitk;
      {
        const int kb0 = ks * p.kb_per_split;
        if (!item_live(p, b, mt * BM, kb0, min(p.kb_total, kb0 + p.kb_per_split))) continue;
      }
      const int acc = tile_it & 1;
      const uint32_t aph = (tile_it >> 1) & 1;
      ++tile_it;
      if (!mbar_wait(&tfull_bar[acc], aph, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = mt * BM + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long row_off = (long long)b * p.stride_c + (long long)row * p.ldc;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN + c * 32), v);
        tmem_wait_ld();
        const int col0 = nt * BN + c * 32;
        if (!row_ok || col0 >= p.N) continue;
        epilogue_chunk<EPI>(v, p, row, row_off, col0);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, ERR_GEMM_TIMEOUT);
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, 2 * BN); }
}

// One head (128 accumulator columns of one row) of the packed q|k|v projection, in place.
__device__ __forceinline__ void qkv_post_head(float (&f)[128], const QkvPostArgs& q, int row, int col_h) {
  const int Dl = q.H * 128;
  const int sec = col_h / Dl;                       // 0 query, 1 key, 2 value
  const int head = (col_h - sec * Dl) >> 7;
  if (sec < 2) {
    const int t = row % q.T;
    const uint4* cp = reinterpret_cast<const uint4*>(q.cos_t + (long long)t * 64);
    const uint4* sp = reinterpret_cast<const uint4*>(q.sin_t + (long long)t * 64);
    float ss = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      const uint4 cu = __ldg(cp + g), su = __ldg(sp + g);
      const uint32_t cw[4] = {cu.x, cu.y, cu.z, cu.w}, sw[4] = {su.x, su.y, su.z, su.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 c2 = unpack_bf16(cw[e]), s2 = unpack_bf16(sw[e]);
        const int j = g * 8 + 2 * e;
        const float lo0 = f[j], hi0 = f[j + 64], lo1 = f[j + 1], hi1 = f[j + 65];
        const float a0 = lo0 * c2.x + hi0 * s2.x, b0 = hi0 * c2.x - lo0 * s2.x;
        const float a1 = lo1 * c2.y + hi1 * s2.y, b1 = hi1 * c2.y - lo1 * s2.y;
        f[j] = a0; f[j + 64] = b0; f[j + 1] = a1; f[j + 65] = b1;
        ss += a0 * a0 + b0 * b0 + a1 * a1 + b1 * b1;
      }
    }
    const float r = rsqrtf(ss * (1.f / 128.f) + q.eps);
#pragma unroll
    for (int j = 0; j < 128; ++j) f[j] *= r;
    q.rstd[(long long)row * (2 * q.H) + sec * q.H + head] = r;
  } else if (q.ve) {
    const __nv_bfloat16* xr = q.xn + (long long)row * q.ld_xn;
    const __nv_bfloat16* gw = q.gate_w + head * q.gate_ch;
    float gl = 0.f;
    for (int j = 0; j < q.gate_ch; j += 8) {
      const uint4 xu = __ldg(reinterpret_cast<const uint4*>(xr + j)), gu = __ldg(reinterpret_cast<const uint4*>(gw + j));
      const uint32_t xw[4] = {xu.x, xu.y, xu.z, xu.w}, gg[4] = {gu.x, gu.y, gu.z, gu.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 a = unpack_bf16(xw[e]), b = unpack_bf16(gg[e]);
        gl += a.x * b.x + a.y * b.y;
      }
    }
    q.gate[(long long)row * q.H + head] = gl;
    const float gs = 2.f / (1.f + __expf(-gl));
    const uint4* vp = reinterpret_cast<const uint4*>(q.ve + (long long)q.ids[row] * Dl + head * 128);
#pragma unroll
    for (int g = 0; g < 16; ++g) {
      const uint4 eu = __ldg(vp + g);
      const uint32_t ew[4] = {eu.x, eu.y, eu.z, eu.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 v = unpack_bf16(ew[e]);
        f[g * 8 + 2 * e] += gs * v.x;
        f[g * 8 + 2 * e + 1] += gs * v.y;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
// 2-CTA variant: a cluster of two CTAs (one SM pair) owns a 256 x 256 tile.  Each CTA loads its
// own 128 rows of A and 128 of the 256 rows of B (half the B traffic per SM of the 1-CTA kernel,
// so six 32 KB stages fit), the pair leader issues tcgen05.mma.cta_group::2 (M = 256) which reads
// both CTAs' shared memory and writes each CTA's half of the accumulator into its own TMEM, and
// each CTA runs the epilogue for its 128 rows.  Loads carry no cluster multicast.
// ------------------------------------------------------------------------------------------
__host__ __device__ constexpr bool epi_is_bf16(int epi) { return epi != EPI_ATOMIC_F32 && epi != EPI_STORE_F32; }
__host__ __device__ constexpr bool epi_has_aux(int epi) { return epi == EPI_NS_COMBINE || epi == EPI_RELU2_BWD || epi == EPI_ADD_AUX; }

// bf16 outputs leave through a swizzled smem staging slab (128 rows x 64 columns, double buffered)
// and TMA stores, so every request to L2 is a full line; aux operands arrive the same way.
template <int EPI>
struct Smem2 {
  static constexpr bool STAGED = true;      // fp32 outputs are staged as 128 x 32 slabs (TMA store / reduce-add)
  static constexpr bool AUX = epi_has_aux(EPI);
  static constexpr int STAGES = AUX ? 5 : 6;
  static constexpr int A_BYTES = 128 * BK * 2;
  static constexpr int B_BYTES = 128 * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int C_STAGE = STAGES * STAGE_BYTES;                       // 2 x 16 KB
  static constexpr int X_STAGE = C_STAGE + (STAGED ? 32768 : 0);             // 2 x 16 KB
  static constexpr int BAR_OFFSET = X_STAGE + (AUX ? 32768 : 0);
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

template <bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmX, const GemmArgs p) {
  using L = Smem2<EPI>;
  constexpr int STAGES = L::STAGES;
  constexpr int BN2 = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);   // used in the leader only (count 1)
  uint64_t* empty_bar = full_bar + STAGES;                                   // per CTA (count 1)
  uint64_t* tfull_bar = empty_bar + STAGES;                                  // per CTA (count 1)
  uint64_t* tempty_bar = tfull_bar + 2;                                      // used in the leader only (count 8)
  uint64_t* xfull_bar = tempty_bar + 2;                                      // aux slab landed (count 1)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xfull_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;
  const int items = p.batch * p.m_tiles * p.n_tiles * p.splitk;   // m_tiles counted in 256-row tiles
  pull_prologue(p);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tfull_bar[a], 1); mbar_init(&tempty_bar[a], 8); mbar_init(&xfull_bar[a], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc_pair(tmem_slot, 512); tmem_relinquish_pair(); }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      uint32_t it = 0;
      bool ok = true;
      for (int w = cluster_id; w < items && ok; w += n_clusters) {
        int t = w;
        const int nt = t % p.n_tiles; t /= p.n_tiles;
        const int mt = t % p.m_tiles; t /= p.m_tiles;
        const int ks = t % p.splitk;
        const int b = t / p.splitk;
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        const int m0 = mt * 256 + int(rank) * 128;
        const int n0 = nt * 256 + int(rank) * 128;
        if (!item_live(p, b, mt * 256, kb0, kb1)) continue;
        const int bB = b / p.b_div;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!kb_live(p, b, kb)) continue;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ++it;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          const uint32_t lead_bar = mapa_u32(smem_u32(&full_bar[s]), 0);
          // only the leader arrives (and announces both CTAs' bytes); the peer's copies just credit
          // their bytes to the same barrier - a remote arrive per stage costs a cluster-scope release
          if (leader) mbar_expect_tx(&full_bar[s], 2 * L::STAGE_BYTES);
          if (A_MN) {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_3d_pair(sa + c * 8192, &tmA, lead_bar, m0 + c * 64, kb * BK, b);
          } else {
            tma_load_3d_pair(sa, &tmA, lead_bar, kb * BK, m0, b);
          }
          if (B_MN) {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_3d_pair(sb + c * 8192, &tmB, lead_bar, n0 + c * 64, kb * BK, bB);
          } else {
            tma_load_3d_pair(sb, &tmB, lead_bar, kb * BK, n0, bB);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_bf16(256, BN2, A_MN, B_MN);
      uint32_t it = 0, tile_it = 0;
      bool ok = true;
      for (int w = cluster_id; w < items && ok; w += n_clusters) {
        int t = w / p.n_tiles;
        const int mt = t % p.m_tiles; t /= p.m_tiles;
        const int ks = t % p.splitk;
        const int b = t / p.splitk;
        const int kb0 = ks * p.kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + p.kb_per_split);
        if (!item_live(p, b, mt * 256, kb0, kb1)) continue;
        const int acc = tile_it & 1;
        const uint32_t aph = (tile_it >> 1) & 1;
        ++tile_it;
        if (!mbar_wait(&tempty_bar[acc], aph ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN2;
        bool first = true;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!kb_live(p, b, kb)) continue;
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ++it;
          if (!mbar_wait(&full_bar[s], ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = A_MN ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 0, 1024);
            const uint64_t bd = B_MN ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 0, 1024);
            tc_mma_ss_pair(d_tmem, ad, bd, idesc, (!first || k > 0) ? 1u : 0u);
          }
          first = false;
          const uint32_t eb = smem_u32(&empty_bar[s]);
          tc_commit_pair(eb);
          tc_commit_pair(mapa_u32(eb, 1));
        }
        if (ok) {
          const uint32_t tb = smem_u32(&tfull_bar[acc]);
          tc_commit_pair(tb);
          tc_commit_pair(mapa_u32(tb, 1));
        }
      }
    }
  } else if (warp == 6) {
    pull_ahead(p, lane);
  } else {
    const int q = warp & 3;
    uint32_t tile_it = 0, slab_it = 0;
    bool ok = true;
    for (int w = cluster_id; w < items; w += n_clusters) {
      int t = w;
      const int nt = t % p.n_tiles; t /= p.n_tiles;
      const int mt = t % p.m_tiles; t /= p.m_tiles;
      const int ks = t % p.splitk;
      const int b = t / p.splitk;
      {
        const int kb0 = ks * p.kb_per_split;
        if (!item_live(p, b, mt * 256, kb0, min(p.kb_total, kb0 + p.kb_per_split))) continue;
      }
      const int acc = tile_it & 1;
      const uint32_t aph = (tile_it >> 1) & 1;
      const bool first_tile = tile_it == 0;
      ++tile_it;
      // after a time-out keep walking the loop (named barriers below need all four warps) but skip waits
      if (ok && !mbar_wait(&tfull_bar[acc], aph, abort_flag)) ok = false;
      tc_fence_after();
      const int row = mt * 256 + int(rank) * 128 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const long long row_off = (long long)b * p.stride_c + (long long)row * p.ldc;
      if (!L::STAGED) {
#pragma unroll 1
        for (int c = 0; c < BN2 / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN2 + c * 32), v);
          tmem_wait_ld();
          const int col0 = nt * BN2 + c * 32;
          if (!row_ok || col0 >= p.N) continue;
          epilogue_chunk<EPI>(v, p, row, row_off, col0);
        }
      } else {
        const bool t0 = (threadIdx.x == 64);              // the thread that drives the TMA copies
        const int r_local = q * 32 + lane;
        const int row0 = mt * 256 + int(rank) * 128;
        if (!epi_is_bf16(EPI)) {
          // fp32 output: eight slabs of 128 rows x 32 columns; accumulate-mode goes out as a TMA
          // reduce-add (full-line atomics at L2), store-mode as a TMA store
#pragma unroll 1
          for (int sl = 0; sl < 8; ++sl, ++slab_it) {
            const int buf = slab_it & 1;
            const int col_s = nt * BN2 + sl * 32;
            if (t0) tma_store_wait_read_1();
            named_barrier(2, 128);
            const uint32_t cbase = smem_u32(smem + L::C_STAGE + buf * 16384);
            uint32_t v[32];
            tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN2 + sl * 32), v);
            tmem_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j += 4) st_sw128(cbase, 128, r_local, j * 2, make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]));
            fence_proxy_async_smem();
            named_barrier(3, 128);
            if (t0) {
              if (col_s < p.N && row0 < p.M) {
                if (EPI == EPI_ATOMIC_F32) tma_reduce_add_3d(&tmC, smem + L::C_STAGE + buf * 16384, col_s, row0, b);
                else tma_store_3d(&tmC, smem + L::C_STAGE + buf * 16384, col_s, row0, b);
              }
              tma_store_commit();
            }
          }
        }
        if (L::AUX && t0 && first_tile) {                 // first aux slab of this CTA's first tile
          mbar_expect_tx(&xfull_bar[0], 16384);
          tma_load_3d(smem + L::X_STAGE, &tmX, &xfull_bar[0], nt * BN2, row0, b);
        }
        if constexpr (EPI == EPI_QKV_POST) {
          // a head (128 columns) at a time: both halves of a rotation pair and the whole RMS sit in one thread's registers;
          // the two 64-column staging slabs are written together and leave as two TMA stores
#pragma unroll 1
          for (int hh = 0; hh < 2; ++hh) {
            const int col_h = nt * BN2 + hh * 128;
            float f[128];
            {
              uint32_t v0[32], v1[32], v2[32], v3[32];
              const uint32_t ta = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN2 + hh * 128);
              tmem_ld32(ta, v0); tmem_ld32(ta + 32u, v1); tmem_ld32(ta + 64u, v2); tmem_ld32(ta + 96u, v3);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                f[j] = __uint_as_float(v0[j]); f[32 + j] = __uint_as_float(v1[j]);
                f[64 + j] = __uint_as_float(v2[j]); f[96 + j] = __uint_as_float(v3[j]);
              }
            }
            if (row_ok && col_h < p.N) qkv_post_head(f, p.qp, row, col_h);
            if (t0) tma_store_wait_read();                // both stores of the previous head have read their slabs
            named_barrier(2, 128);                        // (they drained while this head was computed)
#pragma unroll
            for (int half = 0; half < 2; ++half) {
              const uint32_t cbase = smem_u32(smem + L::C_STAGE + half * 16384);
#pragma unroll
              for (int j = 0; j < 64; j += 8) {
                const float* g = f + half * 64 + j;
                uint4 u;
                u.x = pack_bf16(g[0], g[1]); u.y = pack_bf16(g[2], g[3]); u.z = pack_bf16(g[4], g[5]); u.w = pack_bf16(g[6], g[7]);
                st_sw128(cbase, 128, r_local, j, u);
              }
            }
            fence_proxy_async_smem();
            named_barrier(3, 128);
            if (t0) {
              if (col_h < p.N && row0 < p.M) {
                tma_store_3d(&tmC, smem + L::C_STAGE, col_h, row0, b);
                tma_store_3d(&tmC, smem + L::C_STAGE + 16384, col_h + 64, row0, b);
              }
              tma_store_commit();
            }
          }
        } else {
#pragma unroll 1
        for (int sl = 0; sl < (epi_is_bf16(EPI) ? 4 : 0); ++sl, ++slab_it) {
          const int buf = slab_it & 1;
          const int col_s = nt * BN2 + sl * 64;
          if (t0) tma_store_wait_read_1();                // the store issued two slabs ago has read its buffer
          named_barrier(2, 128);
          if (L::AUX) {
            if (t0) {                                      // prefetch the next aux slab (this tile or the next one)
              int nsl = sl + 1, nw = w;
              if (nsl == 4) {                              // the next item of this cluster that is not skipped
                nsl = 0;
                for (nw = w + n_clusters; nw < items; nw += n_clusters) {
                  int tt = nw / p.n_tiles;
                  const int nmt = tt % p.m_tiles; tt /= p.m_tiles;
                  const int nks = tt % p.splitk;
                  const int nkb0 = nks * p.kb_per_split;
                  if (item_live(p, tt / p.splitk, nmt * 256, nkb0, min(p.kb_total, nkb0 + p.kb_per_split))) break;
                }
              }
              if (nw < items) {
                int tt = nw;
                const int nnt = tt % p.n_tiles; tt /= p.n_tiles;
                const int nmt = tt % p.m_tiles; tt /= p.m_tiles;
                const int nb = tt / p.splitk;
                mbar_expect_tx(&xfull_bar[buf ^ 1], 16384);
                tma_load_3d(smem + L::X_STAGE + (buf ^ 1) * 16384, &tmX, &xfull_bar[buf ^ 1], nnt * BN2 + nsl * 64,
                            nmt * 256 + int(rank) * 128, nb);
              }
            }
            if (!mbar_wait(&xfull_bar[buf], (slab_it >> 1) & 1, abort_flag)) { ok = false; }
          }
          const uint32_t cbase = smem_u32(smem + L::C_STAGE + buf * 16384);
          const uint32_t xbase = smem_u32(smem + L::X_STAGE + buf * 16384);
#pragma unroll
          for (int hc = 0; hc < 2; ++hc) {
            uint32_t v[32];
            tmem_ld32(tmem_base + (uint32_t(q * 32) << 16) + uint32_t(acc * BN2 + sl * 64 + hc * 32), v);
            tmem_wait_ld();
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
            if (EPI == EPI_RELU2) {
#pragma unroll
              for (int j = 0; j < 32; ++j) { const float r = fmaxf(f[j], 0.f); f[j] = r * r; }
            }
            if (L::AUX) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                const uint4 u = ld_sw128(xbase, 128, r_local, hc * 32 + j);
                const float2 a0 = unpack_bf16(u.x), a1 = unpack_bf16(u.y), a2 = unpack_bf16(u.z), a3 = unpack_bf16(u.w);
                const float ax[8] = {a0.x, a0.y, a1.x, a1.y, a2.x, a2.y, a3.x, a3.y};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  float& x = f[j + e];
                  if (EPI == EPI_NS_COMBINE) x = p.beta * ax[e] + p.gamma * x + ((row == col_s + hc * 32 + j + e) ? p.alpha : 0.f);
                  else if (EPI == EPI_RELU2_BWD) x = x * 2.f * sqrtf(fmaxf(ax[e], 0.f));
                  else x = x + ax[e];
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 u;
              u.x = pack_bf16(f[j], f[j + 1]); u.y = pack_bf16(f[j + 2], f[j + 3]);
              u.z = pack_bf16(f[j + 4], f[j + 5]); u.w = pack_bf16(f[j + 6], f[j + 7]);
              st_sw128(cbase, 128, r_local, hc * 32 + j, u);
            }
          }
          fence_proxy_async_smem();
          named_barrier(3, 128);
          if (t0 && col_s < p.N && row0 < p.M) {
            tma_store_3d(&tmC, smem + L::C_STAGE + buf * 16384, col_s, row0, b);
            tma_store_commit();
          } else if (t0) {
            tma_store_commit();                           // keep the group count in step with the slab count
          }
        }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&tempty_bar[acc]);
        else mbar_arrive_remote(mapa_u32(smem_u32(&tempty_bar[acc]), 0));
      }
    }
    if (L::STAGED && threadIdx.x == 64) tma_store_wait_all();   // staged tiles are on their way before smem goes away
  }

  tc_fence_before();
  cluster_sync_all();
  if (threadIdx.x == 0 && *abort_flag && p.err) atomicExch(p.err, ERR_GEMM_TIMEOUT);
  if (warp == 1) { __syncwarp(); tc_fence_after(); tmem_dealloc_pair(tmem_base, 512); }
}

// ------------------------------------------------------------------------------------------
static int g_num_sms = 0;
// Counters of the prologue pull: a ring per device, one slot per pulling launch (round-robin), each slot with a
// running target, so that pulling GEMMs in flight on different streams never share a counter.
constexpr int PULL_MAX_DEV = 64;
constexpr int PULL_SLOTS = 64;
static unsigned* g_pull_counter[PULL_MAX_DEV] = {nullptr};
static unsigned g_pull_total[PULL_MAX_DEV][PULL_SLOTS] = {{0}};
static unsigned g_pull_next_slot[PULL_MAX_DEV] = {0};

// Fills the counter fields of a launch of `grid_ctas` CTAs whose prologue pull is set; 0 on success.
static int arm_pull(GemmArgs& a, int grid_ctas) {
  a.pull_counter = nullptr; a.pull_target = 0;
  if (a.pull_n16 <= 0) return 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PULL_MAX_DEV) return -7;
  if (!g_pull_counter[dev]) {
    if (cudaMalloc(&g_pull_counter[dev], PULL_SLOTS * sizeof(unsigned)) != cudaSuccess) return -7;
    if (cudaMemset(g_pull_counter[dev], 0, PULL_SLOTS * sizeof(unsigned)) != cudaSuccess) return -7;
  }
  const unsigned slot = g_pull_next_slot[dev]++ % PULL_SLOTS;
  g_pull_total[dev][slot] += unsigned(grid_ctas);
  a.pull_counter = g_pull_counter[dev] + slot;
  a.pull_target = g_pull_total[dev][slot];
  return 0;
}
static int g_gemm_mode = 0;   // 0 = automatic, 1 = always 1-CTA tiles, 2 = always 2-CTA tiles

template <bool A_MN, bool B_MN, int EPI, int BN>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, cudaStream_t st) {
  using L = SmemLayout<BN>;
  auto kern = gemm_kernel<A_MN, B_MN, EPI, BN>;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return int(e);
  }
  const int items = a.batch * a.m_tiles * a.n_tiles * a.splitk;
  const int grid = items < g_num_sms ? items : g_num_sms;
  GemmArgs args = a;
  if (int r = arm_pull(args, grid)) return r;
  kern<<<grid, GEMM_THREADS, L::TOTAL, st>>>(ta, tb, args);
  return int(cudaGetLastError());
}

template <bool A_MN, bool B_MN, int EPI>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, cudaStream_t st) {
  auto kern = gemm_pair_kernel<A_MN, B_MN, EPI>;
  static PerDeviceOnce configured;
  CUtensorMap tc, tx;
  std::memset(&tc, 0, sizeof tc);
  std::memset(&tx, 0, sizeof tx);
  {
    const uint64_t es = epi_is_bf16(EPI) ? 2 : 4;
    uint64_t dims[3] = {uint64_t(a.N), uint64_t(a.M), uint64_t(a.batch)};
    uint64_t str[2] = {uint64_t(a.ldc) * es, a.batch > 1 ? uint64_t(a.stride_c) * es : uint64_t(a.M) * uint64_t(a.ldc) * es};
    uint32_t box[3] = {uint32_t(epi_is_bf16(EPI) ? 64 : 32), 128, 1};
    int r = make_tmap_typed(&tc, a.C, 3, dims, str, box,
                            epi_is_bf16(EPI) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
    if (r) return 3000 + r;
    if (epi_has_aux(EPI)) {
      r = make_tmap_bf16(&tx, a.aux, 3, dims, str, box);
      if (r) return 4000 + r;
    }
  }
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem2<EPI>::TOTAL);
    if (e != cudaSuccess) return int(e);
  }
  const int items = a.batch * a.m_tiles * a.n_tiles * a.splitk;
  int clusters = g_num_sms / 2;
  if (items < clusters) clusters = items;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(clusters * 2));
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = Smem2<EPI>::TOTAL;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GemmArgs args = a;
  if (int r = arm_pull(args, clusters * 2)) return r;
  return int(cudaLaunchKernelEx(&cfg, kern, ta, tb, tc, tx, args));
}

template <bool A_MN, bool B_MN>
static int dispatch_pair(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, cudaStream_t st) {
  switch (epi) {
    case EPI_STORE_BF16: return launch_pair<A_MN, B_MN, EPI_STORE_BF16>(ta, tb, a, st);
    case EPI_RELU2: return launch_pair<A_MN, B_MN, EPI_RELU2>(ta, tb, a, st);
    case EPI_ATOMIC_F32: return launch_pair<A_MN, B_MN, EPI_ATOMIC_F32>(ta, tb, a, st);
    case EPI_NS_COMBINE: return launch_pair<A_MN, B_MN, EPI_NS_COMBINE>(ta, tb, a, st);
    case EPI_RELU2_BWD: return launch_pair<A_MN, B_MN, EPI_RELU2_BWD>(ta, tb, a, st);
    case EPI_STORE_F32: return launch_pair<A_MN, B_MN, EPI_STORE_F32>(ta, tb, a, st);
    case EPI_ADD_AUX: return launch_pair<A_MN, B_MN, EPI_ADD_AUX>(ta, tb, a, st);
    case EPI_QKV_POST:
      if constexpr (!A_MN && !B_MN) return launch_pair<false, false, EPI_QKV_POST>(ta, tb, a, st);
      else return -3;
  }
  return -2;
}

template <bool A_MN, bool B_MN, int BN>
static int dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, cudaStream_t st) {
  switch (epi) {
    case EPI_STORE_BF16: return launch<A_MN, B_MN, EPI_STORE_BF16, BN>(ta, tb, a, st);
    case EPI_RELU2: return launch<A_MN, B_MN, EPI_RELU2, BN>(ta, tb, a, st);
    case EPI_ATOMIC_F32: return launch<A_MN, B_MN, EPI_ATOMIC_F32, BN>(ta, tb, a, st);
    case EPI_NS_COMBINE: return launch<A_MN, B_MN, EPI_NS_COMBINE, BN>(ta, tb, a, st);
    case EPI_RELU2_BWD: return launch<A_MN, B_MN, EPI_RELU2_BWD, BN>(ta, tb, a, st);
    case EPI_STORE_F32: return launch<A_MN, B_MN, EPI_STORE_F32, BN>(ta, tb, a, st);
    case EPI_ADD_AUX: return launch<A_MN, B_MN, EPI_ADD_AUX, BN>(ta, tb, a, st);
  }
  return -2;
}

}  // namespace arb

using namespace arb;

static thread_local QkvPostArgs g_qkv_post;
static thread_local bool g_qkv_post_set = false;

extern "C" int arb_gemm_qkv_post_args(const void* cos_t, const void* sin_t, float* rstd_qk, int T, int H, const void* xn,
                                      long long ld_xn, const int* ids, const void* ve_w, const void* gate_w, float* gate_out,
                                      int gate_ch, float eps) {
  g_qkv_post_set = false;
  if (!cos_t || !sin_t || !rstd_qk || T <= 0 || H <= 0) return -3;
  if ((reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t)) & 15) return -4;
  if (ve_w) {
    if (!xn || !ids || !gate_w || !gate_out || gate_ch <= 0 || (gate_ch & 7) || (ld_xn & 7)) return -3;
    if ((reinterpret_cast<uintptr_t>(xn) | reinterpret_cast<uintptr_t>(ve_w) | reinterpret_cast<uintptr_t>(gate_w)) & 15) return -4;
  }
  QkvPostArgs& q = g_qkv_post;
  q.cos_t = (const __nv_bfloat16*)cos_t; q.sin_t = (const __nv_bfloat16*)sin_t; q.rstd = rstd_qk; q.T = T; q.H = H;
  q.xn = (const __nv_bfloat16*)xn; q.ld_xn = ld_xn; q.ids = ids; q.ve = (const __nv_bfloat16*)ve_w;
  q.gate_w = (const __nv_bfloat16*)gate_w; q.gate = gate_out; q.gate_ch = gate_ch; q.eps = eps;
  g_qkv_post_set = true;
  return 0;
}

extern "C" int arb_gemm_set_mode(int mode) {
  if (mode < 0 || mode > 2) return -3;
  g_gemm_mode = mode;
  return 0;
}
static bool bad_copy(const void* src, const void* dst, long long bytes) {
  return !src || !dst || bytes <= 0 || (bytes & 15) ||
         ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15);
}

extern "C" int arb_gemm_bf16(const void* A, const void* B, void* C, const void* aux, int M, int N, int K, int batch,
                             long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                             long long stride_c, int a_mn_major, int b_mn_major, int epi, int splitk, float alpha,
                             float beta, float gamma, int* err_flag, cudaStream_t stream) {
  return arb_gemm_bf16_ex(A, B, C, aux, M, N, K, batch, lda, ldb, ldc, stride_a, stride_b, stride_c, a_mn_major, b_mn_major,
                          epi, splitk, alpha, beta, gamma, err_flag, stream, nullptr, 0, nullptr, nullptr, 0);
}

extern "C" int arb_gemm_bf16_ex(const void* A, const void* B, void* C, const void* aux, int M, int N, int K, int batch,
                                long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                                long long stride_c, int a_mn_major, int b_mn_major, int epi, int splitk, float alpha,
                                float beta, float gamma, int* err_flag, cudaStream_t stream, const void* pull_src,
                                long long pull_bytes, const void* ahead_src, void* ahead_dst, long long ahead_bytes) {
  return arb_gemm_bf16_ragged(A, B, C, aux, M, N, K, batch, lda, ldb, ldc, stride_a, stride_b, stride_c, a_mn_major, b_mn_major,
                              epi, splitk, alpha, beta, gamma, err_flag, stream, pull_src, pull_bytes, ahead_src, ahead_dst,
                              ahead_bytes, nullptr, 1, nullptr, 0);
}

extern "C" int arb_gemm_bf16_ragged(const void* A, const void* B, void* C, const void* aux, int M, int N, int K, int batch,
                                    long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                                    long long stride_c, int a_mn_major, int b_mn_major, int epi, int splitk, float alpha,
                                    float beta, float gamma, int* err_flag, cudaStream_t stream, const void* pull_src,
                                    long long pull_bytes, const void* ahead_src, void* ahead_dst, long long ahead_bytes,
                                    const int* m_valid, int b_div, const int* k_valid, int k_seg_rows) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return -3;
  if (b_div < 1 || batch % b_div) return -3;
  if (k_valid && (k_seg_rows <= 0 || (k_seg_rows % BK) || (K % k_seg_rows) || epi != EPI_ATOMIC_F32)) return -3;
  if (pull_src && bad_copy(pull_src, B, pull_bytes)) return -3;
  if (ahead_src && bad_copy(ahead_src, ahead_dst, ahead_bytes)) return -3;
  // TMA needs 16-byte aligned bases and row strides; vector epilogue needs ldc % 8 == 0.
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return -4;
  if ((lda % 8) || (ldb % 8) || (stride_a % 8) || (stride_b % 8)) return -4;
  const bool c_f32 = (epi == EPI_ATOMIC_F32 || epi == EPI_STORE_F32);
  if (ldc % (c_f32 ? 4 : 8)) return -4;
  if (aux && (reinterpret_cast<uintptr_t>(aux) & 15)) return -4;
  if ((epi == EPI_NS_COMBINE || epi == EPI_RELU2_BWD || epi == EPI_ADD_AUX) && !aux) return -5;
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const int BN = (N > 128) ? 256 : 128;
  // 2-CTA tiles (256 x 256) for problems that are large in both output dimensions
  const bool pair = (g_gemm_mode != 1) && (g_gemm_mode == 2 || (M >= 512 && N >= 256));
  const int bm_eff = pair ? 256 : BM;
  GemmArgs a;
  a.M = M; a.N = N; a.K = K; a.batch = batch;
  a.m_tiles = (M + bm_eff - 1) / bm_eff;
  a.n_tiles = pair ? (N + 255) / 256 : (N + BN - 1) / BN;
  a.kb_total = (K + BK - 1) / BK;
  if (epi != EPI_ATOMIC_F32) splitk = 1;
  if (splitk <= 0) {  // automatic: fill the SMs when there are few output tiles
    const int tiles = batch * a.m_tiles * a.n_tiles;
    const int units = pair ? g_num_sms / 2 : g_num_sms;     // CTAs, or CTA pairs, that can run at once
    int max_split = a.kb_total / 8 > 0 ? a.kb_total / 8 : 1;        // at least 8 K blocks per split
    if (max_split > 32) max_split = 32;
    // pick the split that fills the last wave best: efficiency = items / (waves * units)
    splitk = 1;
    double best = 0.0;
    for (int sp = 1; sp <= max_split; ++sp) {
      const long long it = (long long)tiles * sp;
      const long long waves = (it + units - 1) / units;
      const double eff = double(it) / double(waves * units);
      if (eff > best + 0.02) { best = eff; splitk = sp; }
    }
  }
  if (splitk > a.kb_total) splitk = a.kb_total;
  a.kb_per_split = (a.kb_total + splitk - 1) / splitk;
  a.splitk = (a.kb_total + a.kb_per_split - 1) / a.kb_per_split;
  a.C = C; a.aux = aux; a.ldc = ldc; a.stride_c = stride_c;
  a.alpha = alpha; a.beta = beta; a.gamma = gamma; a.err = err_flag;
  a.pull_src = reinterpret_cast<const uint4*>(pull_src);
  a.pull_dst = reinterpret_cast<uint4*>(const_cast<void*>(B));
  a.pull_n16 = pull_src ? pull_bytes / 16 : 0;
  a.ahead_src = reinterpret_cast<const uint4*>(ahead_src);
  a.ahead_dst = reinterpret_cast<uint4*>(ahead_dst);
  a.ahead_n16 = ahead_src ? ahead_bytes / 16 : 0;
  a.m_valid = m_valid; a.b_div = b_div; a.k_valid = k_valid;
  a.k_seg_kb = k_valid ? k_seg_rows / BK : 1;
  a.k_nseg = k_valid ? K / k_seg_rows : 1;
  std::memset(&a.qp, 0, sizeof a.qp);
  if (epi == EPI_QKV_POST) {
    const bool have = g_qkv_post_set;
    g_qkv_post_set = false;
    if (!have || !pair || a_mn_major || b_mn_major || batch != 1 || N != 3 * g_qkv_post.H * 128) return -6;
    a.qp = g_qkv_post;
  }

  CUtensorMap ta, tb;
  {
    uint64_t dims[3], str[2];
    uint32_t box[3];
    if (a_mn_major) { dims[0] = uint64_t(M); dims[1] = uint64_t(K); box[0] = 64; box[1] = BK; }
    else { dims[0] = uint64_t(K); dims[1] = uint64_t(M); box[0] = BK; box[1] = 128; }
    dims[2] = uint64_t(batch); box[2] = 1;
    str[0] = uint64_t(lda) * 2;
    str[1] = batch > 1 ? uint64_t(stride_a) * 2 : dims[1] * str[0];
    int r = make_tmap_bf16(&ta, A, 3, dims, str, box);
    if (r) return 1000 + r;
    if (b_mn_major) { dims[0] = uint64_t(N); dims[1] = uint64_t(K); box[0] = 64; box[1] = BK; }
    else { dims[0] = uint64_t(K); dims[1] = uint64_t(N); box[0] = BK; box[1] = uint32_t(pair ? 128 : BN); }
    dims[2] = uint64_t(batch / b_div);
    str[0] = uint64_t(ldb) * 2;
    str[1] = batch > 1 ? uint64_t(stride_b) * 2 : dims[1] * str[0];
    r = make_tmap_bf16(&tb, B, 3, dims, str, box);
    if (r) return 2000 + r;
  }
  if (pair) {
    if (!a_mn_major && !b_mn_major) return dispatch_pair<false, false>(epi, ta, tb, a, stream);
    if (!a_mn_major && b_mn_major) return dispatch_pair<false, true>(epi, ta, tb, a, stream);
    if (a_mn_major && b_mn_major) return dispatch_pair<true, true>(epi, ta, tb, a, stream);
    return dispatch_pair<true, false>(epi, ta, tb, a, stream);
  }
#define ARB_DISPATCH(AM, BMJ)                                                                              \
  (BN == 256 ? dispatch_epi<AM, BMJ, 256>(epi, ta, tb, a, stream) : dispatch_epi<AM, BMJ, 128>(epi, ta, tb, a, stream))
  if (!a_mn_major && !b_mn_major) return ARB_DISPATCH(false, false);
  if (!a_mn_major && b_mn_major) return ARB_DISPATCH(false, true);
  if (a_mn_major && b_mn_major) return ARB_DISPATCH(true, true);
  return ARB_DISPATCH(true, false);
#undef ARB_DISPATCH
}
