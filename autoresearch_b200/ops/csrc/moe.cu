// Mixture-of-experts kernels: fused router (logits + softmax + top-k + renormalised gates),
// its backward, and the dispatch / combine data movement.  Dispatch writes token rows straight
// into the owning expert's buffer and combine reads expert outputs straight from it; the buffers
// are addressed through a per-expert pointer table, so with expert parallelism those pointers are
// NVLink peer mappings and the all-to-all happens inside these kernels (peer stores on dispatch,
// peer loads on combine) - no library collective, no host synchronisation.
//
// Reference counterparts (single GPU, host-synchronised, experts looped through cuBLAS):
// brain/kernels/moe_dispatch.cu:39-488, moe_backward.cu:48-325, moe_aux_loss.cu:25-114.
// Slot order inside an expert is the token order (deterministic), where the reference claims
// slots with atomics.
#include "api.h"
#include "ptx.cuh"

namespace arb {

constexpr int MOE_MAX_E = 32;
constexpr int MOE_MAX_K = 4;
struct ExpertPtrs { void* p[MOE_MAX_E]; };

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// one warp per token
__global__ void __launch_bounds__(256) moe_router_fwd_k(const __nv_bfloat16* __restrict__ xn, const __nv_bfloat16* __restrict__ wr,
                                                        float* __restrict__ probs, int* __restrict__ idx, float* __restrict__ gates,
                                                        long long N, int D, int E, int K) {
  extern __shared__ __nv_bfloat16 w_s[];   // [E, D]
  for (int i = threadIdx.x; i < E * D; i += blockDim.x) w_s[i] = wr[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long tok = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= N) return;
  float logit[MOE_MAX_E];
#pragma unroll 1
  for (int e = 0; e < E; ++e) {
    float acc = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      uint4 a = *reinterpret_cast<const uint4*>(xn + tok * D + c);
      uint4 b = *reinterpret_cast<const uint4*>(w_s + e * D + c);
      float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), a2 = unpack_bf16(a.z), a3 = unpack_bf16(a.w);
      float2 b0 = unpack_bf16(b.x), b1 = unpack_bf16(b.y), b2 = unpack_bf16(b.z), b3 = unpack_bf16(b.w);
      acc += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
    }
    logit[e] = wsum(acc);
  }
  if (lane == 0) {
    float mx = logit[0];
    for (int e = 1; e < E; ++e) mx = fmaxf(mx, logit[e]);
    float sum = 0.f;
    for (int e = 0; e < E; ++e) { logit[e] = __expf(logit[e] - mx); sum += logit[e]; }
    const float inv = 1.f / sum;
    for (int e = 0; e < E; ++e) { logit[e] *= inv; probs[tok * E + e] = logit[e]; }
    int sel[MOE_MAX_K];
    float top = 0.f;
    for (int k = 0; k < K; ++k) {
      int best = -1;
      float bv = -1.f;
      for (int e = 0; e < E; ++e) {
        bool used = false;
        for (int j = 0; j < k; ++j) used |= (sel[j] == e);
        if (!used && logit[e] > bv) { bv = logit[e]; best = e; }   // ties -> lower index
      }
      sel[k] = best;
      top += bv;
    }
    for (int k = 0; k < K; ++k) { idx[tok * K + k] = sel[k]; gates[tok * K + k] = logit[sel[k]] / top; }
  }
}

// d_logits = softmax_bwd(top-k renormalisation bwd(d_gates) + aux term); one thread per token
__global__ void moe_router_bwd_k(const float* __restrict__ probs, const int* __restrict__ idx, const float* __restrict__ gates,
                                 const float* __restrict__ d_gates, const float* __restrict__ aux_dp,
                                 __nv_bfloat16* __restrict__ d_logits, long long ld, long long N, int E, int K) {
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= N) return;
  float dp[MOE_MAX_E];
  for (int e = 0; e < E; ++e) dp[e] = aux_dp ? aux_dp[e] : 0.f;
  float s = 0.f, dot = 0.f;
  for (int k = 0; k < K; ++k) { s += probs[t * E + idx[t * K + k]]; dot += d_gates[t * K + k] * gates[t * K + k]; }
  for (int k = 0; k < K; ++k) dp[idx[t * K + k]] += (d_gates[t * K + k] - dot) / s;
  float pd = 0.f;
  for (int e = 0; e < E; ++e) pd += probs[t * E + e] * dp[e];
  for (int e = 0; e < E; ++e) d_logits[t * ld + e] = __float2bfloat16(probs[t * E + e] * (dp[e] - pd));
}

// slot (t, k) with row >= 0: expert_buf[idx][row, :] = x[t, :]      (one warp per slot)
__global__ void __launch_bounds__(256) moe_dispatch_k(const __nv_bfloat16* __restrict__ x, ExpertPtrs bufs, const int* __restrict__ idx,
                                                      const int* __restrict__ row, long long slots, int K, int D) {
  const long long s = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (s >= slots) return;
  const int r = row[s];
  if (r < 0) return;
  const long long t = s / K;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(bufs.p[idx[s]]) + (long long)r * D;
  for (int c = (threadIdx.x & 31) * 8; c < D; c += 256)
    *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(x + t * D + c);
}

// After a dispatch: for every expert e, c = min(counts[e], keep) (keep <= cap = rows of a slab) is written to *cnt[e] (the entry of this source in the
// owner's row-count table; a peer store with expert parallelism) and the rows [c, next multiple of `tile`) of the
// expert's slab are zeroed, so that the grouped GEMMs, which work in whole tiles and skip everything beyond, never
// multiply stale rows.  grid (E, tile / 8), one warp per row.
struct CountPtrs { int* p[MOE_MAX_E]; };
__global__ void __launch_bounds__(256) moe_finish_dispatch_k(ExpertPtrs bufs, CountPtrs cnt, const int* __restrict__ counts, int keep,
                                                             int cap, int D, int tile) {
  const int e = blockIdx.x;
  const int c = min(counts[e], keep);
  if (blockIdx.y == 0 && threadIdx.x == 0 && cnt.p[e]) *cnt.p[e] = c;
  const int r = c + int(blockIdx.y) * 8 + (threadIdx.x >> 5);
  const int end = min((c + tile - 1) / tile * tile, cap);
  if (r >= end) return;
  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(bufs.p[e]) + (long long)r * D;
  for (int col = (threadIdx.x & 31) * 8; col < D; col += 256) *reinterpret_cast<uint4*>(dst + col) = make_uint4(0, 0, 0, 0);
}

// out[t] = resid[t] + sum_k gate[t,k] * y_buf[idx][row]       (one warp per token)
__global__ void __launch_bounds__(256) moe_combine_fwd_k(const __nv_bfloat16* __restrict__ resid, ExpertPtrs bufs, const int* __restrict__ idx,
                                                         const int* __restrict__ row, const float* __restrict__ gates,
                                                         __nv_bfloat16* __restrict__ out, long long N, int K, int D) {
  const long long t = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= N) return;
  for (int c = (threadIdx.x & 31) * 8; c < D; c += 256) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (resid) {
      uint4 u = *reinterpret_cast<const uint4*>(resid + t * D + c);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] = a.x; acc[1] = a.y; acc[2] = b.x; acc[3] = b.y; acc[4] = cc.x; acc[5] = cc.y; acc[6] = d.x; acc[7] = d.y;
    }
    for (int k = 0; k < K; ++k) {
      const int r = row[t * K + k];
      if (r < 0) continue;
      const float g = gates ? gates[t * K + k] : 1.f;
      uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.p[idx[t * K + k]]) + (long long)r * D + c);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += g * a.x; acc[1] += g * a.y; acc[2] += g * b.x; acc[3] += g * b.y;
      acc[4] += g * cc.x; acc[5] += g * cc.y; acc[6] += g * d.x; acc[7] += g * d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]); o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + t * D + c) = o;
  }
}

// d_y_buf[idx][row] = gate * d_out[t] ; d_gate[t,k] = <y_buf[idx][row], d_out[t]>    (one warp per slot)
__global__ void __launch_bounds__(256) moe_combine_bwd_k(const __nv_bfloat16* __restrict__ d_out, ExpertPtrs ybufs,
                                                         const __nv_bfloat16* __restrict__ y_rows, ExpertPtrs dybufs,
                                                         const int* __restrict__ idx, const int* __restrict__ row,
                                                         const float* __restrict__ gates, float* __restrict__ d_gates,
                                                         long long slots, int K, int D) {
  const long long s = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (s >= slots) return;
  const int lane = threadIdx.x & 31;
  const int r = row[s];
  if (r < 0) { if (lane == 0) d_gates[s] = 0.f; return; }
  const long long t = s / K;
  const float g = gates[s];
  const __nv_bfloat16* y = y_rows ? y_rows + s * D
                                  : reinterpret_cast<const __nv_bfloat16*>(ybufs.p[idx[s]]) + (long long)r * D;
  __nv_bfloat16* dy = reinterpret_cast<__nv_bfloat16*>(dybufs.p[idx[s]]) + (long long)r * D;
  float dot = 0.f;
  for (int c = lane * 8; c < D; c += 256) {
    uint4 u = *reinterpret_cast<const uint4*>(d_out + t * D + c);
    uint4 w = *reinterpret_cast<const uint4*>(y + c);
    float2 a0 = unpack_bf16(u.x), a1 = unpack_bf16(u.y), a2 = unpack_bf16(u.z), a3 = unpack_bf16(u.w);
    float2 b0 = unpack_bf16(w.x), b1 = unpack_bf16(w.y), b2 = unpack_bf16(w.z), b3 = unpack_bf16(w.w);
    dot += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y + a2.x * b2.x + a2.y * b2.y + a3.x * b3.x + a3.y * b3.y;
    uint4 o;
    o.x = pack_bf16(g * a0.x, g * a0.y); o.y = pack_bf16(g * a1.x, g * a1.y);
    o.z = pack_bf16(g * a2.x, g * a2.y); o.w = pack_bf16(g * a3.x, g * a3.y);
    *reinterpret_cast<uint4*>(dy + c) = o;
  }
  dot = wsum(dot);
  if (lane == 0) d_gates[s] = dot;
}

static int fill_ptrs(ExpertPtrs& ep, void* const* host_ptrs, int E) {
  if (E < 1 || E > MOE_MAX_E) return -3;
  for (int e = 0; e < E; ++e) {
    if (reinterpret_cast<uintptr_t>(host_ptrs[e]) & 15) return -4;
    ep.p[e] = host_ptrs[e];
  }
  return 0;
}

}  // namespace arb

using namespace arb;
typedef __nv_bfloat16 bf16;


// ------------------------------------------------------------------------------------------------
// Slot positions: pos[s] = number of earlier slots (token-major order) routed to the same expert,
// i.e. the row a slot takes in its expert's buffer; counts[e] = slots per expert.  Deterministic
// two-pass prefix sum over chunks of 1024 slots (the reference uses atomics and a host-synchronised
// offset table, brain/kernels/moe_dispatch.cu:154-230).
// ------------------------------------------------------------------------------------------------
constexpr int SLOT_CHUNK = 1024;

__global__ void __launch_bounds__(SLOT_CHUNK) moe_slot_count_k(const int* __restrict__ idx, long long S, int E, int* __restrict__ chunk_counts) {
  __shared__ int cnt[MOE_MAX_E];
  if (threadIdx.x < E) cnt[threadIdx.x] = 0;
  __syncthreads();
  const long long s = (long long)blockIdx.x * SLOT_CHUNK + threadIdx.x;
  const int e = (s < S) ? idx[s] : -1;
  for (int x = 0; x < E; ++x) {
    const unsigned m = __ballot_sync(0xffffffffu, e == x);
    if ((threadIdx.x & 31) == 0 && m) atomicAdd(&cnt[x], __popc(m));   // integer adds: order does not matter
  }
  __syncthreads();
  if (threadIdx.x < E) chunk_counts[(long long)blockIdx.x * E + threadIdx.x] = cnt[threadIdx.x];
}

__global__ void __launch_bounds__(SLOT_CHUNK) moe_slot_pos_k(const int* __restrict__ idx, long long S, int E,
                                                           const int* __restrict__ chunk_counts, int n_chunks,
                                                           int* __restrict__ pos, int* __restrict__ counts) {
  __shared__ int base[MOE_MAX_E];               // slots of expert e in earlier chunks
  __shared__ int warp_cnt[32][MOE_MAX_E + 1];   // per warp, per expert, inside this chunk
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < E) {
    int b = 0, tot = 0;
    for (int c = 0; c < n_chunks; ++c) {
      const int v = chunk_counts[(long long)c * E + threadIdx.x];
      if (c < int(blockIdx.x)) b += v;
      tot += v;
    }
    base[threadIdx.x] = b;
    if (blockIdx.x == 0) counts[threadIdx.x] = tot;
  }
  const long long s = (long long)blockIdx.x * SLOT_CHUNK + threadIdx.x;
  const int e = (s < S) ? idx[s] : -1;
  int in_warp = 0;
  for (int x = 0; x < E; ++x) {
    const unsigned m = __ballot_sync(0xffffffffu, e == x);
    if (e == x) in_warp = __popc(m & ((1u << lane) - 1u));
    if (lane == 0) warp_cnt[warp][x] = __popc(m);
  }
  __syncthreads();
  if (e >= 0) {
    int before = base[e];
    for (int w = 0; w < warp; ++w) before += warp_cnt[w][e];
    pos[s] = before + in_warp;
  }
}

extern "C" {

int arb_moe_router_fwd(const void* xn, const void* wr, float* probs, int* idx, float* gates, long long N, int D, int E, int K,
                       cudaStream_t s) {
  if (N <= 0 || D <= 0 || (D & 7) || E < 1 || E > MOE_MAX_E || K < 1 || K > MOE_MAX_K || K > E) return -3;
  if ((reinterpret_cast<uintptr_t>(xn) | reinterpret_cast<uintptr_t>(wr)) & 15) return -4;
  const size_t smem = size_t(E) * D * 2;
  if (smem > 200 * 1024) return -3;
  static PerDeviceOnce cfg;
  if (cfg.first()) {
    cudaError_t e = cudaFuncSetAttribute(moe_router_fwd_k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return int(e);
  }
  moe_router_fwd_k<<<unsigned((N + 7) / 8), 256, smem, s>>>((const bf16*)xn, (const bf16*)wr, probs, idx, gates, N, D, E, K);
  return int(cudaGetLastError());
}

int arb_moe_router_bwd(const float* probs, const int* idx, const float* gates, const float* d_gates, const float* aux_dp,
                       void* d_logits, long long ld, long long N, int E, int K, cudaStream_t s) {
  if (N <= 0 || E < 1 || E > MOE_MAX_E || K < 1 || K > MOE_MAX_K || ld < E) return -3;
  moe_router_bwd_k<<<unsigned((N + 255) / 256), 256, 0, s>>>(probs, idx, gates, d_gates, aux_dp, (bf16*)d_logits, ld, N, E, K);
  return int(cudaGetLastError());
}

int arb_moe_dispatch(const void* x, void* const* expert_bufs, const int* idx, const int* row, long long N, int K, int D, int E,
                     cudaStream_t s) {
  ExpertPtrs ep;
  int rc = fill_ptrs(ep, expert_bufs, E);
  if (rc || N <= 0 || (D & 7)) return rc ? rc : -3;
  moe_dispatch_k<<<unsigned((N * K + 7) / 8), 256, 0, s>>>((const bf16*)x, ep, idx, row, N * K, K, D);
  return int(cudaGetLastError());
}

int arb_moe_finish_dispatch(void* const* expert_bufs, int* const* count_slots, const int* counts, int keep, int cap, int D, int E,
                            int tile, cudaStream_t s) {
  ExpertPtrs ep;
  int rc = fill_ptrs(ep, expert_bufs, E);
  if (rc || cap <= 0 || keep < 0 || keep > cap || (D & 7) || tile < 8 || tile > 256 || (tile & 7)) return rc ? rc : -3;
  CountPtrs cp;
  for (int e = 0; e < E; ++e) cp.p[e] = count_slots ? count_slots[e] : nullptr;
  moe_finish_dispatch_k<<<dim3(unsigned(E), unsigned(tile / 8)), 256, 0, s>>>(ep, cp, counts, keep, cap, D, tile);
  return int(cudaGetLastError());
}

int arb_moe_combine_fwd(const void* resid, void* const* expert_bufs, const int* idx, const int* row, const float* gates, void* out,
                        long long N, int K, int D, int E, cudaStream_t s) {
  ExpertPtrs ep;
  int rc = fill_ptrs(ep, expert_bufs, E);
  if (rc || N <= 0 || (D & 7)) return rc ? rc : -3;
  moe_combine_fwd_k<<<unsigned((N + 7) / 8), 256, 0, s>>>((const bf16*)resid, ep, idx, row, gates, (bf16*)out, N, K, D);
  return int(cudaGetLastError());
}

int arb_moe_combine_bwd(const void* d_out, void* const* y_bufs, const void* y_rows, void* const* dy_bufs, const int* idx,
                        const int* row, const float* gates, float* d_gates, long long N, int K, int D, int E, cudaStream_t s) {
  ExpertPtrs ey{}, ed;
  int rc = 0;
  if (!y_rows) rc = fill_ptrs(ey, y_bufs, E);
  else if (reinterpret_cast<uintptr_t>(y_rows) & 15) rc = -4;
  if (!rc) rc = fill_ptrs(ed, dy_bufs, E);
  if (rc || N <= 0 || (D & 7)) return rc ? rc : -3;
  moe_combine_bwd_k<<<unsigned((N * K + 7) / 8), 256, 0, s>>>((const bf16*)d_out, ey, (const bf16*)y_rows, ed, idx, row, gates, d_gates,
                                                             N * K, K, D);
  return int(cudaGetLastError());
}

// pos[S], counts[E]; scratch: int[ceil(S/1024) * E]
int arb_moe_slot_positions(const int* idx, long long S, int E, int* scratch, int* pos, int* counts, cudaStream_t s) {
  if (S <= 0 || E < 1 || E > MOE_MAX_E) return -3;
  const long long chunks = (S + SLOT_CHUNK - 1) / SLOT_CHUNK;
  if (chunks > 65535) return -3;
  moe_slot_count_k<<<unsigned(chunks), SLOT_CHUNK, 0, s>>>(idx, S, E, scratch);
  moe_slot_pos_k<<<unsigned(chunks), SLOT_CHUNK, 0, s>>>(idx, S, E, scratch, int(chunks), pos, counts);
  return int(cudaGetLastError());
}

}  // extern "C"
