// Soft-capped cross entropy over a chunk of logits, forward and backward in one pass.
// Math: s = cap*tanh(x/cap); loss = logsumexp(s) - s[tgt];
//       d_logit = (softmax(s) - 1[tgt]) * scale * (1 - (s/cap)^2)
// (brain/kernels/cross_entropy.cu:60-150).  The reference runs a forward kernel, recomputes
// the logits GEMM in backward and runs a second kernel; here each row is read once into
// registers and, when a gradient scale is given, overwritten in place by its gradient.
#include "api.h"
#include "ptx.cuh"

namespace arb {

constexpr int CE_THREADS = 256;

template <int VPT>  // 8-element vectors per thread
__global__ void __launch_bounds__(CE_THREADS) softcap_ce_k(__nv_bfloat16* __restrict__ logits, long long ld,
                                                           const int* __restrict__ targets, float* __restrict__ loss,
                                                           int V, float cap, float gscale) {
  __shared__ float red[CE_THREADS / 32];
  __shared__ float bcast;
  const long long row = blockIdx.x;
  __nv_bfloat16* p = logits + row * ld;
  const int nch = V >> 3;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float inv_cap = 1.f / cap;
  float s[VPT][8];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = tid + CE_THREADS * i;
    if (c < nch) {
      uint4 u = *reinterpret_cast<const uint4*>(p + c * 8);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), cc = unpack_bf16(u.z), d = unpack_bf16(u.w);
      float x[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, d.x, d.y};
#pragma unroll
      for (int j = 0; j < 8; ++j) { s[i][j] = cap * tanhf(x[j] * inv_cap); mx = fmaxf(mx, s[i][j]); }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (tid == 0) { float m = red[0]; for (int w = 1; w < CE_THREADS / 32; ++w) m = fmaxf(m, red[w]); bcast = m; }
  __syncthreads();
  mx = bcast;
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = tid + CE_THREADS * i;
    if (c < nch) {
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += __expf(s[i][j] - mx);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (tid == 0) { float t = 0.f; for (int w = 0; w < CE_THREADS / 32; ++w) t += red[w]; bcast = t; }
  __syncthreads();
  sum = bcast;
  const float lse = mx + __logf(sum);
  int tgt = targets[row];
  const bool tgt_ok = tgt >= 0 && tgt < V;
  if (tid == 0) {
    float st = 0.f;
    if (tgt_ok) st = cap * tanhf(__bfloat162float(p[tgt]) * inv_cap);
    loss[row] = tgt_ok ? (lse - st) : 0.f;
  }
  if (gscale != 0.f) {
    __syncthreads();  // p[tgt] has been read before anyone overwrites it
    const float inv_sum = 1.f / sum;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = tid + CE_THREADS * i;
      if (c < nch) {
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float pr = __expf(s[i][j] - mx) * inv_sum;
          const float t = s[i][j] * inv_cap;
          const float ind = (tgt_ok && (c * 8 + j == tgt)) ? 1.f : 0.f;
          g[j] = tgt_ok ? (pr - ind) * gscale * (1.f - t * t) : 0.f;
        }
        uint4 u;
        u.x = pack_bf16(g[0], g[1]); u.y = pack_bf16(g[2], g[3]); u.z = pack_bf16(g[4], g[5]); u.w = pack_bf16(g[6], g[7]);
        *reinterpret_cast<uint4*>(p + c * 8) = u;
      }
    }
  }
}

}  // namespace arb

using namespace arb;

extern "C" int arb_softcap_ce(void* logits, long long ld, const int* targets, float* loss, long long rows, int V,
                              float softcap, float dlogits_scale, cudaStream_t s) {
  if (rows <= 0 || V <= 0 || (V & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(logits) & 15) || softcap <= 0.f) return -3;
  const int nch = V / 8;
  const int vpt = (nch + CE_THREADS - 1) / CE_THREADS;
  __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(logits);
  if (vpt <= 1) softcap_ce_k<1><<<unsigned(rows), CE_THREADS, 0, s>>>(p, ld, targets, loss, V, softcap, dlogits_scale);
  else if (vpt <= 2) softcap_ce_k<2><<<unsigned(rows), CE_THREADS, 0, s>>>(p, ld, targets, loss, V, softcap, dlogits_scale);
  else if (vpt <= 4) softcap_ce_k<4><<<unsigned(rows), CE_THREADS, 0, s>>>(p, ld, targets, loss, V, softcap, dlogits_scale);
  else if (vpt <= 8) softcap_ce_k<8><<<unsigned(rows), CE_THREADS, 0, s>>>(p, ld, targets, loss, V, softcap, dlogits_scale);
  else if (vpt <= 16) softcap_ce_k<16><<<unsigned(rows), CE_THREADS, 0, s>>>(p, ld, targets, loss, V, softcap, dlogits_scale);
  else return -3;  // vocabularies above 32768 are not supported by this kernel
  return int(cudaGetLastError());
}
