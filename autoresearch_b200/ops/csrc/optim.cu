// Optimizer kernels: fused AdamW on fp32 masters, and the elementwise parts of Muon
// (Nesterov momentum + Frobenius norm, NorMuon statistics, cautious update).
// Math: brain/kernels/adamw.cu:9-76, brain/kernels/muon.cu:63-177,244-356,89-112.
// Differences from the reference's launch structure: one launch per shape group instead of
// several per matrix, the Frobenius partial sums are produced by the momentum kernel, and the
// update writes the fp32 master and the bf16 parameter together.
#include "api.h"
#include "ptx.cuh"

namespace arb {

__global__ void adamw_k(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                        __nv_bfloat16* __restrict__ shadow, long long n, float lr, float b1, float b2, float eps, float wd,
                        float bc1, float bc2) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float pi = p[i], gi = g[i], mi = m[i], vi = v[i];
    pi -= lr * wd * pi;
    mi = b1 * mi + (1.f - b1) * gi;
    vi = b2 * vi + (1.f - b2) * gi * gi;
    pi -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    p[i] = pi; m[i] = mi; v[i] = vi;
    if (shadow) shadow[i] = __float2bfloat16(pi);
  }
}

// grid: (blocks_per_mat, n_mat)
__global__ void __launch_bounds__(256) muon_nesterov_k(float* __restrict__ buf, const float* __restrict__ g,
                                                       __nv_bfloat16* __restrict__ u, float* __restrict__ sumsq,
                                                       long long per_mat, float mu) {
  __shared__ float red[8];
  const int mat = blockIdx.y;
  const long long base = (long long)mat * per_mat;
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_mat; i += (long long)gridDim.x * blockDim.x) {
    const float gi = g[base + i];
    const float b = mu * buf[base + i] + (1.f - mu) * gi;
    buf[base + i] = b;
    const __nv_bfloat16 ub = __float2bfloat16((1.f - mu) * gi + mu * b);
    u[base + i] = ub;
    const float uf = __bfloat162float(ub);
    acc += uf * uf;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    atomicAdd(sumsq + mat, t);
  }
}

__global__ void muon_frob_scale_k(__nv_bfloat16* __restrict__ u, const float* __restrict__ sumsq, long long per_mat) {
  const int mat = blockIdx.y;
  const float inv = 1.f / (sqrtf(sumsq[mat]) * 1.02f + 1e-6f);
  const long long base = (long long)mat * per_mat;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_mat; i += (long long)gridDim.x * blockDim.x)
    u[base + i] = __float2bfloat16(__bfloat162float(u[base + i]) * inv);
}

// v_mean[mat, r] = mean_c x[mat, r, c]^2 (ROWS=true, one warp per row) or the column version
// (ROWS=false: one thread per column, coalesced across threads).
template <bool ROWS>
__global__ void __launch_bounds__(256) normuon_stats_k(const __nv_bfloat16* __restrict__ x, float* __restrict__ v_mean, int m, int n) {
  const int mat = blockIdx.y;
  const __nv_bfloat16* xm = x + (long long)mat * m * n;
  if (ROWS) {
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (r >= m) return;
    float acc = 0.f;
    for (int c = threadIdx.x & 31; c < n; c += 32) { const float f = __bfloat162float(xm[(long long)r * n + c]); acc += f * f; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) v_mean[(long long)mat * m + r] = acc / n;
  } else {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= n) return;
    float acc = 0.f;
    for (int r = 0; r < m; ++r) { const float f = __bfloat162float(xm[(long long)r * n + c]); acc += f * f; }
    v_mean[(long long)mat * n + c] = acc / m;
  }
}

// one CTA per matrix: EMA of the statistic, rsqrt step, norm-preserving rescale factor
__global__ void __launch_bounds__(256) normuon_scales_k(const float* __restrict__ v_mean, float* __restrict__ second,
                                                        float* __restrict__ scale, int n_stat, int red_size, float beta2) {
  __shared__ float red[2][8];
  const int mat = blockIdx.x;
  const float* v = v_mean + (long long)mat * n_stat;
  float* sm = second + (long long)mat * n_stat;
  float a = 0.f, b = 0.f;
  for (int i = threadIdx.x; i < n_stat; i += blockDim.x) {
    const float vi = v[i];
    const float s = beta2 * sm[i] + (1.f - beta2) * vi;
    sm[i] = s;
    const float ss = rsqrtf(fmaxf(s, 1e-10f));
    a += vi * red_size;
    b += vi * red_size * ss * ss;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = a; red[1][threadIdx.x >> 5] = b; }
  __syncthreads();
  a = 0.f; b = 0.f;
  for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; }
  const float ratio = sqrtf(a) / fmaxf(sqrtf(b), 1e-10f);
  for (int i = threadIdx.x; i < n_stat; i += blockDim.x)
    scale[(long long)mat * n_stat + i] = rsqrtf(fmaxf(sm[i], 1e-10f)) * ratio;
}

// g = x*scale[row or col]; mask = (g*p >= 0); p -= lr*g + lr*wd*p*mask
template <bool ROWS>
__global__ void muon_update_k(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow, const __nv_bfloat16* __restrict__ x,
                              const float* __restrict__ scale, int m, int n, float lr, float wd) {
  const int mat = blockIdx.y;
  const long long per = (long long)m * n;
  const int n_stat = ROWS ? m : n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / n), c = int(i - (long long)r * n);
    const float g = __bfloat162float(x[mat * per + i]) * scale[(long long)mat * n_stat + (ROWS ? r : c)];
    float p = master[mat * per + i];
    const float mask = (g * p >= 0.f) ? 1.f : 0.f;
    p -= lr * g + lr * wd * p * mask;
    master[mat * per + i] = p;
    shadow[mat * per + i] = __float2bfloat16(p);
  }
}

static inline int blocks_for(long long n, int threads, int cap) {
  long long b = (n + threads - 1) / threads;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace arb

using namespace arb;

extern "C" {

int arb_adamw(float* master, const float* grad, float* m, float* v, void* shadow_bf16, long long n, float lr, float beta1,
              float beta2, float eps, float wd, float bc1, float bc2, cudaStream_t s) {
  if (n <= 0) return -3;
  adamw_k<<<blocks_for(n, 256, 148 * 8), 256, 0, s>>>(master, grad, m, v, (__nv_bfloat16*)shadow_bf16, n, lr, beta1, beta2, eps, wd, bc1, bc2);
  return int(cudaGetLastError());
}
int arb_muon_nesterov(float* buf, const float* grad, void* u_bf16, float* sumsq, long long per_mat, int n_mat, float mu, cudaStream_t s) {
  if (per_mat <= 0 || n_mat <= 0 || n_mat > 65535) return -3;
  cudaError_t e = cudaMemsetAsync(sumsq, 0, sizeof(float) * n_mat, s);
  if (e != cudaSuccess) return int(e);
  const int bpm = blocks_for(per_mat, 256 * 4, 64);
  muon_nesterov_k<<<dim3(bpm, n_mat), 256, 0, s>>>(buf, grad, (__nv_bfloat16*)u_bf16, sumsq, per_mat, mu);
  return int(cudaGetLastError());
}
int arb_muon_frob_scale(void* u_bf16, const float* sumsq, long long per_mat, int n_mat, cudaStream_t s) {
  if (per_mat <= 0 || n_mat <= 0 || n_mat > 65535) return -3;
  muon_frob_scale_k<<<dim3(blocks_for(per_mat, 256 * 4, 64), n_mat), 256, 0, s>>>((__nv_bfloat16*)u_bf16, sumsq, per_mat);
  return int(cudaGetLastError());
}
int arb_normuon_stats(const void* x_bf16, float* v_mean, int n_mat, int m, int n, cudaStream_t s) {
  if (n_mat <= 0 || m <= 0 || n <= 0 || n_mat > 65535) return -3;
  if (m >= n) normuon_stats_k<true><<<dim3((m + 7) / 8, n_mat), 256, 0, s>>>((const __nv_bfloat16*)x_bf16, v_mean, m, n);
  else normuon_stats_k<false><<<dim3((n + 255) / 256, n_mat), 256, 0, s>>>((const __nv_bfloat16*)x_bf16, v_mean, m, n);
  return int(cudaGetLastError());
}
int arb_normuon_scales(const float* v_mean, float* second, float* scale, int n_mat, int n_stat, int red_size, float beta2, cudaStream_t s) {
  if (n_mat <= 0 || n_stat <= 0) return -3;
  normuon_scales_k<<<n_mat, 256, 0, s>>>(v_mean, second, scale, n_stat, red_size, beta2);
  return int(cudaGetLastError());
}
int arb_muon_update(float* master, void* shadow_bf16, const void* x_bf16, const float* scale, int n_mat, int m, int n, float lr,
                    float wd, cudaStream_t s) {
  if (n_mat <= 0 || m <= 0 || n <= 0 || n_mat > 65535) return -3;
  const int bpm = blocks_for((long long)m * n, 256 * 4, 64);
  if (m >= n) muon_update_k<true><<<dim3(bpm, n_mat), 256, 0, s>>>(master, (__nv_bfloat16*)shadow_bf16, (const __nv_bfloat16*)x_bf16, scale, m, n, lr, wd);
  else muon_update_k<false><<<dim3(bpm, n_mat), 256, 0, s>>>(master, (__nv_bfloat16*)shadow_bf16, (const __nv_bfloat16*)x_bf16, scale, m, n, lr, wd);
  return int(cudaGetLastError());
}

}  // extern "C"
