// Row-wise fused kernels: parameter-free RMSNorm, the residual-scale / residual-add norm
// fusions, RoPE + QK-norm + value-embedding application on the packed qkv buffer, ReLU^2,
// embedding gather / scatter-add, small casts.
//
// Math: brain/kernels/rms_norm.cu:20-90, fused_norm_residual.cu:22-350, rope.cu:10-107,
// ve_apply.cu:10-99, embedding.cu:8-80, relu_sq.cu:8-75.  Layout choices are new: one warp
// per row with the row cached in registers as 16-byte vectors (one global read per
// element), q/k/v processed in place inside the packed [N, 3D] GEMM output, and the
// QK-norm backward works from the saved inverse RMS instead of recomputing q and k.
#include "api.h"
#include "ptx.cuh"

namespace arb {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

constexpr int ROWS_PER_CTA = 8;  // 8 warps, one row each

// ---------------------------------------------------------------------------------------------
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_fwd_k(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                                     long long rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nch = D >> 3;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nch) {
      ld8(x + row * D + c * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[i][j] * v[i][j];
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / D + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nch) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] *= r;
      st8(y + row * D + c * 8, v[i]);
    }
  }
}

// gx = (add_to ? add_to : 0) + r*(g - x*(g.x)/D*r^2)
template <int NV>
__global__ void __launch_bounds__(256) rmsnorm_bwd_k(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ g,
                                                     const __nv_bfloat16* __restrict__ add_to, __nv_bfloat16* __restrict__ gx,
                                                     long long rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nch = D >> 3;
  float xv[NV][8], gv[NV][8];
  float ss = 0.f, dot = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nch) {
      ld8(x + row * D + c * 8, xv[i]);
      ld8(g + row * D + c * 8, gv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) { ss += xv[i][j] * xv[i][j]; dot += xv[i][j] * gv[i][j]; }
    }
  }
  ss = warp_sum(ss);
  dot = warp_sum(dot);
  const float r = rsqrtf(ss / D + eps);
  const float coef = dot / D * r * r;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nch) {
      float o[8];
      if (add_to) ld8(add_to + row * D + c * 8, o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float t = r * (gv[i][j] - xv[i][j] * coef);
        o[j] = add_to ? o[j] + t : t;
      }
      st8(gx + row * D + c * 8, o);
    }
  }
}

// x' = lr*x + l0*x0 (stored bf16) ; xn = rmsnorm(x')
template <int NV, bool SCALE>
__global__ void __launch_bounds__(256) resid_norm_fwd_k(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x0,
                                                        const __nv_bfloat16* __restrict__ lam_r, const __nv_bfloat16* __restrict__ lam_0,
                                                        int idx, __nv_bfloat16* __restrict__ xo, __nv_bfloat16* __restrict__ xn,
                                                        long long rows, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nch = D >> 3;
  const float lr = SCALE ? __bfloat162float(lam_r[idx]) : 1.f;
  const float l0 = SCALE ? __bfloat162float(lam_0[idx]) : 1.f;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nch) {
      float b[8];
      ld8(x + row * D + c * 8, v[i]);
      ld8(x0 + row * D + c * 8, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        v[i][j] = bf16_round(lr * v[i][j] + l0 * b[j]);
        ss += v[i][j] * v[i][j];
      }
      st8(xo + row * D + c * 8, v[i]);
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / D + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < nch) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] *= r;
      st8(xn + row * D + c * 8, v[i]);
    }
  }
}

template <int NV>
__global__ void __launch_bounds__(256) resid_norm_bwd_k(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x0,
                                                        const __nv_bfloat16* __restrict__ lam_r, const __nv_bfloat16* __restrict__ lam_0,
                                                        int idx, const __nv_bfloat16* __restrict__ g_xs, const __nv_bfloat16* __restrict__ g_xn,
                                                        __nv_bfloat16* __restrict__ d_x, __nv_bfloat16* d_x0,
                                                        const __nv_bfloat16* d_x0_acc,
                                                        float* __restrict__ dlam_r, float* __restrict__ dlam_0,
                                                        long long rows, int D, float eps) {
  // d_x0_acc (may equal d_x0): the x0 gradient of the layers above, added here instead of by a separate pass
  __shared__ float red[2][ROWS_PER_CTA];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long row = (long long)blockIdx.x * ROWS_PER_CTA + warp;
  const int nch = D >> 3;
  const float lr = __bfloat162float(lam_r[idx]);
  const float l0 = __bfloat162float(lam_0[idx]);
  float sr = 0.f, s0 = 0.f;
  if (row < rows) {
    // the row is kept as packed bf16 (4 registers per 8 values) between the two passes: with fp32 copies of
    // three arrays the kernel needed 127 registers and ran at a quarter of the possible occupancy
    uint4 xq[NV], bq[NV], gq[NV];
    float ss = 0.f, dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nch) {
        xq[i] = *reinterpret_cast<const uint4*>(x + row * D + c * 8);
        bq[i] = *reinterpret_cast<const uint4*>(x0 + row * D + c * 8);
        gq[i] = *reinterpret_cast<const uint4*>(g_xn + row * D + c * 8);
        float xv[8], bv[8], gv[8];
        unpack8(xq[i], xv); unpack8(bq[i], bv); unpack8(gq[i], gv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xs = bf16_round(lr * xv[j] + l0 * bv[j]);
          ss += xs * xs;
          dot += xs * gv[j];
        }
      }
    }
    ss = warp_sum(ss);
    dot = warp_sum(dot);
    const float r = rsqrtf(ss / D + eps);
    const float coef = dot / D * r * r;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < nch) {
        float gs[8], o1[8], o2[8], xv[8], bv[8], gv[8], av[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        ld8(g_xs + row * D + c * 8, gs);
        if (d_x0_acc) ld8(d_x0_acc + row * D + c * 8, av);
        unpack8(xq[i], xv); unpack8(bq[i], bv); unpack8(gq[i], gv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xs = bf16_round(lr * xv[j] + l0 * bv[j]);
          const float t = gs[j] + r * (gv[j] - xs * coef);
          o1[j] = lr * t;
          o2[j] = l0 * t + av[j];
          sr += xv[j] * t;
          s0 += bv[j] * t;
        }
        st8(d_x + row * D + c * 8, o1);
        st8(d_x0 + row * D + c * 8, o2);
      }
    }
  }
  sr = warp_sum(sr);
  s0 = warp_sum(s0);
  if (lane == 0) { red[0][warp] = sr; red[1][warp] = s0; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int w = 0; w < ROWS_PER_CTA; ++w) { a += red[0][w]; b += red[1][w]; }
    atomicAdd(dlam_r + idx, a);
    atomicAdd(dlam_0 + idx, b);
  }
}

// ---------------------------------------------------------------------------------------------
__global__ void residual_add_k(const uint4* __restrict__ a, const uint4* __restrict__ b, uint4* __restrict__ o, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    ld8(reinterpret_cast<const __nv_bfloat16*>(a + i), x);
    ld8(reinterpret_cast<const __nv_bfloat16*>(b + i), y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    st8(reinterpret_cast<__nv_bfloat16*>(o + i), x);
  }
}
__global__ void relu_sq_fwd_k(const uint4* __restrict__ a, uint4* __restrict__ o, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float x[8];
    ld8(reinterpret_cast<const __nv_bfloat16*>(a + i), x);
#pragma unroll
    for (int j = 0; j < 8; ++j) { const float r = fmaxf(x[j], 0.f); x[j] = r * r; }
    st8(reinterpret_cast<__nv_bfloat16*>(o + i), x);
  }
}
__global__ void relu_sq_bwd_k(const uint4* __restrict__ a, const uint4* __restrict__ g, uint4* __restrict__ o, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    ld8(reinterpret_cast<const __nv_bfloat16*>(a + i), x);
    ld8(reinterpret_cast<const __nv_bfloat16*>(g + i), y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = 2.f * fmaxf(x[j], 0.f) * y[j];
    st8(reinterpret_cast<__nv_bfloat16*>(o + i), x);
  }
}
__global__ void cast_f32_bf16_k(const float4* __restrict__ s, uint2* __restrict__ d, long long n4, float scale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = s[i];
    d[i] = make_uint2(pack_bf16(v.x * scale, v.y * scale), pack_bf16(v.z * scale, v.w * scale));
  }
}
__global__ void accum_bf16_f32_k(const uint2* __restrict__ s, float4* __restrict__ d, long long n4) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    uint2 u = s[i];
    float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
    float4 v = d[i];
    v.x += a.x; v.y += a.y; v.z += b.x; v.w += b.y;
    d[i] = v;
  }
}
// dst[r, 0:cols] += src[r, 0:cols]  (dst row stride ld_dst, src dense)
__global__ void add_cols_k(__nv_bfloat16* dst, long long ld_dst, const __nv_bfloat16* src, long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols;
    const int c = int(i - r * cols);
    __nv_bfloat16* p = dst + r * ld_dst + c;
    *p = __float2bfloat16(__bfloat162float(*p) + __bfloat162float(src[i]));
  }
}

// ---------------------------------------------------------------------------------------------
// embedding
__global__ void embedding_fwd_k(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                long long N, int D, int vocab) {
  const int nch = D >> 3;
  const long long total = N * nch;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / nch;
    const int c = int(i - t * nch);
    int id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(w + (long long)id * D + c * 8);
  }
}
__global__ void embedding_bwd_k(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ g, float* __restrict__ dw,
                                long long N, int D, int vocab) {
  const int nch = D >> 3;
  const long long total = N * nch;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / nch;
    const int c = int(i - t * nch);
    int id = ids[t];
    if (id < 0 || id >= vocab) continue;
    float f[8];
    ld8(g + i * 8, f);
    float* dst = dw + (long long)id * D + c * 8;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(f[0]), "f"(f[1]), "f"(f[2]), "f"(f[3]) : "memory");
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + 4), "f"(f[4]), "f"(f[5]), "f"(f[6]), "f"(f[7]) : "memory");
  }
}

// Deterministic embedding backward: rows sorted by token id (stable), one work item per (id, chunk of at most
// `R` rows).  An item sums its rows in sorted order in fp32; an id with a single item adds the sum to its table
// row (it is the only writer), longer ids leave per-item partial sums that embedding_bwd_combine_k adds up in
// item order.  No atomics: the result does not depend on scheduling (the reference's histogram kernel,
// brain/kernels/embedding.cu, and the kernel above both rely on the order of atomic adds).
__global__ void __launch_bounds__(128) embedding_bwd_sorted_k(const long long* __restrict__ perm, const int* __restrict__ item_id,
                                                              const int* __restrict__ item_start, const int* __restrict__ seg_start,
                                                              const int* __restrict__ seg_count, const __nv_bfloat16* __restrict__ g,
                                                              float* __restrict__ dw, float* __restrict__ partial, int n_items_max,
                                                              int D, int R, int vocab) {
  const int item = blockIdx.x;
  const int id = item_id[item];
  if (id < 0 || id >= vocab) return;                 // padding items beyond the real count
  const int cnt = seg_count[id];
  const int sub = item - item_start[id];
  const int r0 = sub * R, r1 = min(cnt, r0 + R);
  if (r0 >= r1) return;
  const long long base = seg_start[id];
  for (int c = threadIdx.x; c < (D >> 3); c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = r0; j < r1; ++j) {
      float f[8];
      ld8(g + perm[base + j] * D + c * 8, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += f[k];
    }
    float* dst = (cnt <= R) ? dw + (long long)id * D + c * 8 : partial + (long long)item * D + c * 8;
    float4 a = make_float4(acc[0], acc[1], acc[2], acc[3]), b = make_float4(acc[4], acc[5], acc[6], acc[7]);
    if (cnt <= R) {
      const float4 x = *reinterpret_cast<float4*>(dst), y = *reinterpret_cast<float4*>(dst + 4);
      a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w; b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
    }
    *reinterpret_cast<float4*>(dst) = a;
    *reinterpret_cast<float4*>(dst + 4) = b;
  }
}
__global__ void __launch_bounds__(128) embedding_bwd_combine_k(const int* __restrict__ item_start, const int* __restrict__ seg_count,
                                                               const float* __restrict__ partial, float* __restrict__ dw, int D, int R) {
  const int id = blockIdx.x;
  const int cnt = seg_count[id];
  if (cnt <= R) return;
  const int n_it = (cnt + R - 1) / R, i0 = item_start[id];
  for (int c = threadIdx.x; c < (D >> 2); c += blockDim.x) {
    float4 acc = *reinterpret_cast<float4*>(dw + (long long)id * D + c * 4);
    for (int i = 0; i < n_it; ++i) {
      const float4 p = *reinterpret_cast<const float4*>(partial + (long long)(i0 + i) * D + c * 4);
      acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    *reinterpret_cast<float4*>(dw + (long long)id * D + c * 4) = acc;
  }
}

// ---------------------------------------------------------------------------------------------
// qkv post-processing, head_dim = 128.  One warp handles one (token, head) slot of q, k or v:
// lane l owns elements [4l, 4l+4) of the head row; the rotate-half partner (element i+64) lives
// in lane l^16.
__device__ __forceinline__ void ld4(const __nv_bfloat16* p, float (&f)[4]) {
  uint2 u = *reinterpret_cast<const uint2*>(p);
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void st4(__nv_bfloat16* p, const float (&f)[4]) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]));
}

// One warp per token: the cos/sin row of the token is loaded once and reused by all 2H q/k heads, the
// token-index arithmetic is done once, and two heads are in flight per iteration.  (One warp per
// (token, head) made these kernels instruction-bound: 2-3 million warps, each with two 64-bit divisions.)
__global__ void __launch_bounds__(256) qkv_post_fwd_k(__nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ cos_t,
                                                      const __nv_bfloat16* __restrict__ sin_t, float* __restrict__ rstd_qk,
                                                      const __nv_bfloat16* __restrict__ xn, const int* __restrict__ ids,
                                                      const __nv_bfloat16* __restrict__ ve_w, const __nv_bfloat16* __restrict__ gate_w,
                                                      float* __restrict__ gate_out, long long N, int T, int H, int D_model,
                                                      int gate_ch, float eps) {
  const int lane = threadIdx.x & 31;
  const long long tok = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= N) return;
  const int Dl = H * 128;
  __nv_bfloat16* base = qkv + tok * 3 * Dl + lane * 4;
  const int t = int(tok % T);
  const int hi = lane >> 4;                 // 0: low half of the head, 1: high half
  const int pos = (lane & 15) * 4;          // index inside the half
  float c[4], sn[4];
  ld4(cos_t + (long long)t * 64 + pos, c);
  ld4(sin_t + (long long)t * 64 + pos, sn);
  if (hi) {
#pragma unroll
    for (int j = 0; j < 4; ++j) sn[j] = -sn[j];   // lo' = lo*c + hi*s ; hi' = hi*c - lo*s
  }
  for (int slot = 0; slot < 2 * H; slot += 2) {
    float v0[4], v1[4], o0[4], o1[4];
    ld4(base + slot * 128, v0);
    ld4(base + (slot + 1) * 128, v1);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float p0 = __shfl_xor_sync(0xffffffffu, v0[j], 16), p1 = __shfl_xor_sync(0xffffffffu, v1[j], 16);
      o0[j] = v0[j] * c[j] + p0 * sn[j];
      o1[j] = v1[j] * c[j] + p1 * sn[j];
      s0 += o0[j] * o0[j];
      s1 += o1[j] * o1[j];
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) { s0 += __shfl_xor_sync(0xffffffffu, s0, m); s1 += __shfl_xor_sync(0xffffffffu, s1, m); }
    const float r0 = rsqrtf(s0 / 128.f + eps), r1 = rsqrtf(s1 / 128.f + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) { o0[j] *= r0; o1[j] *= r1; }
    st4(base + slot * 128, o0);
    st4(base + (slot + 1) * 128, o1);
    if (lane == 0) *reinterpret_cast<float2*>(rstd_qk + tok * 2 * H + slot) = make_float2(r0, r1);
  }
  if (ve_w) {
    const int id = ids[tok];
    // gate logit of head h = xn[tok, :gate_ch] . Wg[h, :]; lane j holds xn[tok, j], xn[tok, j+32], ...
    for (int h = 0; h < H; ++h) {
      float part = 0.f;
      for (int j = lane; j < gate_ch; j += 32)
        part += __bfloat162float(xn[tok * D_model + j]) * __bfloat162float(gate_w[h * gate_ch + j]);
      const float gl = warp_sum(part);
      if (lane == 0) gate_out[tok * H + h] = gl;
      const float gs = 2.f / (1.f + __expf(-gl));
      float v[4], e[4];
      ld4(base + (2 * H + h) * 128, v);
      ld4(ve_w + (long long)id * Dl + h * 128 + lane * 4, e);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] += gs * e[j];
      st4(base + (2 * H + h) * 128, v);
    }
  }
}

__global__ void __launch_bounds__(256) qkv_post_bwd_k(__nv_bfloat16* __restrict__ dqkv, const __nv_bfloat16* __restrict__ qkv,
                                                      const __nv_bfloat16* __restrict__ cos_t, const __nv_bfloat16* __restrict__ sin_t,
                                                      const float* __restrict__ rstd_qk, const __nv_bfloat16* __restrict__ xn,
                                                      const int* __restrict__ ids, const __nv_bfloat16* __restrict__ ve_w,
                                                      const __nv_bfloat16* __restrict__ gate_w, const float* __restrict__ gate,
                                                      __nv_bfloat16* __restrict__ d_ve, float* __restrict__ d_gate_logit,
                                                      long long N, int T, int H) {
  const int lane = threadIdx.x & 31;
  const long long tok = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (tok >= N) return;
  const int Dl = H * 128;
  const long long off = tok * 3 * Dl + lane * 4;
  const int t = int(tok % T);
  const int hi = lane >> 4;
  const int pos = (lane & 15) * 4;
  float c[4], sn[4];
  ld4(cos_t + (long long)t * 64 + pos, c);
  ld4(sin_t + (long long)t * 64 + pos, sn);
  if (!hi) {
#pragma unroll
    for (int j = 0; j < 4; ++j) sn[j] = -sn[j];   // transpose of the rotation: d_lo = g_lo*c - g_hi*s ; d_hi = g_hi*c + g_lo*s
  }
  for (int slot = 0; slot < 2 * H; slot += 2) {
    float y0[4], y1[4], g0[4], g1[4];
    ld4(qkv + off + slot * 128, y0);
    ld4(qkv + off + (slot + 1) * 128, y1);
    ld4(dqkv + off + slot * 128, g0);
    ld4(dqkv + off + (slot + 1) * 128, g1);
    const float2 r = *reinterpret_cast<const float2*>(rstd_qk + tok * 2 * H + slot);
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) { d0 += y0[j] * g0[j]; d1 += y1[j] * g1[j]; }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) { d0 += __shfl_xor_sync(0xffffffffu, d0, m); d1 += __shfl_xor_sync(0xffffffffu, d1, m); }
    d0 *= (1.f / 128.f); d1 *= (1.f / 128.f);
    float o0[4], o1[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a0 = r.x * (g0[j] - y0[j] * d0), a1 = r.y * (g1[j] - y1[j] * d1);   // grad wrt the rotated value
      const float p0 = __shfl_xor_sync(0xffffffffu, a0, 16), p1 = __shfl_xor_sync(0xffffffffu, a1, 16);
      o0[j] = a0 * c[j] + p0 * sn[j];
      o1[j] = a1 * c[j] + p1 * sn[j];
    }
    st4(dqkv + off + slot * 128, o0);
    st4(dqkv + off + (slot + 1) * 128, o1);
  }
  if (ve_w) {
    const int id = ids[tok];
    for (int h = 0; h < H; ++h) {
      const float gl = gate[tok * H + h];
      const float sg = 1.f / (1.f + __expf(-gl));
      float g[4], e[4], o[4];
      ld4(dqkv + off + (2 * H + h) * 128, g);
      ld4(ve_w + (long long)id * Dl + h * 128 + lane * 4, e);
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) { o[j] = 2.f * sg * g[j]; dot += e[j] * g[j]; }
      st4(d_ve + tok * Dl + h * 128 + lane * 4, o);
      dot = warp_sum(dot);
      if (lane == 0) d_gate_logit[tok * H + h] = 2.f * sg * (1.f - sg) * dot;
    }
  }
}

// d_gate_w[h, j] += sum_t dgl[t, h] * xn[t, j] ; d_xn_gate[t, j] = sum_h dgl[t, h] * Wg[h, j]
// One CTA handles a slab of tokens; thread (h, j) accumulates its column.
__global__ void __launch_bounds__(256) ve_gate_bwd_k(const float* __restrict__ dgl, const __nv_bfloat16* __restrict__ xn,
                                                     const __nv_bfloat16* __restrict__ gate_w, float* __restrict__ d_gate_w,
                                                     __nv_bfloat16* __restrict__ d_xn_gate, long long N, int H, int D_model,
                                                     int ch, int tok_per_cta) {
  const long long t0 = (long long)blockIdx.x * tok_per_cta;
  const long long t1 = min(N, t0 + tok_per_cta);
  const int tid = threadIdx.x;
  for (int p = tid; p < H * ch; p += blockDim.x) {
    const int h = p / ch, j = p - h * ch;
    float acc = 0.f;
    for (long long t = t0; t < t1; ++t) acc += dgl[t * H + h] * __bfloat162float(xn[t * D_model + j]);
    atomicAdd(d_gate_w + h * ch + j, acc);
  }
  for (long long i = t0 * ch + tid; i < t1 * ch; i += blockDim.x) {
    const long long t = i / ch;
    const int j = int(i - t * ch);
    float acc = 0.f;
    for (int h = 0; h < H; ++h) acc += dgl[t * H + h] * __bfloat162float(gate_w[h * ch + j]);
    d_xn_gate[i] = __float2bfloat16(acc);
  }
}

static inline int grid_for(long long n, int threads, int cap = 148 * 16) {
  long long b = (n + threads - 1) / threads;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return int(b);
}

#define ROW_DISPATCH(KERNEL, ...)                                                        \
  do {                                                                                     \
    const int blocks = int((rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA);                      \
    if (D <= 256) KERNEL<1><<<blocks, 256, 0, s>>>(__VA_ARGS__);                           \
    else if (D <= 512) KERNEL<2><<<blocks, 256, 0, s>>>(__VA_ARGS__);                      \
    else if (D <= 1024) KERNEL<4><<<blocks, 256, 0, s>>>(__VA_ARGS__);                     \
    else if (D <= 2048) KERNEL<8><<<blocks, 256, 0, s>>>(__VA_ARGS__);                     \
    else KERNEL<16><<<blocks, 256, 0, s>>>(__VA_ARGS__);                                   \
  } while (0)

static inline int check_row_args(long long rows, int D) {
  if (rows <= 0 || D <= 0 || (D & 7) || D > 4096) return -3;
  return 0;
}
static inline bool misaligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) != 0; }

}  // namespace arb

using namespace arb;
typedef __nv_bfloat16 bf16;

extern "C" {

int arb_rmsnorm_fwd(const void* x, void* y, long long rows, int D, float eps, cudaStream_t s) {
  if (check_row_args(rows, D) || misaligned(x) || misaligned(y)) return -3;
  ROW_DISPATCH(rmsnorm_fwd_k, (const bf16*)x, (bf16*)y, rows, D, eps);
  return int(cudaGetLastError());
}
int arb_rmsnorm_bwd(const void* x, const void* g, const void* add_to, void* gx, long long rows, int D, float eps, cudaStream_t s) {
  if (check_row_args(rows, D) || misaligned(x) || misaligned(g) || misaligned(gx) || misaligned(add_to)) return -3;
  ROW_DISPATCH(rmsnorm_bwd_k, (const bf16*)x, (const bf16*)g, (const bf16*)add_to, (bf16*)gx, rows, D, eps);
  return int(cudaGetLastError());
}
int arb_resid_scale_norm_fwd(const void* x, const void* x0, const void* lam_r, const void* lam_0, int idx, void* x_out,
                             void* xn_out, long long rows, int D, float eps, cudaStream_t s) {
  if (check_row_args(rows, D) || misaligned(x) || misaligned(x0) || misaligned(x_out) || misaligned(xn_out)) return -3;
#define RSN(NV) resid_norm_fwd_k<NV, true>
  const int blocks = int((rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA);
  if (D <= 256) RSN(1)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)x0, (const bf16*)lam_r, (const bf16*)lam_0, idx, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
  else if (D <= 512) RSN(2)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)x0, (const bf16*)lam_r, (const bf16*)lam_0, idx, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
  else if (D <= 1024) RSN(4)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)x0, (const bf16*)lam_r, (const bf16*)lam_0, idx, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
  else if (D <= 2048) RSN(8)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)x0, (const bf16*)lam_r, (const bf16*)lam_0, idx, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
  else RSN(16)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)x0, (const bf16*)lam_r, (const bf16*)lam_0, idx, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
#undef RSN
  return int(cudaGetLastError());
}
int arb_add_norm_fwd(const void* x, const void* proj, void* x_out, void* xn_out, long long rows, int D, float eps, cudaStream_t s) {
  if (check_row_args(rows, D) || misaligned(x) || misaligned(proj) || misaligned(x_out) || misaligned(xn_out)) return -3;
#define RSN(NV) resid_norm_fwd_k<NV, false>
  const int blocks = int((rows + ROWS_PER_CTA - 1) / ROWS_PER_CTA);
  if (D <= 256) RSN(1)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)proj, nullptr, nullptr, 0, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
  else if (D <= 512) RSN(2)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)proj, nullptr, nullptr, 0, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
  else if (D <= 1024) RSN(4)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)proj, nullptr, nullptr, 0, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
  else if (D <= 2048) RSN(8)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)proj, nullptr, nullptr, 0, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
  else RSN(16)<<<blocks, 256, 0, s>>>((const bf16*)x, (const bf16*)proj, nullptr, nullptr, 0, (bf16*)x_out, (bf16*)xn_out, rows, D, eps);
#undef RSN
  return int(cudaGetLastError());
}
int arb_resid_scale_norm_bwd(const void* x, const void* x0, const void* lam_r, const void* lam_0, int idx, const void* g_xs,
                             const void* g_xn, void* d_x, void* d_x0, const void* d_x0_acc, float* dlam_r, float* dlam_0,
                             long long rows, int D, float eps, cudaStream_t s) {
  if (check_row_args(rows, D) || misaligned(x) || misaligned(x0) || misaligned(g_xs) || misaligned(g_xn) || misaligned(d_x) ||
      misaligned(d_x0) || (d_x0_acc && misaligned(d_x0_acc)))
    return -3;
  ROW_DISPATCH(resid_norm_bwd_k, (const bf16*)x, (const bf16*)x0, (const bf16*)lam_r, (const bf16*)lam_0, idx, (const bf16*)g_xs,
               (const bf16*)g_xn, (bf16*)d_x, (bf16*)d_x0, (const bf16*)d_x0_acc, dlam_r, dlam_0, rows, D, eps);
  return int(cudaGetLastError());
}
int arb_residual_add(const void* a, const void* b, void* out, long long n, cudaStream_t s) {
  if (n <= 0 || (n & 7) || misaligned(a) || misaligned(b) || misaligned(out)) return -3;
  residual_add_k<<<grid_for(n / 8, 256), 256, 0, s>>>((const uint4*)a, (const uint4*)b, (uint4*)out, n / 8);
  return int(cudaGetLastError());
}
int arb_relu_sq_fwd(const void* x, void* y, long long n, cudaStream_t s) {
  if (n <= 0 || (n & 7) || misaligned(x) || misaligned(y)) return -3;
  relu_sq_fwd_k<<<grid_for(n / 8, 256), 256, 0, s>>>((const uint4*)x, (uint4*)y, n / 8);
  return int(cudaGetLastError());
}
int arb_relu_sq_bwd(const void* x, const void* g, void* gx, long long n, cudaStream_t s) {
  if (n <= 0 || (n & 7) || misaligned(x) || misaligned(g) || misaligned(gx)) return -3;
  relu_sq_bwd_k<<<grid_for(n / 8, 256), 256, 0, s>>>((const uint4*)x, (const uint4*)g, (uint4*)gx, n / 8);
  return int(cudaGetLastError());
}
int arb_qkv_post_fwd(void* qkv, const void* cos_t, const void* sin_t, float* rstd_qk, const void* xn, const int* ids,
                     const void* ve_w, const void* gate_w, float* gate_out, long long N, int T, int H, int D_model,
                     int gate_ch, float eps, cudaStream_t s) {
  if (N <= 0 || T <= 0 || H <= 0 || misaligned(qkv) || (reinterpret_cast<uintptr_t>(cos_t) & 7) || (reinterpret_cast<uintptr_t>(sin_t) & 7)) return -3;
  if (ve_w && (!gate_w || !gate_out || !xn || !ids || misaligned(ve_w))) return -3;
  qkv_post_fwd_k<<<int((N + 7) / 8), 256, 0, s>>>((bf16*)qkv, (const bf16*)cos_t, (const bf16*)sin_t, rstd_qk, (const bf16*)xn, ids,
                                                      (const bf16*)ve_w, (const bf16*)gate_w, gate_out, N, T, H, D_model, gate_ch, eps);
  return int(cudaGetLastError());
}
int arb_qkv_post_bwd(void* d_qkv, const void* qkv, const void* cos_t, const void* sin_t, const float* rstd_qk, const void* xn,
                     const int* ids, const void* ve_w, const void* gate_w, const float* gate, void* d_ve, float* d_gate_w,
                     void* d_xn_gate, float* dgl, long long N, int T, int H, int D_model, int gate_ch, cudaStream_t s) {
  if (N <= 0 || T <= 0 || H <= 0 || misaligned(d_qkv) || misaligned(qkv)) return -3;
  if (ve_w && (!gate_w || !gate || !xn || !ids || !d_ve || !d_gate_w || !d_xn_gate || !dgl)) return -3;
  qkv_post_bwd_k<<<int((N + 7) / 8), 256, 0, s>>>((bf16*)d_qkv, (const bf16*)qkv, (const bf16*)cos_t, (const bf16*)sin_t, rstd_qk,
                                                      (const bf16*)xn, ids, (const bf16*)ve_w, (const bf16*)gate_w, gate, (bf16*)d_ve,
                                                      dgl, N, T, H);
  int rc = int(cudaGetLastError());
  if (ve_w) {
    const int tpc = 512;
    ve_gate_bwd_k<<<int((N + tpc - 1) / tpc), 256, 0, s>>>(dgl, (const bf16*)xn, (const bf16*)gate_w, d_gate_w, (bf16*)d_xn_gate, N, H,
                                                            D_model, gate_ch, tpc);
    if (!rc) rc = int(cudaGetLastError());
  }
  return rc;
}
int arb_embedding_fwd(const int* ids, const void* w, void* out, long long N, int D, int vocab, cudaStream_t s) {
  if (N <= 0 || (D & 7) || misaligned(w) || misaligned(out)) return -3;
  embedding_fwd_k<<<grid_for(N * (D / 8), 256), 256, 0, s>>>(ids, (const bf16*)w, (bf16*)out, N, D, vocab);
  return int(cudaGetLastError());
}
int arb_embedding_bwd(const int* ids, const void* g, float* dw, long long N, int D, int vocab, cudaStream_t s) {
  if (N <= 0 || (D & 7) || misaligned(g) || misaligned(dw)) return -3;
  embedding_bwd_k<<<grid_for(N * (D / 8), 256), 256, 0, s>>>(ids, (const bf16*)g, dw, N, D, vocab);
  return int(cudaGetLastError());
}
// Deterministic variant: perm[N] = row indices sorted by token id (stable); seg_start / seg_count [vocab] = first
// sorted position and number of rows of every id; item_start[vocab] = first work item of every id (exclusive
// prefix sum of ceil(count / R)); item_id[n_items_max] = id of every item, -1 for unused ones; partial =
// n_items_max * D floats of scratch.
int arb_embedding_bwd_sorted(const long long* perm, const int* item_id, const int* item_start, const int* seg_start,
                             const int* seg_count, const void* g, float* dw, float* partial, int n_items_max, int D, int R,
                             int vocab, cudaStream_t s) {
  if (n_items_max <= 0 || (D & 7) || R <= 0 || vocab <= 0 || misaligned(g) || misaligned(dw) || misaligned(partial)) return -3;
  embedding_bwd_sorted_k<<<n_items_max, 128, 0, s>>>(perm, item_id, item_start, seg_start, seg_count, (const bf16*)g, dw, partial,
                                                     n_items_max, D, R, vocab);
  int rc = int(cudaGetLastError());
  if (rc) return rc;
  embedding_bwd_combine_k<<<vocab, 128, 0, s>>>(item_start, seg_count, partial, dw, D, R);
  return int(cudaGetLastError());
}
int arb_add_cols(void* dst, long long ld_dst, const void* src, long long rows, int cols, cudaStream_t s) {
  if (rows <= 0 || cols <= 0) return -3;
  add_cols_k<<<grid_for(rows * cols, 256), 256, 0, s>>>((bf16*)dst, ld_dst, (const bf16*)src, rows, cols);
  return int(cudaGetLastError());
}
int arb_cast_f32_to_bf16(const float* src, void* dst, long long n, float scale, cudaStream_t s) {
  if (n <= 0 || (n & 3) || misaligned(src) || (reinterpret_cast<uintptr_t>(dst) & 7)) return -3;
  cast_f32_bf16_k<<<grid_for(n / 4, 256), 256, 0, s>>>((const float4*)src, (uint2*)dst, n / 4, scale);
  return int(cudaGetLastError());
}
int arb_accum_bf16_into_f32(const void* src, float* dst, long long n, cudaStream_t s) {
  if (n <= 0 || (n & 3) || misaligned(dst) || (reinterpret_cast<uintptr_t>(src) & 7)) return -3;
  accum_bf16_f32_k<<<grid_for(n / 4, 256), 256, 0, s>>>((const uint2*)src, (float4*)dst, n / 4);
  return int(cudaGetLastError());
}

}  // extern "C"
