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

// Frobenius norms without atomics: every block of a matrix leaves ONE partial sum in its own slot of
// partials[mat][MUON_PARTS] (unused slots are zeroed by block 0), and the scale kernel adds the slots in a fixed
// order, so the norm - and with it the whole Muon update - is the same bit pattern run after run.
constexpr int MUON_PARTS = 64;

__device__ __forceinline__ void muon_store_partial(float acc, float* __restrict__ partials, int mat) {
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    partials[mat * MUON_PARTS + blockIdx.x] = t;
  }
  if (blockIdx.x == 0 && threadIdx.x >= gridDim.x && threadIdx.x < MUON_PARTS) partials[mat * MUON_PARTS + threadIdx.x] = 0.f;
}

// One step for 8 consecutive elements: b = mu*b + (1-mu)*g ; u = bf16((1-mu)*g + mu*b); returns sum u^2
__device__ __forceinline__ float nesterov8(float* __restrict__ buf, __nv_bfloat16* __restrict__ u, long long at, const float (&g)[8],
                                           float mu) {
  float4 b0 = *reinterpret_cast<const float4*>(buf + at), b1 = *reinterpret_cast<const float4*>(buf + at + 4);
  float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
  float uu[8], acc = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    b[j] = mu * b[j] + (1.f - mu) * g[j];
    uu[j] = __bfloat162float(__float2bfloat16((1.f - mu) * g[j] + mu * b[j]));
    acc += uu[j] * uu[j];
  }
  *reinterpret_cast<float4*>(buf + at) = make_float4(b[0], b[1], b[2], b[3]);
  *reinterpret_cast<float4*>(buf + at + 4) = make_float4(b[4], b[5], b[6], b[7]);
  uint4 o;
  o.x = pack_bf16(uu[0], uu[1]); o.y = pack_bf16(uu[2], uu[3]); o.z = pack_bf16(uu[4], uu[5]); o.w = pack_bf16(uu[6], uu[7]);
  *reinterpret_cast<uint4*>(u + at) = o;
  return acc;
}

// grid: (blocks_per_mat <= MUON_PARTS, n_mat).  VEC: per_mat is a multiple of 8 and every pointer 16-byte aligned.
template <bool VEC>
__global__ void __launch_bounds__(256) muon_nesterov_k(float* __restrict__ buf, const float* __restrict__ g,
                                                       __nv_bfloat16* __restrict__ u, float* __restrict__ partials,
                                                       long long per_mat, float mu) {
  const int mat = blockIdx.y;
  const long long base = (long long)mat * per_mat;
  float acc = 0.f;
  if (VEC) {
    const long long stride = (long long)gridDim.x * blockDim.x * 8;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < per_mat; i += stride) {
      const float4 g0 = *reinterpret_cast<const float4*>(g + base + i), g1 = *reinterpret_cast<const float4*>(g + base + i + 4);
      const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      acc += nesterov8(buf, u, base + i, gg, mu);
    }
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_mat; i += (long long)gridDim.x * blockDim.x) {
      const float gi = g[base + i];
      const float b = mu * buf[base + i] + (1.f - mu) * gi;
      buf[base + i] = b;
      const __nv_bfloat16 ub = __float2bfloat16((1.f - mu) * gi + mu * b);
      u[base + i] = ub;
      const float uf = __bfloat162float(ub);
      acc += uf * uf;
    }
  }
  muon_store_partial(acc, partials, mat);
}

template <bool VEC>
__global__ void __launch_bounds__(256) muon_frob_scale_k(__nv_bfloat16* __restrict__ u, const float* __restrict__ partials,
                                                         long long per_mat) {
  __shared__ float s_inv;
  const int mat = blockIdx.y;
  if (threadIdx.x < 32) {      // fixed-order sum of the 64 slots
    float t = partials[mat * MUON_PARTS + threadIdx.x] + partials[mat * MUON_PARTS + 32 + threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) s_inv = 1.f / (sqrtf(t) * 1.02f + 1e-6f);
  }
  __syncthreads();
  const float inv = s_inv;
  const long long base = (long long)mat * per_mat;
  if (VEC) {
    const long long stride = (long long)gridDim.x * blockDim.x * 8;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < per_mat; i += stride) {
      uint4 v = *reinterpret_cast<const uint4*>(u + base + i);
      const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), d = unpack_bf16(v.w);
      v.x = pack_bf16(a.x * inv, a.y * inv); v.y = pack_bf16(b.x * inv, b.y * inv);
      v.z = pack_bf16(c.x * inv, c.y * inv); v.w = pack_bf16(d.x * inv, d.y * inv);
      *reinterpret_cast<uint4*>(u + base + i) = v;
    }
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_mat; i += (long long)gridDim.x * blockDim.x)
      u[base + i] = __float2bfloat16(__bfloat162float(u[base + i]) * inv);
  }
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

// g = x*scale[row or col]; mask = (g*p >= 0); p -= lr*g + lr*wd*p*mask.  VEC: n is a multiple of 8 (a chunk of 8
// elements never crosses a row) and every pointer is 16-byte aligned; one division per chunk instead of per element.
template <bool ROWS, bool VEC>
__global__ void muon_update_k(float* __restrict__ master, __nv_bfloat16* __restrict__ shadow, const __nv_bfloat16* __restrict__ x,
                              const float* __restrict__ scale, int m, int n, float lr, float wd) {
  const int mat = blockIdx.y;
  const long long per = (long long)m * n;
  const int n_stat = ROWS ? m : n;
  const float* sc = scale + (long long)mat * n_stat;
  if (VEC) {
    const long long stride = (long long)gridDim.x * blockDim.x * 8;
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8; i < per; i += stride) {
      const int r = int(i / n), c = int(i - (long long)r * n);
      float s8[8];
      if (ROWS) {
        const float sr = sc[r];
#pragma unroll
        for (int j = 0; j < 8; ++j) s8[j] = sr;
      } else {
        const float4 s0 = *reinterpret_cast<const float4*>(sc + c), s1 = *reinterpret_cast<const float4*>(sc + c + 4);
        s8[0] = s0.x; s8[1] = s0.y; s8[2] = s0.z; s8[3] = s0.w; s8[4] = s1.x; s8[5] = s1.y; s8[6] = s1.z; s8[7] = s1.w;
      }
      const long long at = mat * per + i;
      const uint4 xv = *reinterpret_cast<const uint4*>(x + at);
      const float2 xa = unpack_bf16(xv.x), xb = unpack_bf16(xv.y), xc = unpack_bf16(xv.z), xd = unpack_bf16(xv.w);
      const float xs[8] = {xa.x, xa.y, xb.x, xb.y, xc.x, xc.y, xd.x, xd.y};
      const float4 p0 = *reinterpret_cast<const float4*>(master + at), p1 = *reinterpret_cast<const float4*>(master + at + 4);
      float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float g = xs[j] * s8[j];
        const float mask = (g * p[j] >= 0.f) ? 1.f : 0.f;
        p[j] -= lr * g + lr * wd * p[j] * mask;
      }
      *reinterpret_cast<float4*>(master + at) = make_float4(p[0], p[1], p[2], p[3]);
      *reinterpret_cast<float4*>(master + at + 4) = make_float4(p[4], p[5], p[6], p[7]);
      uint4 o;
      o.x = pack_bf16(p[0], p[1]); o.y = pack_bf16(p[2], p[3]); o.z = pack_bf16(p[4], p[5]); o.w = pack_bf16(p[6], p[7]);
      *reinterpret_cast<uint4*>(shadow + at) = o;
    }
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
      const int r = int(i / n), c = int(i - (long long)r * n);
      const float g = __bfloat162float(x[mat * per + i]) * sc[ROWS ? r : c];
      float p = master[mat * per + i];
      const float mask = (g * p >= 0.f) ? 1.f : 0.f;
      p -= lr * g + lr * wd * p * mask;
      master[mat * per + i] = p;
      shadow[mat * per + i] = __float2bfloat16(p);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Reduce-scatter fused into the optimizer: the gradient of an owned element is summed on the fly
// over every rank's bf16 bucket (NVLink peer loads, or one multimem.ld_reduce through the
// switch), scaled, and consumed by the momentum / Adam update in the same thread - the reduced
// fp32 gradient is never written to memory.
// ---------------------------------------------------------------------------------------------
constexpr int OPT_MAX_WORLD = 16;
struct GradPeers { const __nv_bfloat16* p[OPT_MAX_WORLD]; const __nv_bfloat16* mc; int world; int rank; float scale; };

__device__ __forceinline__ void load_grad8(const GradPeers& g, long long idx, float (&o)[8]) {
  if (g.mc) {
    uint32_t r0, r1, r2, r3;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "l"(g.mc + idx) : "memory");
    float2 a = unpack_bf16(r0), b = unpack_bf16(r1), c = unpack_bf16(r2), d = unpack_bf16(r3);
    o[0] = a.x; o[1] = a.y; o[2] = b.x; o[3] = b.y; o[4] = c.x; o[5] = c.y; o[6] = d.x; o[7] = d.y;
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = 0.f;
    for (int q = 0; q < g.world; ++q) {
      const int pr = (g.rank + q) % g.world;
      const uint4 u = *reinterpret_cast<const uint4*>(g.p[pr] + idx);
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      o[0] += a.x; o[1] += a.y; o[2] += b.x; o[3] += b.y; o[4] += c.x; o[5] += c.y; o[6] += d.x; o[7] += d.y;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j] *= g.scale;
}

// Two chunks at once: their peer (or multimem) loads are issued back to back, so that a thread has several NVLink
// loads in flight.  With one chunk per iteration the fused kernels reached 160 GB/s on two GPUs, where every
// thread has a single peer to read from.
__device__ __forceinline__ void load_grad8x2(const GradPeers& g, long long i0, long long i1, float (&o0)[8], float (&o1)[8]) {
  if (g.mc) {
    uint32_t r[8];
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "l"(g.mc + i0));
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "l"(g.mc + i1));
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 a = unpack_bf16(r[k]), b = unpack_bf16(r[4 + k]);
      o0[2 * k] = a.x; o0[2 * k + 1] = a.y; o1[2 * k] = b.x; o1[2 * k + 1] = b.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) { o0[j] = 0.f; o1[j] = 0.f; }
#pragma unroll 2
    for (int q = 0; q < g.world; ++q) {
      const int pr = (g.rank + q) % g.world;
      const uint4 u = *reinterpret_cast<const uint4*>(g.p[pr] + i0), w = *reinterpret_cast<const uint4*>(g.p[pr] + i1);
      const uint32_t uu[4] = {u.x, u.y, u.z, u.w}, ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 a = unpack_bf16(uu[k]), b = unpack_bf16(ww[k]);
        o0[2 * k] += a.x; o0[2 * k + 1] += a.y; o1[2 * k] += b.x; o1[2 * k + 1] += b.y;
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { o0[j] *= g.scale; o1[j] *= g.scale; }
}

// grid (blocks_per_mat <= MUON_PARTS, n_mat); elements of matrix `mat` sit at bucket offset `offset + mat*per_mat`
__global__ void __launch_bounds__(256) muon_nesterov_rs_k(float* __restrict__ buf, GradPeers gp, long long offset,
                                                          __nv_bfloat16* __restrict__ u, float* __restrict__ partials,
                                                          long long per_mat, float mu) {
  const int mat = blockIdx.y;
  const long long base = (long long)mat * per_mat;
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  for (; i + stride < per_mat; i += 2 * stride) {
    float g0[8], g1[8];
    load_grad8x2(gp, offset + base + i, offset + base + i + stride, g0, g1);
    acc += nesterov8(buf, u, base + i, g0, mu);
    acc += nesterov8(buf, u, base + i + stride, g1, mu);
  }
  if (i < per_mat) {
    float g[8];
    load_grad8(gp, offset + base + i, g);
    acc += nesterov8(buf, u, base + i, g, mu);
  }
  muon_store_partial(acc, partials, mat);
}

__device__ __forceinline__ void adamw8(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                       __nv_bfloat16* __restrict__ shadow, long long i, const float (&g)[8], float lr, float b1,
                                       float b2, float eps, float wd, float bc1, float bc2) {
  float4 pa = *reinterpret_cast<float4*>(p + i), pb = *reinterpret_cast<float4*>(p + i + 4);
  float4 ma = *reinterpret_cast<float4*>(m + i), mb = *reinterpret_cast<float4*>(m + i + 4);
  float4 va = *reinterpret_cast<float4*>(v + i), vb = *reinterpret_cast<float4*>(v + i + 4);
  float pp[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
  float mm[8] = {ma.x, ma.y, ma.z, ma.w, mb.x, mb.y, mb.z, mb.w};
  float vv[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    pp[j] -= lr * wd * pp[j];
    mm[j] = b1 * mm[j] + (1.f - b1) * g[j];
    vv[j] = b2 * vv[j] + (1.f - b2) * g[j] * g[j];
    pp[j] -= lr * (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps);
  }
  *reinterpret_cast<float4*>(p + i) = make_float4(pp[0], pp[1], pp[2], pp[3]);
  *reinterpret_cast<float4*>(p + i + 4) = make_float4(pp[4], pp[5], pp[6], pp[7]);
  *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
  *reinterpret_cast<float4*>(m + i + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
  *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
  *reinterpret_cast<float4*>(v + i + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
  if (shadow) {
    uint4 u;
    u.x = pack_bf16(pp[0], pp[1]); u.y = pack_bf16(pp[2], pp[3]); u.z = pack_bf16(pp[4], pp[5]); u.w = pack_bf16(pp[6], pp[7]);
    *reinterpret_cast<uint4*>(shadow + i) = u;
  }
}

__global__ void __launch_bounds__(256) adamw_rs_k(float* __restrict__ p, GradPeers gp, long long offset, float* __restrict__ m,
                                                  float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, long long n, float lr,
                                                  float b1, float b2, float eps, float wd, float bc1, float bc2) {
  const long long stride = (long long)gridDim.x * blockDim.x * 8;
  long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  for (; i + stride < n; i += 2 * stride) {
    float g0[8], g1[8];
    load_grad8x2(gp, offset + i, offset + i + stride, g0, g1);
    adamw8(p, m, v, shadow, i, g0, lr, b1, b2, eps, wd, bc1, bc2);
    adamw8(p, m, v, shadow, i + stride, g1, lr, b1, b2, eps, wd, bc1, bc2);
  }
  if (i < n) {
    float g[8];
    load_grad8(gp, offset + i, g);
    adamw8(p, m, v, shadow, i, g, lr, b1, b2, eps, wd, bc1, bc2);
  }
}

static int fill_peers(GradPeers& gp, const void* const* peers, int world, int rank, const void* mc, float scale) {
  if (world < 1 || world > OPT_MAX_WORLD || rank < 0 || rank >= world) return -3;
  for (int i = 0; i < world; ++i) {
    if (!mc && (reinterpret_cast<uintptr_t>(peers[i]) & 15)) return -4;
    gp.p[i] = reinterpret_cast<const __nv_bfloat16*>(peers ? peers[i] : nullptr);
  }
  gp.mc = reinterpret_cast<const __nv_bfloat16*>(mc);
  gp.world = world; gp.rank = rank; gp.scale = scale;
  return 0;
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
static inline bool aligned16(const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr) {
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
           reinterpret_cast<uintptr_t>(d)) & 15) == 0;
}
// `partials`: n_mat x 64 floats (per-block partial sums of u^2, consumed by arb_muon_frob_scale)
int arb_muon_nesterov(float* buf, const float* grad, void* u_bf16, float* partials, long long per_mat, int n_mat, float mu, cudaStream_t s) {
  if (per_mat <= 0 || n_mat <= 0 || n_mat > 65535) return -3;
  if ((per_mat & 7) == 0 && aligned16(buf, grad, u_bf16)) {
    muon_nesterov_k<true><<<dim3(blocks_for(per_mat / 8, 256, MUON_PARTS), n_mat), 256, 0, s>>>(buf, grad, (__nv_bfloat16*)u_bf16, partials, per_mat, mu);
  } else {
    muon_nesterov_k<false><<<dim3(blocks_for(per_mat, 256 * 4, MUON_PARTS), n_mat), 256, 0, s>>>(buf, grad, (__nv_bfloat16*)u_bf16, partials, per_mat, mu);
  }
  return int(cudaGetLastError());
}
int arb_muon_nesterov_rs(float* buf, const void* const* peer_buckets, int world, int rank, const void* mc_bucket,
                         long long bucket_offset, float grad_scale, void* u_bf16, float* partials, long long per_mat, int n_mat,
                         float mu, cudaStream_t s) {
  if (per_mat <= 0 || (per_mat & 7) || (bucket_offset & 7) || n_mat <= 0 || n_mat > 65535) return -3;
  if (!aligned16(buf, u_bf16)) return -4;
  GradPeers gp;
  int rc = fill_peers(gp, peer_buckets, world, rank, mc_bucket, grad_scale);
  if (rc) return rc;
  const int bpm = blocks_for(per_mat / 8, 256, MUON_PARTS);
  muon_nesterov_rs_k<<<dim3(bpm, n_mat), 256, 0, s>>>(buf, gp, bucket_offset, (__nv_bfloat16*)u_bf16, partials, per_mat, mu);
  return int(cudaGetLastError());
}
int arb_adamw_rs(float* master, const void* const* peer_buckets, int world, int rank, const void* mc_bucket,
                 long long bucket_offset, float grad_scale, float* m, float* v, void* shadow_bf16, long long n, float lr,
                 float beta1, float beta2, float eps, float wd, float bc1, float bc2, cudaStream_t s) {
  if (n <= 0 || (n & 7) || (bucket_offset & 7)) return -3;
  GradPeers gp;
  int rc = fill_peers(gp, peer_buckets, world, rank, mc_bucket, grad_scale);
  if (rc) return rc;
  adamw_rs_k<<<blocks_for(n / 8, 256, 148 * 8), 256, 0, s>>>(master, gp, bucket_offset, m, v, (__nv_bfloat16*)shadow_bf16, n, lr, beta1,
                                                              beta2, eps, wd, bc1, bc2);
  return int(cudaGetLastError());
}
int arb_muon_frob_scale(void* u_bf16, const float* partials, long long per_mat, int n_mat, cudaStream_t s) {
  if (per_mat <= 0 || n_mat <= 0 || n_mat > 65535) return -3;
  if ((per_mat & 7) == 0 && aligned16(u_bf16))
    muon_frob_scale_k<true><<<dim3(blocks_for(per_mat / 8, 256, 64), n_mat), 256, 0, s>>>((__nv_bfloat16*)u_bf16, partials, per_mat);
  else
    muon_frob_scale_k<false><<<dim3(blocks_for(per_mat, 256 * 4, 64), n_mat), 256, 0, s>>>((__nv_bfloat16*)u_bf16, partials, per_mat);
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
  auto* sh = (__nv_bfloat16*)shadow_bf16;
  auto* xx = (const __nv_bfloat16*)x_bf16;
  if ((n & 7) == 0 && aligned16(master, shadow_bf16, x_bf16, scale)) {
    const dim3 grid(blocks_for((long long)m * n / 8, 256, 128), n_mat);
    if (m >= n) muon_update_k<true, true><<<grid, 256, 0, s>>>(master, sh, xx, scale, m, n, lr, wd);
    else muon_update_k<false, true><<<grid, 256, 0, s>>>(master, sh, xx, scale, m, n, lr, wd);
  } else {
    const dim3 grid(blocks_for((long long)m * n, 256 * 4, 64), n_mat);
    if (m >= n) muon_update_k<true, false><<<grid, 256, 0, s>>>(master, sh, xx, scale, m, n, lr, wd);
    else muon_update_k<false, false><<<grid, 256, 0, s>>>(master, sh, xx, scale, m, n, lr, wd);
  }
  return int(cudaGetLastError());
}

}  // extern "C"
