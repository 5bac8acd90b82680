// Collectives issued from kernels over NVLink peer memory (no library collective, no TMA
// from remote memory): every rank's bucket lives in a symmetric allocation that is mapped
// into all peers, so a kernel can read a peer's shard with plain loads or reduce across all
// ranks inside the NVSwitch with multimem.ld_reduce.
//
// The reference has no collective at all (its only cross-GPU traffic is pipeline send/recv,
// brain/src/nccl.rs:18-24, and cuMemcpyPeerAsync, brain/src/pipeline.rs:153-259).
#include "api.h"
#include "ptx.cuh"

namespace arb {

constexpr int MAX_WORLD = 16;
struct PeerPtrs { const void* p[MAX_WORLD]; };
struct PeerPtrsMut { void* p[MAX_WORLD]; };

// out[i] = scale * sum_p src_p[offset + i]
template <bool BF16>
__global__ void __launch_bounds__(256) reduce_scatter_peers_k(PeerPtrs peers, int world, int rank, long long offset, long long n,
                                                              float* __restrict__ out, float scale) {
  if (BF16) {
    const long long n8 = n >> 3;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int q = 0; q < world; ++q) {
        const int pr = (rank + q) % world;  // stagger so ranks do not all hit one peer at once
        const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peers.p[pr]) + offset + i * 8);
        float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
        acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
      }
      float4* o = reinterpret_cast<float4*>(out + i * 8);
      o[0] = make_float4(acc[0] * scale, acc[1] * scale, acc[2] * scale, acc[3] * scale);
      o[1] = make_float4(acc[4] * scale, acc[5] * scale, acc[6] * scale, acc[7] * scale);
    }
  } else {
    const long long n4 = n >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
      float4 acc = make_float4(0, 0, 0, 0);
      for (int q = 0; q < world; ++q) {
        const int pr = (rank + q) % world;
        const float4 v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peers.p[pr]) + offset + i * 4);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
      reinterpret_cast<float4*>(out)[i] = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
    }
  }
}

// out[i] = bf16(sum_s slab_s[i]), fp32 accumulation: the local half of a tensor-parallel reduce-scatter (the slabs
// were filled by the peers' GEMM epilogues or push copies; every read here is local memory).
__global__ void __launch_bounds__(256) sum_slabs_bf16_k(PeerPtrs slabs, int count, long long n8, uint4* __restrict__ out) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int q = 0; q < count; ++q) {
      const uint4 u = reinterpret_cast<const uint4*>(slabs.p[q])[i];
      float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y; acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]); o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    out[i] = o;
  }
}

// The same reduction performed by the switch: one multimem.ld_reduce per 16 bytes.
template <bool BF16>
__global__ void __launch_bounds__(256) reduce_scatter_mc_k(const void* mc, long long offset, long long n, float* __restrict__ out,
                                                           float scale) {
  if (BF16) {
    const long long n8 = n >> 3;
    const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(mc) + offset;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
      uint32_t r0, r1, r2, r3;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                   : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "l"(base + i * 8) : "memory");
      float2 a = unpack_bf16(r0), b = unpack_bf16(r1), c = unpack_bf16(r2), d = unpack_bf16(r3);
      float4* o = reinterpret_cast<float4*>(out + i * 8);
      o[0] = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
      o[1] = make_float4(c.x * scale, c.y * scale, d.x * scale, d.y * scale);
    }
  } else {
    const long long n4 = n >> 2;
    const float* base = reinterpret_cast<const float*>(mc) + offset;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
      float4 v;
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(base + i * 4) : "memory");
      reinterpret_cast<float4*>(out)[i] = make_float4(v.x * scale, v.y * scale, v.z * scale, v.w * scale);
    }
  }
}

// dst[i] = src[i] for i = first, first + stride, ... < n (16-byte units), four loads in flight per thread
__device__ __forceinline__ void copy16_unrolled(uint4* __restrict__ dst, const uint4* __restrict__ src, long long n, long long first,
                                                long long stride) {
  long long i = first;
  for (; i + 3 * stride < n; i += 4 * stride) {
    const uint4 a = src[i], b = src[i + stride], c = src[i + 2 * stride], d = src[i + 3 * stride];
    dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
  }
  for (; i < n; i += stride) dst[i] = src[i];
}

// dst_local[p-th shard] = peer_p[p-th shard] for every p != rank (16-byte units)
__global__ void __launch_bounds__(256) all_gather_pull_k(PeerPtrs peers, int world, int rank, uint4* __restrict__ local,
                                                         long long shard16) {
  // peer by peer (every rank starts with a different one), four independent 16-byte loads in flight per thread
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int q = 0; q < world - 1; ++q) {
    const int pr = (rank + 1 + q) % world;
    copy16_unrolled(local + (long long)pr * shard16, reinterpret_cast<const uint4*>(peers.p[pr]) + (long long)pr * shard16, shard16,
                    (long long)blockIdx.x * blockDim.x + threadIdx.x, stride);
  }
}

// Copies up to PULL_MAX_RANGES address ranges (16-byte units) from peer memory into local memory.
constexpr int PULL_MAX_RANGES = 96;
struct PullRanges {
  const uint4* src[PULL_MAX_RANGES];
  uint4* dst[PULL_MAX_RANGES];
  long long end16[PULL_MAX_RANGES];   // running end of each range in the concatenated index space
  int n;
};
__global__ void pull_ranges_k(const __grid_constant__ PullRanges r) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (int k = 0; k < r.n; ++k) {
    const long long n = r.end16[k] - (k ? r.end16[k - 1] : 0);
    copy16_unrolled(r.dst[k], r.src[k], n, (long long)blockIdx.x * blockDim.x + threadIdx.x, stride);
  }
}

__global__ void all_gather_push_k(PeerPtrsMut peers, int world, int rank, const uint4* __restrict__ src, long long off16, long long n16) {
  const long long total = n16 * (world - 1);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int q = int(i / n16);
    const long long j = i - (long long)q * n16;
    const int pr = (rank + 1 + q) % world;
    reinterpret_cast<uint4*>(peers.p[pr])[off16 + j] = src[off16 + j];
  }
}

// flags: int[world] per rank in symmetric memory.  Bounded wait (2 s of device time).
__global__ void peer_barrier_k(PeerPtrsMut flags, int world, int rank, int epoch, int* err) {
  const int t = threadIdx.x;
  if (t < world) {
    int* remote = reinterpret_cast<int*>(flags.p[t]) + rank;
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(epoch) : "memory");
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + t;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (v - epoch >= 0) break;
      if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
        if (err) atomicExch(err, ERR_COMM_TIMEOUT);
        break;
      }
      __nanosleep(200);
    }
  }
}

}  // namespace arb

using namespace arb;

static inline int comm_grid(long long work) {
  long long b = (work + 255) / 256;
  const long long cap = 148 * 4;
  return int(b < 1 ? 1 : (b > cap ? cap : b));
}

extern "C" {

int arb_reduce_scatter_peers(const void* const* peer_bufs, int world, long long offset, long long n, int src_is_bf16,
                             float* out, float scale, cudaStream_t s) {
  if (world < 1 || world > MAX_WORLD || n <= 0 || (n & 7) || (offset & 7)) return -3;
  PeerPtrs pp;
  for (int i = 0; i < world; ++i) pp.p[i] = peer_bufs[i];
  // peer_bufs[world] carries this rank's index (host array of world+1 entries)
  const int rank = int(reinterpret_cast<intptr_t>(peer_bufs[world]));
  if (src_is_bf16) reduce_scatter_peers_k<true><<<comm_grid(n / 8), 256, 0, s>>>(pp, world, rank, offset, n, out, scale);
  else reduce_scatter_peers_k<false><<<comm_grid(n / 4), 256, 0, s>>>(pp, world, rank, offset, n, out, scale);
  return int(cudaGetLastError());
}

int arb_sum_slabs_bf16(const void* const* slabs, int count, long long n, void* out_bf16, cudaStream_t s) {
  if (count < 1 || count > MAX_WORLD || n <= 0 || (n & 7) || (reinterpret_cast<uintptr_t>(out_bf16) & 15)) return -3;
  PeerPtrs pp;
  for (int i = 0; i < count; ++i) {
    if (reinterpret_cast<uintptr_t>(slabs[i]) & 15) return -4;
    pp.p[i] = slabs[i];
  }
  sum_slabs_bf16_k<<<comm_grid(n / 8), 256, 0, s>>>(pp, count, n / 8, reinterpret_cast<uint4*>(out_bf16));
  return int(cudaGetLastError());
}

int arb_reduce_scatter_multimem(const void* mc_ptr, long long offset, long long n, int src_is_bf16, float* out, float scale,
                                cudaStream_t s) {
  if (!mc_ptr || n <= 0 || (n & 7) || (offset & 7)) return -3;
  if (src_is_bf16) reduce_scatter_mc_k<true><<<comm_grid(n / 8), 256, 0, s>>>(mc_ptr, offset, n, out, scale);
  else reduce_scatter_mc_k<false><<<comm_grid(n / 4), 256, 0, s>>>(mc_ptr, offset, n, out, scale);
  return int(cudaGetLastError());
}

int arb_all_gather_push(void* const* peer_bufs, int world, int rank, const void* src, long long offset, long long n_bytes,
                        cudaStream_t s) {
  if (world < 1 || world > MAX_WORLD || n_bytes <= 0 || (n_bytes & 15) || (offset & 15)) return -3;
  if (world == 1) return 0;
  PeerPtrsMut pp;
  for (int i = 0; i < world; ++i) pp.p[i] = peer_bufs[i];
  all_gather_push_k<<<comm_grid(n_bytes / 16 * (world - 1)), 256, 0, s>>>(pp, world, rank, (const uint4*)src, offset / 16, n_bytes / 16);
  return int(cudaGetLastError());
}

int arb_all_gather_pull(const void* const* peer_bufs, int world, int rank, void* local, long long shard_bytes, cudaStream_t s) {
  if (world < 1 || world > MAX_WORLD || shard_bytes <= 0 || (shard_bytes & 15)) return -3;
  if (world == 1) return 0;
  PeerPtrs pp;
  for (int i = 0; i < world; ++i) pp.p[i] = peer_bufs[i];
  all_gather_pull_k<<<comm_grid(shard_bytes / 16 * (world - 1)), 256, 0, s>>>(pp, world, rank, (uint4*)local, shard_bytes / 16);
  return int(cudaGetLastError());
}

int arb_peer_barrier(int* const* peer_flags, int world, int rank, int epoch, int* err_flag, cudaStream_t s) {
  if (world < 1 || world > MAX_WORLD) return -3;
  PeerPtrsMut pp;
  for (int i = 0; i < world; ++i) pp.p[i] = peer_flags[i];
  peer_barrier_k<<<1, 32, 0, s>>>(pp, world, rank, epoch, err_flag);
  return int(cudaGetLastError());
}

// n ranges: dst[i][0..bytes[i]) = src[i][0..bytes[i]); pointers and sizes multiples of 16 bytes; one launch per
// PULL_MAX_RANGES ranges.
int arb_pull_ranges(const void* const* src, void* const* dst, const long long* bytes, int n, cudaStream_t s) {
  if (n < 0) return -3;
  for (int base = 0; base < n; base += PULL_MAX_RANGES) {
    PullRanges r;
    r.n = (n - base < PULL_MAX_RANGES) ? n - base : PULL_MAX_RANGES;
    long long run = 0;
    for (int i = 0; i < r.n; ++i) {
      const long long b = bytes[base + i];
      if (b <= 0 || (b & 15) || ((reinterpret_cast<uintptr_t>(src[base + i]) | reinterpret_cast<uintptr_t>(dst[base + i])) & 15)) return -3;
      r.src[i] = reinterpret_cast<const uint4*>(src[base + i]);
      r.dst[i] = reinterpret_cast<uint4*>(dst[base + i]);
      run += b / 16;
      r.end16[i] = run;
    }
    pull_ranges_k<<<comm_grid(run), 256, 0, s>>>(r);
    const int rc = int(cudaGetLastError());
    if (rc) return rc;
  }
  return 0;
}

}  // extern "C"
