// How fast can tcgen05.mma instructions be issued?  One CTA; W warps each issue R back-to-back
// M=128 x N x K=16 bf16 MMAs (operands in shared memory or, for A, in TMEM) into their own accumulator.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I autoresearch_b200/ops/csrc \
//        autoresearch_b200/bench/csrc/tcgen05_issue_rate.cu -o tcgen05_issue_rate && ./tcgen05_issue_rate
//
// Measured on B200 (clk per instruction, one issuing warp, R = 64): N=32 63, N=64 52-63, N=128 66-70,
// N=256 124-134, the same with A in TMEM; two or four issuing warps: N=64 50, N=128 66-68.  So an
// instruction costs about 50 clk to issue whatever its size, on the whole SM and not per warp: N=64
// (32 clk of tensor work) runs at 60 % of peak, N=128 (64 clk) at 97 %.  A batch of 8 followed by a
// commit and a wait costs about 80 clk per instruction.  The attention kernels therefore use N=128 only.
#include "ptx.cuh"
#include <cstdio>
using namespace arb;

template <int N, bool A_IN_TMEM>
__global__ void __launch_bounds__(128, 1) rate_k(long long* out, int R, int W) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar[4];
  __shared__ uint32_t slot;
  __shared__ int abort_flag;
  __shared__ long long tend[4], tbeg[4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 65536 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { for (int i = 0; i < 4; ++i) mbar_init(&bar[i], 1); abort_flag = 0; fence_barrier_init(); }
  fence_proxy_async_smem();
  if (warp == 0) { tmem_alloc(&slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = slot;
  constexpr int ACC = N > 128 ? 256 : 128;   // accumulator columns per issuing warp
  if (lane == 0 && warp < W) {
    constexpr uint32_t idesc = make_idesc_bf16(128, N, false, false);
    const uint32_t sa = smem_u32(smem), sb = smem_u32(smem + 16384);
    const uint64_t da = make_smem_desc(sa, 0, 1024), db = make_smem_desc(sb, 0, 1024);
    const long long t0 = clock64();
    for (int i = 0; i < R; ++i) {
      const uint64_t off = uint64_t((i & 3) * 2);   // +32 B k-step inside the 128-byte row, as the real kernels do
      if (A_IN_TMEM) tc_mma_ts(tmem + warp * ACC, tmem + ((warp + 1) % (512 / ACC)) * ACC + (i & 3) * 8, db + off, idesc, 1u);
      else tc_mma_ss(tmem + warp * ACC, da + off, db + off, idesc, 1u);
    }
    tc_commit(&bar[warp]);
    mbar_wait(&bar[warp], 0, &abort_flag);   // bounded
    tbeg[warp] = t0; tend[warp] = clock64();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    long long b = tbeg[0], e = tend[0];
    for (int w = 1; w < W; ++w) { b = min(b, tbeg[w]); e = max(e, tend[w]); }
    out[0] = e - b;
    out[1] = abort_flag;
  }
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int N, bool A_IN_TMEM>
void run(int R, int W, long long* d) {
  if (N > 128 && W > 2) return;
  cudaFuncSetAttribute(rate_k<N, A_IN_TMEM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 70000);
  rate_k<N, A_IN_TMEM><<<1, 128, 70000>>>(d, R, W);
  long long h[2] = {0, 0};
  cudaError_t e = cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
  printf("N=%3d A in %s  warps=%d  R=%3d each: %6.1f clk per MMA overall (tensor work %d clk)%s%s\n", N, A_IN_TMEM ? "TMEM" : "smem",
         W, R, double(h[0]) / (double(R) * W), N / 2, h[1] ? "  WAIT TIMED OUT" : "", e == cudaSuccess ? "" : cudaGetErrorString(e));
}

int main() {
  long long* d;
  cudaMalloc(&d, 128);
  for (int R : {8, 64})
    for (int W : {1, 2, 4}) {
      run<64, false>(R, W, d); run<128, false>(R, W, d); run<256, false>(R, W, d);
      run<64, true>(R, W, d); run<128, true>(R, W, d);
    }
  cudaFree(d);
  return 0;
}
