// C launchers of every sm_100a kernel (one per op, raw pointers + stream), the layer the
// reference exposes through brain/src/ffi.rs.  All return 0 on success, a cudaError_t or a
// negative argument-validation code otherwise.  Kernels that wait on barriers or peers
// never spin unbounded: on expiry they store one of the ERR_* codes to `err_flag` (device
// int, may be null) and return normally.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum ArbEpilogue {
  EPI_STORE_BF16 = 0,   // C = acc                      (bf16)
  EPI_RELU2 = 1,        // C = max(acc, 0)^2            (bf16)
  EPI_ATOMIC_F32 = 2,   // C += acc   (fp32, red.global; split-K allowed)
  EPI_NS_COMBINE = 3,   // C = alpha*I + beta*aux + gamma*acc   (bf16)
  EPI_RELU2_BWD = 4,    // C = acc * 2*sqrt(max(aux, 0)): aux = relu(h)^2 saved by the forward (bf16)
  EPI_STORE_F32 = 5,    // C = acc                      (fp32)
  EPI_ADD_AUX = 6,      // C = aux + acc                (bf16)
  EPI_QKV_POST = 7,     // packed q|k|v projection: RoPE + RMS norm on q and k heads, value embedding on v heads (bf16);
                        // 2-CTA tiles, NT layout; parameters from arb_gemm_qkv_post_args
};

enum ArbError {
  ERR_NONE = 0,
  ERR_GEMM_TIMEOUT = 1,
  ERR_ATTN_TIMEOUT = 2,
  ERR_COMM_TIMEOUT = 3,
  ERR_MOE_TIMEOUT = 4,
  ERR_SMEM_ALIGN = 5,   // dynamic shared memory base not 1 KB aligned (kernel returned before doing any work)
};

// Function attributes (dynamic shared memory size) belong to a device's context: a launcher sets them the first
// time it runs on EACH device, so that one process can drive several GPUs (the in-process pipeline driver).
struct PerDeviceOnce {
  unsigned long long done = 0;
  bool first() {
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) return true;
    const unsigned long long bit = 1ull << (d & 63);
    if (done & bit) return false;
    done |= bit;
    return true;
  }
};

extern "C" {

// ---- tensor-core GEMM (gemm_sm100.cu) ----------------------------------------------------
// C[b] (op)= A[b] * B[b];  A is M x K, B is K x N.  *_mn_major = 0: the operand is stored
// with K contiguous (A as [M, K], B as [N, K]); 1: with M (resp. N) contiguous (A as [K, M],
// B as [K, N]).  ld* / stride_* in elements.  splitk <= 0 = automatic (EPI_ATOMIC_F32 only).
int arb_gemm_bf16(const void* A, const void* B, void* C, const void* aux, int M, int N, int K, int batch,
                  long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                  long long stride_c, int a_mn_major, int b_mn_major, int epi, int splitk, float alpha, float beta,
                  float gamma, int* err_flag, cudaStream_t stream);

// The same with ragged batches (grouped expert GEMMs; device arrays, read by the kernel, no host synchronisation):
//   m_valid[batch]     rows of each batch item that hold data; output tiles starting at or beyond it are skipped
//                      (neither computed nor written).  b_div: B is indexed by batch_item / b_div, so b_div row slabs
//                      share one weight matrix (B then holds batch / b_div matrices).
//   k_valid[batch * (K / k_seg_rows)]   for EPI_ATOMIC_F32 products whose K dimension runs over rows: K is a sequence
//                      of segments of k_seg_rows rows (a multiple of 64), and of every segment only the 64-row blocks
//                      below k_valid are multiplied.  Rows between k_valid and the next multiple of 64 must be zero in
//                      at least one operand.
int arb_gemm_bf16_ragged(const void* A, const void* B, void* C, const void* aux, int M, int N, int K, int batch,
                         long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                         long long stride_c, int a_mn_major, int b_mn_major, int epi, int splitk, float alpha, float beta,
                         float gamma, int* err_flag, cudaStream_t stream, const void* pull_src, long long pull_bytes,
                         const void* ahead_src, void* ahead_dst, long long ahead_bytes, const int* m_valid, int b_div,
                         const int* k_valid, int k_seg_rows);
// Parameters of the next EPI_QKV_POST product on this host thread (consumed by it).  The product is
// [rows, D] x [3 * H * 128, D]^T; column blocks of 128 are heads: H query heads, H key heads, H value heads.
// Query and key heads are rotated (cos / sin: bf16 [T, 64], position = row % T; lo' = lo c + hi s, hi' = hi c - lo s)
// and divided by their RMS over 128 (its inverse goes to rstd_qk[row, 2H]).  With ve_w given, value head h gets
// 2 sigmoid(xn[row, :gate_ch] . gate_w[h]) * ve_w[ids[row], h] added; the gate logit goes to gate_out[row, H].
int arb_gemm_qkv_post_args(const void* cos_t, const void* sin_t, float* rstd_qk, int T, int H, const void* xn,
                           long long ld_xn, const int* ids, const void* ve_w, const void* gate_w, float* gate_out,
                           int gate_ch, float eps);

// Tile selection: 0 = automatic (2-CTA 256x256 tiles when M >= 512 and N >= 256, else 1-CTA
// 128x256/128x128), 1 = always 1-CTA, 2 = always 2-CTA.  Process-wide; meant for tests / benchmarks.
int arb_gemm_set_mode(int mode);
// The same GEMM with up to two copies from another GPU's memory folded into the kernel (the data-parallel
// all-gather of updated weights, see parallel/fused_dp.py).  Sizes are multiples of 16 bytes, pointers 16-byte
// aligned; a null source switches the copy off.
//   pull_src / pull_bytes   B itself is stale: every CTA first copies pull_src -> B (peer loads), the grid meets
//                           at a bounded counter barrier, then the tiles are computed.  Needs the whole grid
//                           resident (it is: one persistent CTA per SM).
//   ahead_src / ahead_dst / ahead_bytes   the operand of a LATER GEMM on the same stream: a spare warp of every CTA
//                           copies it while the tiles are computed; the kernel boundary orders the copy before its
//                           consumer.
int arb_gemm_bf16_ex(const void* A, const void* B, void* C, const void* aux, int M, int N, int K, int batch,
                     long long lda, long long ldb, long long ldc, long long stride_a, long long stride_b,
                     long long stride_c, int a_mn_major, int b_mn_major, int epi, int splitk, float alpha, float beta,
                     float gamma, int* err_flag, cudaStream_t stream, const void* pull_src, long long pull_bytes,
                     const void* ahead_src, void* ahead_dst, long long ahead_bytes);

// ---- flash attention (attn_sm100.cu) ----------------------------------------------------------
// q, k, v, o: [B, T, H, hd=128] bf16 with token stride `ld*` elements (head h at column
// h*128); lse: [B, H, T] fp32.  window >= T means plain causal; key j is visible to query i
// iff i - window <= j <= i.
// Backward variant: 2 (default) = 128 x 128 tiles with the two-phase softmax (attn_wide_sm100.cu);
// 1 = 64-wide sub-tiles, P / dS through TMEM; 0 = 64-wide sub-tiles, P / dS through shared memory.
// The forward hands P to the second MMA through TMEM unless the mode is 0.
void arb_attn_set_mode(int mode);
int arb_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int T, int H,
                 long long ldq, long long ldk, long long ldv, long long ldo, int window, float scale,
                 int* err_flag, cudaStream_t stream);
int arb_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                 void* dq, void* dk, void* dv, float* delta, float* dq_accum, int B, int T, int H, long long ldq,
                 long long ldk, long long ldv, long long ldo, long long lddo, long long lddq, long long lddk,
                 long long lddv, int window, float scale, int* err_flag, cudaStream_t stream);

// ---- row-wise fused norm / residual kernels (elementwise.cu) --------------------------------
int arb_rmsnorm_fwd(const void* x, void* y, long long rows, int D, float eps, cudaStream_t s);
// gx (=|+=) rmsnorm_bwd(x, g);  add_to != null: gx = add_to + rmsnorm_bwd
int arb_rmsnorm_bwd(const void* x, const void* g, const void* add_to, void* gx, long long rows, int D, float eps,
                    cudaStream_t s);
int arb_resid_scale_norm_fwd(const void* x, const void* x0, const void* lam_r, const void* lam_0, int idx,
                             void* x_out, void* xn_out, long long rows, int D, float eps, cudaStream_t s);
// t = g_xs + rmsnorm_bwd(x', g_xn);  d_x = lam_r*t;  d_x0 = lam_0*t (+ d_x0_acc when given; it may be d_x0 itself);
// dlam_r[idx] += sum(x*t);  dlam_0[idx] += sum(x0*t)   (fp32 atomics, one per CTA)
int arb_resid_scale_norm_bwd(const void* x, const void* x0, const void* lam_r, const void* lam_0, int idx,
                             const void* g_xs, const void* g_xn, void* d_x, void* d_x0, const void* d_x0_acc,
                             float* dlam_r, float* dlam_0, long long rows, int D, float eps, cudaStream_t s);
int arb_add_norm_fwd(const void* x, const void* proj, void* x_out, void* xn_out, long long rows, int D, float eps,
                     cudaStream_t s);
int arb_residual_add(const void* a, const void* b, void* out, long long n, cudaStream_t s);
int arb_relu_sq_fwd(const void* x, void* y, long long n, cudaStream_t s);
int arb_relu_sq_bwd(const void* x, const void* g, void* gx, long long n, cudaStream_t s);
// In-place on the packed qkv buffer [N, 3*H*128]: RoPE + per-head RMSNorm on the q and k
// column blocks (rstd saved to rstd_qk [N, 2H] fp32); on value-embedding layers also
// v += 2*sigmoid(xn[:, :32] . Wg[h]) * VE[ids]   (gate logits saved to gate_out [N, H] fp32).
int arb_qkv_post_fwd(void* qkv, const void* cos_t, const void* sin_t, float* rstd_qk, const void* xn,
                     const int* ids, const void* ve_w, const void* gate_w, float* gate_out, long long N, int T,
                     int H, int D_model, int gate_ch, float eps, cudaStream_t s);
// In-place on d_qkv: norm/RoPE backward on the q, k blocks (needs the forward outputs in
// qkv); value-embedding backward: d_ve (dense [N, H*128] bf16), d_gate_w += (fp32 [H, ch]),
// d_xn_gate [N, ch] bf16; dgl is caller-provided scratch of N*H floats (gate-logit gradient).
int arb_qkv_post_bwd(void* d_qkv, const void* qkv, const void* cos_t, const void* sin_t, const float* rstd_qk,
                     const void* xn, const int* ids, const void* ve_w, const void* gate_w, const float* gate,
                     void* d_ve, float* d_gate_w, void* d_xn_gate, float* dgl, long long N, int T, int H,
                     int D_model, int gate_ch, cudaStream_t s);
int arb_embedding_fwd(const int* ids, const void* w, void* out, long long N, int D, int vocab, cudaStream_t s);
// dW[ids[i], :] += g[i, :]  (fp32 accumulate with red.global)
int arb_embedding_bwd(const int* ids, const void* g, float* dw, long long N, int D, int vocab, cudaStream_t s);
// deterministic (sorted, atomic-free) form of arb_embedding_bwd; see elementwise.cu for the plan arrays
int arb_embedding_bwd_sorted(const long long* perm, const int* item_id, const int* item_start, const int* seg_start,
                             const int* seg_count, const void* g, float* dw, float* partial, int n_items_max, int D, int R,
                             int vocab, cudaStream_t s);
int arb_add_cols(void* dst, long long ld_dst, const void* src, long long rows, int cols, cudaStream_t s);
int arb_cast_f32_to_bf16(const float* src, void* dst, long long n, float scale, cudaStream_t s);
int arb_accum_bf16_into_f32(const void* src, float* dst, long long n, cudaStream_t s);

// ---- soft-capped cross entropy (cross_entropy.cu) ------------------------------------------
// logits [rows, V] bf16 (row stride ld).  Writes per-token loss; if dlogits_scale != 0 the
// logits are overwritten in place by d_logits = (p - 1[tgt]) * scale * (1 - (s/cap)^2).
int arb_softcap_ce(void* logits, long long ld, const int* targets, float* loss, long long rows, int V,
                   float softcap, float dlogits_scale, cudaStream_t s);

// ---- optimizer (optim.cu) -----------------------------------------------------------------------
int arb_adamw(float* master, const float* grad, float* m, float* v, void* shadow_bf16, long long n, float lr,
              float beta1, float beta2, float eps, float wd, float bc1, float bc2, cudaStream_t s);
// buf = mu*buf + (1-mu)*g ; u = (1-mu)*g + mu*buf -> bf16 ; partials[mat][64] = per-block sums of u_bf16^2
// (no atomics: arb_muon_frob_scale adds the 64 slots in a fixed order)
int arb_muon_nesterov(float* buf, const float* grad, void* u_bf16, float* partials, long long per_mat, int n_mat,
                      float mu, cudaStream_t s);
// The same two updates with the data-parallel reduce-scatter fused in: the gradient of element i
// is grad_scale * sum_p bucket_p[bucket_offset + i] over all ranks' bf16 buckets, read through
// NVLink peer pointers (HOST array peer_buckets, world entries) or, when mc_bucket is non-null,
// with one multimem.ld_reduce through the switch.  n / per_mat / bucket_offset multiples of 8.
int arb_muon_nesterov_rs(float* buf, const void* const* peer_buckets, int world, int rank, const void* mc_bucket,
                         long long bucket_offset, float grad_scale, void* u_bf16, float* partials, long long per_mat,
                         int n_mat, float mu, cudaStream_t s);
int arb_adamw_rs(float* master, const void* const* peer_buckets, int world, int rank, const void* mc_bucket,
                 long long bucket_offset, float grad_scale, float* m, float* v, void* shadow_bf16, long long n,
                 float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2, cudaStream_t s);
// x = u / (sqrt(sum of partials[mat][0..63])*1.02 + 1e-6)
int arb_muon_frob_scale(void* u_bf16, const float* partials, long long per_mat, int n_mat, cudaStream_t s);
// NorMuon statistics + cautious update, per matrix [m, n]; reduce over columns if m >= n.
int arb_normuon_stats(const void* x_bf16, float* v_mean, int n_mat, int m, int n, cudaStream_t s);
int arb_normuon_scales(const float* v_mean, float* second, float* scale, int n_mat, int n_stat, int red_size,
                       float beta2, cudaStream_t s);
int arb_muon_update(float* master, void* shadow_bf16, const void* x_bf16, const float* scale, int n_mat, int m,
                    int n, float lr, float wd, cudaStream_t s);

// ---- peer-memory collectives (comm.cu) ----------------------------------------------------------
// out[i] = scale * sum_p peer_p[offset + i] for i in [0, n): every peer pointer addresses that
// rank's whole gradient bucket (bf16 or fp32) mapped into this process.
// peer_bufs is a HOST array of world+1 entries: the world peer pointers, then this rank's
// index cast to a pointer.
int arb_reduce_scatter_peers(const void* const* peer_bufs, int world, long long offset, long long n, int src_is_bf16,
                             float* out, float scale, cudaStream_t s);
// out[i] = bf16(sum over the `count` bf16 buffers slabs[s][i]), fp32 accumulation; n a multiple of 8.
int arb_sum_slabs_bf16(const void* const* slabs, int count, long long n, void* out_bf16, cudaStream_t s);
int arb_reduce_scatter_multimem(const void* mc_ptr, long long offset, long long n, int src_is_bf16, float* out,
                                float scale, cudaStream_t s);
// push this rank's shard [offset, offset+n) of `src` to the same offset of every peer buffer
int arb_all_gather_push(void* const* peer_bufs, int world, int rank, const void* src, long long offset,
                        long long n_bytes, cudaStream_t s);
// local[p-th shard] = peer_p[p-th shard] for every p != rank (peer_bufs: host array)
int arb_all_gather_pull(const void* const* peer_bufs, int world, int rank, void* local, long long shard_bytes,
                        cudaStream_t s);
// Bounded flag barrier among ranks: each rank writes `epoch` to flags[rank] of every peer,
// then waits (<= 2 s) until all of its own flags reach `epoch`.
// dst[i][0..bytes[i]) = src[i][0..bytes[i]) for n ranges (peer or local memory), 16-byte granularity
int arb_pull_ranges(const void* const* src, void* const* dst, const long long* bytes, int n, cudaStream_t s);
int arb_peer_barrier(int* const* peer_flags, int world, int rank, int epoch, int* err_flag, cudaStream_t s);

// ---- mixture of experts (moe.cu) ---------------------------------------------------------------
// Router: probs [N,E] fp32 = softmax(xn . Wr^T); idx [N,K]; gates [N,K] = p_k / sum_top p.
int arb_moe_router_fwd(const void* xn, const void* wr, float* probs, int* idx, float* gates, long long N, int D,
                       int E, int K, cudaStream_t s);
// d_logits [N,E] bf16 (row stride ld >= E) from d_gates [N,K] and a per-expert constant added to
// d_probs (aux loss).
int arb_moe_router_bwd(const float* probs, const int* idx, const float* gates, const float* d_gates,
                       const float* aux_dp, void* d_logits, long long ld, long long N, int E, int K,
                       cudaStream_t s);
// expert_bufs: HOST array of E device pointers (local or NVLink peer mappings) to [rows, D] bf16
// buffers; row [N,K] = destination row of each slot inside its expert's buffer, -1 = dropped.
// pos[s] = rank of slot s among the slots of its expert (token-major order), counts[e] = slots per expert;
// scratch holds ceil(S / 1024) * E ints
int arb_moe_slot_positions(const int* idx, long long S, int E, int* scratch, int* pos, int* counts, cudaStream_t s);
int arb_moe_dispatch(const void* x, void* const* expert_bufs, const int* idx, const int* row, long long N, int K,
                     int D, int E, cudaStream_t s);
// After a dispatch (or the backward's scatter of output gradients): *count_slots[e] = c = min(counts[e], keep), keep <= cap
// = rows of a slab, when the slot pointer is non-null (with expert parallelism it points into the owner's row-count table: a peer store), and rows
// [c, next multiple of `tile`) of expert e's slab are zeroed (the grouped GEMMs work in whole tiles of `tile` rows).
int arb_moe_finish_dispatch(void* const* expert_bufs, int* const* count_slots, const int* counts, int keep, int cap, int D,
                            int E, int tile, cudaStream_t s);
// out[t] = resid[t] + sum_k gates[t,k] * buf[idx][row]  (resid / gates may be null: 0 / 1)
int arb_moe_combine_fwd(const void* resid, void* const* expert_bufs, const int* idx, const int* row,
                        const float* gates, void* out, long long N, int K, int D, int E, cudaStream_t s);
// dy_buf[idx][row] = gates * d_out[t];  d_gates[t,k] = <y, d_out[t]> where y is y_buf[idx][row]
// or, when y_rows is given, row t*K+k of that dense [N*K, D] tensor (expert outputs saved by slot).
int arb_moe_combine_bwd(const void* d_out, void* const* y_bufs, const void* y_rows, void* const* dy_bufs,
                        const int* idx, const int* row, const float* gates, float* d_gates, long long N, int K, int D,
                        int E, cudaStream_t s);

}  // extern "C"
