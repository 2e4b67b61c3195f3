// C entry points of the sm_100a kernel library.  Every function enqueues work on `stream`
// and returns 0 on success or a negative code for a rejected argument / failed launch.
// Pointers are device pointers unless stated otherwise.  No function allocates memory.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---------------------------------------------------------------- GEMM (gemm_tcgen05.cu)
enum { OLB_GEMM_DENSE = 0, OLB_GEMM_RAGGED_M = 1, OLB_GEMM_RAGGED_K = 2 };
enum { OLB_EPI_PLAIN = 0, OLB_EPI_SWIGLU = 1, OLB_EPI_SWIGLU_BWD = 2 };

typedef struct {
  const void* A;  // bf16. K-major: [a_rows, K] with row stride lda; MN-major: [a_rows (=K extent), M]
  const void* B;  // bf16. K-major: [b_rows, K] with row stride ldb; MN-major: [b_rows (=K extent), N]
  void* C;        // bf16 (or fp32 when out_fp32), row-major [M, N], row stride ldc
  long long lda, ldb, ldc;  // in elements
  long long a_rows, b_rows; // outer extent of the operand's 2D view (bounds for TMA)
  int M, N, K;
  int a_mn_major, b_mn_major;
  int mode;                  // OLB_GEMM_*
  const int* meta;           // RAGGED_M: [0]=#row blocks, [1+i]=expert of block i; RAGGED_K: row offsets [E+1]
  int num_experts;
  int b_expert_rows;
  long long c_expert_stride;
  int accumulate;
  int out_fp32;
  int block_n;               // 0 = choose
  int max_ctas;              // 0 = all SMs
  int* status;               // device status word (may be NULL)
  const void* B2;            // optional second B of the same layout: K range [k_split, K) is read from it
  int k_split;               // multiple of 64; 0 = single B
  // All-gather fused into the GEMM (dense mode, A K-major): n_peers > 0 enables it.  A is this GPU's gathered copy
  // [n_peers * a_peer_rows, K]; its own a_peer_rows rows (block my_peer) are already there.  A_peers[r] points at
  // peer r's slice [a_peer_rows, K] (mapped in this process, row stride lda).  Extra warps of every CTA copy the
  // other peers' rows into A over NVLink and count them per 128-row block in stage_flags (zero at launch, one int
  // per block); the TMA producer waits for a block's count before it loads tiles of it, and the tile order starts
  // on the rows this GPU owns.  Each remote row crosses NVLink once.
  int n_peers, my_peer;
  const void* const* A_peers;
  int a_peer_rows;
  int* stage_flags;
  // Reduce-scatter's transport fused into the GEMM (dense mode): n_peers > 0 with C_peers set (and A_peers null).
  // C [n_peers * a_peer_rows, N] is this GPU's partial result; row block r of it belongs to peer r.  The epilogue
  // counts finished tiles per 128-row block in stage_flags (zero at launch), and the extra warps copy each
  // finished row of another peer's block to C_peers[r] (that peer's receive slot for this GPU, [a_peer_rows, N] with
  // row stride ldc) with stores over NVLink.  The tile order starts on the next peer's rows and ends on this GPU's
  // own.  The sum over the slots is a local pass after a barrier.
  void* const* C_peers;
  // Expert-parallel combine transport (RAGGED_M mode with n_peers > 0 and C_peers set): row u of C is the expert
  // output of the routed pair (token ep_src_of[u] in the group-wide numbering with ep_tokens tokens per rank, choice
  // ep_k_of[u]); once every tile of its 128-row block is stored (stage_flags, zero at launch) the extra warps copy
  // it to C_peers[owner] + ((token % ep_tokens) * ep_topk + k) * N: the owner's receive buffer [ep_tokens, ep_topk, N].
  const int* ep_src_of;
  const int* ep_k_of;
  int ep_tokens, ep_topk;
  const int* blk_range;      // RAGGED_M, optional (device memory): only row blocks [blk_range[0], blk_range[1])
  // Expert-parallel dispatch fused into the GEMM (RAGGED_M mode with n_peers > 0, A_peers set, C_peers null): row u of
  // A is token ep_src_of[u] of the group-wide numbering (ep_tokens per rank); extra warps copy it from
  // A_peers[token / ep_tokens] + (token % ep_tokens) * a_src_ld into A + u * lda (zeros for padding rows) and count the
  // rows per 128-row block in stage_flags (zero at launch); the TMA producer waits for a block before it loads it.
  // With n_peers == 1 this is the local permutation of the tokens into expert-grouped rows.
  long long a_src_ld;
  // Fused gate|up projection (epilogue == OLB_EPI_SWIGLU; DENSE or RAGGED_M, K-major operands): B / B2 are the gate /
  // up weights ([b_rows, K], b_expert_rows rows per expert), N the width of one of them per expert.  One tile holds
  // 128 gate and the matching 128 up columns; the epilogue writes gate | up to C [M, 2 N] (row stride ldc) and
  // w(row) * silu(gate) * up to C2 [M, N] (row stride ldc2), computed from the bf16-rounded gate and up values.
  // w(row) = row_weights[row_src_of[row] * row_topk + row_k_of[row]], 0 where row_src_of[row] < 0; 1 when the three
  // pointers are null.
  int pair_rows;             // RAGGED_M: the expert groups are padded to 256 rows (olb_moe_build_index with row_pad
                             // 256), which lets two CTAs on neighbouring SMs share one 256-row tile
  int epilogue;
  void* C2;
  long long ldc2;
  const int* row_src_of;
  const int* row_k_of;
  const float* row_weights;
  int row_topk;
  // Down projection's input gradient with the SwiGLU backward in the epilogue (epilogue == OLB_EPI_SWIGLU_BWD;
  // RAGGED_M with pair_rows, N a multiple of 256): the product d(act) [M, N] stays in the accumulator; aux_in is the
  // saved gate | up [M, 2 N] (row stride aux_ld), C receives d(gate) | d(up) [M, 2 N], and aux_out [M, N / 256] the
  // per-row, per-column-tile partial of <d(act), silu(gate) * up> (the routing-weight gradient before its small sum).
  const void* aux_in;
  long long aux_ld;
  float* aux_out;
  // Parameter all-gather fused into the first GEMM that consumes a weight (DENSE mode, B K-major and contiguous [N, K];
  // n_peers > 0 with B_peers set): after a sharded optimizer step the elements [b_seg[2r], b_seg[2r+1]) of B (counted
  // from B's first element, multiples of 8; empty for this GPU itself) are current only in peer r's copy B_peers[r].
  // Extra warps copy them into B over NVLink while the tiles whose rows of B are already complete run; stage_flags
  // (one int per 128 rows of B, zero at launch) counts the 16-byte vectors landed.  B is complete when the launch ends.
  const void* const* B_peers;
  const long long* b_seg;    // host array [2 * n_peers]
} olb_gemm_desc;

int olb_gemm_bf16(const olb_gemm_desc* d, cudaStream_t stream);

// ---------------------------------------------------------------- normalisation (norm.cu)
// y = x * rsqrt(mean(x^2) + eps) * w   (w may be NULL).  rstd [rows] fp32 is saved for backward.
int olb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps,
                    cudaStream_t stream);
// dx and, when dw_partial != NULL, per-block partial sums of dw ([olb_rmsnorm_bwd_blocks(rows), cols] fp32).
int olb_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_partial,
                    int rows, int cols, cudaStream_t stream);
int olb_rmsnorm_bwd_blocks(int rows);
// Residual add fused with the norm: h = a + b (bf16), y = rmsnorm(h) * w, rstd of h.
int olb_add_rmsnorm_fwd(const void* a, const void* b, const void* w, void* h, void* y, float* rstd, int rows, int cols,
                        float eps, cudaStream_t stream);
// olb_rmsnorm_bwd with the residual path's gradient `dres` [rows, cols] (may be NULL) added to dx.
int olb_rmsnorm_bwd_res(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw_partial,
                        const void* dres, int rows, int cols, cudaStream_t stream);
// dw[cols] (bf16 or fp32 by dw_fp32) (+)= sum over `nparts` rows of dw_partial.
int olb_colsum_finalize(const float* partial, int nparts, int cols, void* dw, int dw_fp32, int accumulate,
                        cudaStream_t stream);
// Non-parametric LayerNorm (fp32 statistics), saves mean and rstd.
int olb_layernorm_fwd(const void* x, void* y, float* mean, float* rstd, int rows, int cols, float eps,
                      cudaStream_t stream);
int olb_layernorm_bwd(const void* dy, const void* x, const float* mean, const float* rstd, void* dx, int rows,
                      int cols, cudaStream_t stream);

// ---------------------------------------------------------------- activation / rope (elementwise.cu)
// act[r, i] = silu(g[r,i]) * u[r,i];   g, u, act have their own row strides (elements).
int olb_swiglu_fwd(const void* g, long long ldg, const void* u, long long ldu, void* act, long long ldact,
                   long long rows, int cols, cudaStream_t stream);
int olb_swiglu_bwd(const void* dact, long long lddact, const void* g, long long ldg, const void* u, long long ldu,
                   void* dg, long long lddg, void* du, long long lddu, long long rows, int cols,
                   cudaStream_t stream);
// Expert-MLP activation with the routing weight folded in (rows are the expert-grouped rows of
// olb_moe_build_index): act[row] = weights[src_of[row], k_of[row]] * silu(g) * u; padding rows -> 0.
int olb_swiglu_rowscale_fwd(const void* g, long long ldg, const void* u, long long ldu, const int* src_of,
                            const int* k_of, const float* weights, int K, const int* meta, void* act,
                            long long ldact, int cap, int cols, cudaStream_t stream);
// Backward of the above; also dweights[t,k] = <dact[row], silu(g)*u> (dweights may be NULL).
int olb_swiglu_rowscale_bwd(const void* dact, long long lddact, const void* g, long long ldg, const void* u,
                            long long ldu, const int* src_of, const int* k_of, const float* weights, int K,
                            const int* meta, void* dg, long long lddg, void* du, long long lddu, float* dweights,
                            int cap, int cols, cudaStream_t stream);
// In-place rotary embedding on x [tokens, heads, head_dim] (bf16), token t uses position t % seq_len.
// cos/sin: fp32 [seq_len, rot_dim].  interleaved: pairs (2i, 2i+1) are de-interleaved first and the
// result is left in de-interleaved order.  conj != 0 applies the inverse rotation (backward).
int olb_rope_inplace(void* x, long long token_stride, int tokens, int heads, int head_dim, int rot_dim,
                     int seq_len, const float* cos_tab, const float* sin_tab, int interleaved, int conj,
                     cudaStream_t stream);

// ---------------------------------------------------------------- router (router.cu)
// Softmax over experts in fp32, top-k (ties -> lowest index), optional renormalisation.
// logits bf16 [T, E]; out: weights fp32 [T, K], indices int32 [T, K];
// optional per-block partials for the load-balance loss: cnt_partial/prob_partial [blocks, E] and
// lse_sq_partial [blocks] (sum of logsumexp^2, for the z-loss).
int olb_router_softmax_topk(const void* logits, int T, int E, int K, int renorm, float* weights, int* indices,
                            float* cnt_partial, float* prob_partial, float* lse_sq_partial, cudaStream_t stream);
int olb_router_blocks(int T);
// dlogits [T,E] (bf16) = softmax-backward of (d_weights scattered to the selected experts, with the
// renormalisation chain) + aux_scale * p o (f - <f,p>) + z_scale * 2 * lse * p
int olb_router_bwd(const void* logits, const int* indices, const float* dweights, int T, int E, int K, int renorm,
                   const float* aux_f, float aux_scale, float z_scale, void* dlogits, cudaStream_t stream);
// Same, with the aux/z scales additionally multiplied by *aux_scale_dev (a device scalar, e.g. the
// upstream gradient of the auxiliary loss) when it is not NULL.
int olb_router_bwd_ex(const void* logits, const int* indices, const float* dweights, int T, int E, int K,
                      int renorm, const float* aux_f, const float* aux_scale_dev, float aux_scale, float z_scale,
                      void* dlogits, cudaStream_t stream);
// DeepSeek-V3 router: sigmoid scores (+bias for selection only), group-limited top-k, renorm, scale.
int olb_router_sigmoid_group_topk(const float* logits, const float* bias, int T, int E, int K, int n_group,
                                  int topk_group, int renorm, float scale, float* weights, int* indices,
                                  cudaStream_t stream);
int olb_router_sigmoid_bwd(const float* logits, const int* indices, const float* dweights, int T, int E, int K,
                           int renorm, float scale, float* dlogits, cudaStream_t stream);

// ---------------------------------------------------------------- MoE permutation (moe.cu)
// Build the expert-grouped row layout for the pairs (t,k) whose expert lies in
// [e_start, e_start+E_loc).  Each expert's rows start at a multiple of `row_pad` (128, or 256 so that a pair of CTAs
// can share a 256-row GEMM tile; `cap` must be a multiple of it).
//   ws          : int workspace, at least olb_moe_ws_ints(T, E_loc) ints
//   row_of      : [T, K]   destination row of pair (t,k) or -1
//   src_of,k_of : [cap]    source token / k slot of each row, -1 for padding rows
//   meta        : [1 + cap/128] GEMM tile table (see OLB_GEMM_RAGGED_M)
//   offsets     : [E_loc+1] padded row offsets (see OLB_GEMM_RAGGED_K); counts: [E_loc] true counts
// If the padded rows exceed `cap`, status receives ST_OVERFLOW and the excess pairs get row -1.
int olb_moe_build_index(const int* indices, int T, int K, int e_start, int E_loc, int cap, int row_pad, int* ws,
                        int* row_of, int* src_of, int* k_of, int* meta, int* offsets, int* counts, int* status,
                        cudaStream_t stream);
// out[src_of[row] * K + k_of[row]] = sum_j partial[row * nblk + j] for the routed rows below meta[0] * 128 (fixed order).
int olb_moe_scatter_dweights(const float* partial, int nblk, const int* src_of, const int* k_of, const int* meta, int K,
                             float* out, int cap, cudaStream_t stream);
long long olb_moe_ws_ints(int T, int E_loc);
// out[row,:] = src_of[row] >= 0 ? x[src_of[row],:] : 0   for row < meta[0]*128   (bf16, cols % 8 == 0)
int olb_moe_gather_rows(const void* x, const int* src_of, const int* meta, void* out, int cap, int cols,
                        cudaStream_t stream);
// out[t,:] = sum_k w[t,k] * y[row_of[t,k],:]  (fp32 accumulation; w == NULL means 1)
int olb_moe_combine(const void* y, const int* row_of, const float* w, void* out, int T, int K, int cols,
                    cudaStream_t stream);
// dy[row,:] = w[t,k] * dout[t,:]; dw[t,k] = <y[row,:], dout[t,:]>  (rows < meta[0]*128; padding rows -> 0)
int olb_moe_combine_bwd(const void* dout, const void* y, const int* src_of, const int* k_of, const int* meta,
                        const float* w, void* dy, float* dw, int cap, int K, int cols, cudaStream_t stream);

// ---------------------------------------------------------------- loss (loss.cu)
// Per-row cross entropy on bf16 logits [rows, V] (row stride ldl) with int64 labels (ignore < 0).
// loss_row [rows] fp32 (0 for ignored rows), lse [rows] fp32.
int olb_ce_fwd(const void* logits, long long ldl, const long long* labels, float* loss_row, float* lse, int rows,
               int V, cudaStream_t stream);
// dlogits = (softmax - onehot) * (*scale_dev); may alias logits.
int olb_ce_bwd(const void* logits, long long ldl, const long long* labels, const float* lse, const float* scale_dev,
               void* dlogits, int rows, int V, cudaStream_t stream);
// Vocabulary-parallel cross entropy: statistics of the slice [v_start, v_start + V) per row (maximum, sum of
// exponentials relative to it, target logit or 0), and the slice's gradient from the merged log-sum-exp.
int olb_ce_partial_fwd(const void* logits, long long ldl, const long long* labels, int v_start, float* part_max,
                       float* part_sum, float* part_tgt, int rows, int V, cudaStream_t stream);
int olb_ce_partial_bwd(const void* logits, long long ldl, const long long* labels, int v_start, int v_total,
                       const float* lse, const float* scale_dev, void* dlogits, int rows, int V, cudaStream_t stream);

// ---------------------------------------------------------------- optimizer (adamw.cu)
typedef struct {
  float lr, beta1, beta2, eps, weight_decay;
  float bias_correction1, bias_correction2;  // 1 - beta^t
  float grad_scale;                          // applied to the gradient before everything else
  int skip_weight_update;
} olb_adamw_hparams;
// Sum of squares of (grad * grad_scale) -> partial [olb_sumsq_blocks(n)] fp32 (deterministic).
int olb_sumsq_partial(const void* grad, int grad_fp32, long long n, float grad_scale, float* partial,
                      cudaStream_t stream);
int olb_sumsq_blocks(long long n);
// out[0] = sum(partial[0..nparts))  (+= when accumulate)
int olb_sum_finalize(const float* partial, int nparts, float* out, int accumulate, cudaStream_t stream);
// AdamW of the reference form on one flat shard: g = grad*grad_scale*(*clip_coef_dev or 1);
// m,v update; master -= lr*mhat/(sqrt(vhat)+eps); master += master*(-lr*wd); param = cast(master).
// `norm_partial` (optional): olb_adamw_blocks(n) floats that receive, per block, the sum of squares of the scaled,
// unclipped gradients - the gradient norm without a pass of its own.
int olb_adamw_blocks(long long n);
int olb_adamw_step(const void* grad, int grad_fp32, float* master, float* m, float* v, void* param, int param_fp32,
                   long long n, const olb_adamw_hparams* hp, const float* clip_coef_dev, float* norm_partial,
                   cudaStream_t stream);

// ---------------------------------------------------------------- reference custom-op interface (customops.cu)
// The seven entry points of the reference's pcl_xpu_customops extension on its data layout (see customops.cu).
// int32 indices; data bf16, or fp32 when `fp32` is set.
int olb_co_partial_token_counts(const int* sel, int T, int K, int e_start, int E_loc, int* partial, int* counts_ep,
                                cudaStream_t stream);
int olb_co_input_output_indices(const int* sel, int T, int K, int e_start, int E_loc, const int* partial_cum, int* incr,
                                const int* cum_ep, int* sel_idx, int* in_idx, int* out_idx, cudaStream_t stream);
int olb_co_index_gather(const void* inp, const int* idx, void* out, int rows_out, int cols, int fp32, cudaStream_t stream);
// out[t] (+)= sum over the slots of t of w * y[out_idx[slot]]; weights NULL = unweighted (shuffle_sub_matrix_reduce).
int olb_co_reduce(const void* y, const void* weights, int K, const int* cum_ep, const int* sel_idx, const int* out_idx,
                  void* out, int T, int cols, int accumulate, int fp32, cudaStream_t stream);
int olb_co_reduce_bwd(const void* dout, const void* y, const void* weights, int K, const int* cum_ep, const int* sel_idx,
                      const int* out_idx, void* dy, void* dw, int T, int cols, int fp32, cudaStream_t stream);
int olb_co_index_add(const void* src, void* dst, const int* idx, int rows, int cols, int fp32, cudaStream_t stream);

// ---------------------------------------------------------------- peer-memory kernels (comm_p2p.cu)
// Host arrays of n (<= 16) device pointers, one per rank of the group, into symmetric buffers.
// Rendezvous of all ranks through signal words pads[rank][channel*16 + src]; `epoch` must grow by one
// per use of a channel.  Bounded wait (`wait_limit_ns`, 0 = the library's default of 4 s); a timeout sets *status to
// ST_TIMEOUT_PEER (5) and the kernel returns, so the context stays usable.
int olb_symm_barrier(void* const* pads, int my_rank, int n, int channel, unsigned epoch, int* status,
                     unsigned long long wait_limit_ns, cudaStream_t stream);
// idx_all[p][off + i] = idx[i], w_all[p][off + i] = w[i] for every peer p and i < count (all-gather by stores).
int olb_ep_publish_meta(void* const* idx_all, void* const* w_all, int n, const int* idx, const float* w, long long off,
                        long long count, cudaStream_t stream);
// out[t, :] = sum_k recv[t, k, :] (bf16 [T, K, cols] -> bf16 [T, cols], fp32 accumulation, fixed order).
int olb_sum_slots(const void* recv, int T, int K, int cols, void* out, cudaStream_t stream);
// out[row,:] = peer_x[g / T][g % T, :], g = src_of[row] (global token id), rows < meta[0]*128; padding -> 0.
int olb_ep_gather_rows(const void* const* peer_x, int n, int T, const int* src_of, const int* meta,
                       const int* blk_range, void* out, int cap, int cols, cudaStream_t stream);
// rows[t,k] = peer_row_of[d][(my_rank*T+t)*K+k], d = idx[t,k] / E_loc  (row of each of my pairs on its owner).
int olb_ep_resolve_rows(const void* const* peer_row_of, int n, const int* idx, int my_rank, int T, int K, int E_loc,
                        int* rows, cudaStream_t stream);
// out[t,:] = sum_k peer_y[d][rows[t,k], :] with d = idx[t,k] / E_loc (fp32 accumulation; rows < 0 skipped).
int olb_ep_combine(const void* const* peer_y, int n, const int* rows, const int* idx, int T, int K, int E_loc,
                   void* out, int cols, cudaStream_t stream);
int olb_ep_pull_dweights(const void* const* peer_dw, int n, const int* idx, int my_rank, int T, int K, int E_loc,
                         float* dw, cudaStream_t stream);
// out[r,:] = sum_p peer_partial[p][row0 + r, :] (row stride ld), bf16 in/out, fp32 accumulation.
int olb_pull_reduce_rows(const void* const* peer_partial, int n, long long row0, int rows, int cols, long long ld,
                         void* out, cudaStream_t stream);
// Gradient reduce-scatter + AdamW + parameter all-gather on the shard [shard_off, shard_off+n_elems) of the
// ranks' flat bf16 gradient / parameter buffers.  mode 0: norm partials only; mode 1: update as well.
// norm_partial: olb_rs_adamw_blocks(n_elems) floats (sum of squares of the reduced, scaled gradient).
int olb_rs_adamw(const void* const* peer_grad, void* const* peer_param, int n, long long shard_off, long long n_elems,
                 float* master, float* m, float* v, const olb_adamw_hparams* hp, const float* clip_coef_dev,
                 float* norm_partial, int mode, cudaStream_t stream);
int olb_rs_adamw_blocks(long long n_elems);
// The same with NVLS: mc_grad / mc_param are the multicast addresses of the flat gradient / parameter buffers (both or
// neither; NULL = plain peer loads and stores).  The reduced gradient is rounded to bf16 once, as after a bf16
// reduce-scatter.
int olb_rs_adamw_mc(const void* const* peer_grad, void* const* peer_param, int n, long long shard_off, long long n_elems,
                    float* master, float* m, float* v, const olb_adamw_hparams* hp, const float* clip_coef_dev,
                    float* norm_partial, int mode, const void* mc_grad, void* mc_param, cudaStream_t stream);
// The same with ranges of the flat buffer whose updated parameters stay on this GPU (`local_only`: device array of
// n_local_only sorted, disjoint [start, end) pairs in elements of the flat buffer): their all-gather is left to the first
// GEMM that consumes the weight (olb_gemm_desc.B_peers).  my_rank = this GPU's index in peer_param.
int olb_rs_adamw_ex(const void* const* peer_grad, void* const* peer_param, int n, long long shard_off, long long n_elems,
                    float* master, float* m, float* v, const olb_adamw_hparams* hp, const float* clip_coef_dev,
                    float* norm_partial, int mode, const void* mc_grad, void* mc_param, const long long* local_only,
                    int n_local_only, int my_rank, cudaStream_t stream);
// dst <- src, `bytes` a multiple of 16; src may point into another GPU's memory.
int olb_peer_copy(const void* src, void* dst, long long bytes, cudaStream_t stream);

// ---------------------------------------------------------------- attention (attention.cu)
// Causal flash attention forward, bf16, q/k/v as [B, S, H, D] with arbitrary token/head strides
// (elements); o [B, S, Hq, Dv]; lse [B, Hq, S] fp32.  D in {64, 128, 192}, Dv in {64, 128}.
typedef struct {
  const void *q, *k, *v;
  void* o;
  float* lse;
  long long q_bs, q_ss, q_hs;  // batch / seq / head strides
  long long k_bs, k_ss, k_hs;
  long long v_bs, v_ss, v_hs;
  long long o_bs, o_ss, o_hs;
  int B, S, Hq, Hkv, D, Dv;
  float scale;
  int* status;
  int variant;  // 0: the kernel the library prefers for the shape; 1: one query tile per CTA; 2: two (S % 256 == 0)
} olb_attn_fwd_desc;
int olb_attn_fwd(const olb_attn_fwd_desc* d, cudaStream_t stream);

typedef struct {
  const void *q, *k, *v, *o, *dout;
  const float* lse;
  void *dq, *dk, *dv;   // bf16, same layouts as q/k/v
  float* dq_acc;        // fp32 scratch [B, S, Hq, D]
  float* delta;         // fp32 scratch [B, Hq, S]
  long long q_bs, q_ss, q_hs, k_bs, k_ss, k_hs, v_bs, v_ss, v_hs, o_bs, o_ss, o_hs;
  long long dq_bs, dq_ss, dq_hs, dk_bs, dk_ss, dk_hs, dv_bs, dv_ss, dv_hs, do_bs, do_ss, do_hs;
  int B, S, Hq, Hkv, D, Dv;
  float scale;
  int* status;
} olb_attn_bwd_desc;
int olb_attn_bwd(const olb_attn_bwd_desc* d, cudaStream_t stream);

// ---------------------------------------------------------------- embedding (embedding.cu)
// out[t,:] = W[ids[t] - v_start,:] for ids inside [v_start, v_start + rows), else 0.  bf16, cols % 8 == 0.
int olb_embedding_fwd(const long long* ids, const void* w, void* out, int tokens, int cols, int v_start, int rows,
                      cudaStream_t stream);
// dW[v,:] (+)= sum of dy[perm[j],:] over the run of sorted_ids equal to v (ids sorted stably, perm = source token).
// Rows of dW that no token hits are left untouched.  padding_idx (or -1): that id gets no gradient.
int olb_embedding_bwd(const long long* sorted_ids, const long long* perm, const void* dy, void* dw, int tokens, int cols,
                      int v_start, int rows, long long padding_idx, int accumulate, cudaStream_t stream);

// ---------------------------------------------------------------- timing (event_profiler.cu)
// Writes %globaltimer (ns) of the moment the kernel runs on `stream` into slot[0].
int olb_stamp_globaltimer(unsigned long long* slot, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
