// Python bindings (module optimus_lm_b200._C): thin tensor -> pointer adapters over the C entry
// points of olb_api.h.  All kernels run on the current CUDA stream of the tensors' device.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "olb_api.h"

namespace {

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

inline void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, what, " failed with code ", rc);
}

#define CHECK_CUDA_BF16(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kBFloat16, #t " must be a CUDA bf16 tensor")
#define CHECK_CUDA_F32(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kFloat, #t " must be a CUDA fp32 tensor")
#define CHECK_CUDA_I32(t) TORCH_CHECK((t).is_cuda() && (t).scalar_type() == at::kInt, #t " must be a CUDA int32 tensor")

template <typename T>
T* opt_ptr(const c10::optional<at::Tensor>& t) {
  return t.has_value() && t->defined() ? static_cast<T*>(t->data_ptr()) : nullptr;
}

// Generic GEMM.  a: 2D bf16 view whose last dim is contiguous; b likewise.
//   a_mn_major == 0: a is [rows, K];  == 1: a is [K, M]      (same for b with N)
void gemm(const at::Tensor& a, const at::Tensor& b, at::Tensor& c, int64_t M, int64_t N, int64_t K, bool a_mn_major,
          bool b_mn_major, bool accumulate, int64_t mode, const c10::optional<at::Tensor>& meta, int64_t num_experts,
          int64_t b_expert_rows, int64_t c_expert_stride, const c10::optional<at::Tensor>& status, int64_t block_n,
          int64_t max_ctas, const c10::optional<at::Tensor>& b2, int64_t k_split,
          const c10::optional<at::Tensor>& blk_range, bool pair_rows) {
  CHECK_CUDA_BF16(a);
  CHECK_CUDA_BF16(b);
  TORCH_CHECK(c.is_cuda() && (c.scalar_type() == at::kBFloat16 || c.scalar_type() == at::kFloat), "c must be bf16/fp32");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1, "a/b must be 2D with unit inner stride");
  TORCH_CHECK(c.stride(-1) == 1, "c must have unit inner stride");
  c10::cuda::CUDAGuard guard(a.device());
  olb_gemm_desc d{};
  d.A = a.data_ptr();
  d.B = b.data_ptr();
  d.C = c.data_ptr();
  d.lda = a.stride(0);
  d.ldb = b.stride(0);
  d.ldc = c.dim() >= 2 ? c.stride(-2) : N;
  d.a_rows = a.size(0);
  d.b_rows = b.size(0);
  d.M = static_cast<int>(M);
  d.N = static_cast<int>(N);
  d.K = static_cast<int>(K);
  d.a_mn_major = a_mn_major;
  d.b_mn_major = b_mn_major;
  d.mode = static_cast<int>(mode);
  d.meta = opt_ptr<const int>(meta);
  d.num_experts = static_cast<int>(num_experts);
  d.b_expert_rows = static_cast<int>(b_expert_rows);
  d.c_expert_stride = c_expert_stride;
  d.accumulate = accumulate;
  d.out_fp32 = c.scalar_type() == at::kFloat;
  d.block_n = static_cast<int>(block_n);
  d.max_ctas = static_cast<int>(max_ctas);
  d.status = opt_ptr<int>(status);
  if (b2.has_value()) {
    TORCH_CHECK(b2->is_cuda() && b2->scalar_type() == at::kBFloat16 && b2->sizes() == b.sizes() && b2->strides() == b.strides(),
                "b2 must have the layout of b");
    d.B2 = b2->data_ptr();
    d.k_split = static_cast<int>(k_split);
  }
  d.blk_range = opt_ptr<const int>(blk_range);
  d.pair_rows = pair_rows;
  check(olb_gemm_bf16(&d, cur_stream()), "olb_gemm_bf16");
}

void embedding_fwd(const at::Tensor& ids, const at::Tensor& w, at::Tensor& out, int64_t v_start) {
  CHECK_CUDA_BF16(w);
  TORCH_CHECK(ids.scalar_type() == at::kLong && ids.is_contiguous() && w.is_contiguous() && out.is_contiguous());
  c10::cuda::CUDAGuard guard(w.device());
  check(olb_embedding_fwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()), w.data_ptr(), out.data_ptr(),
                          static_cast<int>(ids.numel()), static_cast<int>(w.size(1)), static_cast<int>(v_start),
                          static_cast<int>(w.size(0)), cur_stream()),
        "olb_embedding_fwd");
}

void embedding_bwd(const at::Tensor& sorted_ids, const at::Tensor& perm, const at::Tensor& dy, at::Tensor& dw,
                   int64_t v_start, int64_t padding_idx, bool accumulate) {
  CHECK_CUDA_BF16(dy);
  TORCH_CHECK(sorted_ids.scalar_type() == at::kLong && perm.scalar_type() == at::kLong && dy.is_contiguous() &&
              dw.is_contiguous() && dw.scalar_type() == at::kBFloat16);
  c10::cuda::CUDAGuard guard(dy.device());
  check(olb_embedding_bwd(reinterpret_cast<const long long*>(sorted_ids.data_ptr<int64_t>()),
                          reinterpret_cast<const long long*>(perm.data_ptr<int64_t>()), dy.data_ptr(), dw.data_ptr(),
                          static_cast<int>(sorted_ids.numel()), static_cast<int>(dw.size(1)), static_cast<int>(v_start),
                          static_cast<int>(dw.size(0)), padding_idx, accumulate, cur_stream()),
        "olb_embedding_bwd");
}

void rmsnorm_fwd(const at::Tensor& x, const c10::optional<at::Tensor>& w, at::Tensor& y, at::Tensor& rstd, double eps) {
  CHECK_CUDA_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = x.size(-1);
  const int rows = x.numel() / cols;
  check(olb_rmsnorm_fwd(x.data_ptr(), opt_ptr<const void>(w), y.data_ptr(), rstd.data_ptr<float>(), rows, cols,
                        static_cast<float>(eps), cur_stream()),
        "olb_rmsnorm_fwd");
}

int64_t rmsnorm_bwd_blocks(int64_t rows) { return olb_rmsnorm_bwd_blocks(static_cast<int>(rows)); }

void rmsnorm_bwd(const at::Tensor& dy, const at::Tensor& x, const c10::optional<at::Tensor>& w, const at::Tensor& rstd,
                 at::Tensor& dx, const c10::optional<at::Tensor>& dw_partial, const c10::optional<at::Tensor>& dres) {
  CHECK_CUDA_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = x.size(-1);
  const int rows = x.numel() / cols;
  if (dres.has_value()) TORCH_CHECK(dres->scalar_type() == at::kBFloat16 && dres->is_contiguous() && dres->numel() == x.numel());
  check(olb_rmsnorm_bwd_res(dy.data_ptr(), x.data_ptr(), opt_ptr<const void>(w), rstd.data_ptr<float>(), dx.data_ptr(),
                            opt_ptr<float>(dw_partial), opt_ptr<const void>(dres), rows, cols, cur_stream()),
        "olb_rmsnorm_bwd");
}

void add_rmsnorm_fwd(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& w, at::Tensor& h,
                     at::Tensor& y, at::Tensor& rstd, double eps) {
  CHECK_CUDA_BF16(a);
  CHECK_CUDA_BF16(b);
  TORCH_CHECK(a.is_contiguous() && b.is_contiguous() && h.is_contiguous() && y.is_contiguous() && a.numel() == b.numel());
  c10::cuda::CUDAGuard guard(a.device());
  const int cols = a.size(-1);
  const int rows = a.numel() / cols;
  check(olb_add_rmsnorm_fwd(a.data_ptr(), b.data_ptr(), opt_ptr<const void>(w), h.data_ptr(), y.data_ptr(),
                            rstd.data_ptr<float>(), rows, cols, static_cast<float>(eps), cur_stream()),
        "olb_add_rmsnorm_fwd");
}

void colsum_finalize(const at::Tensor& partial, int64_t nparts, at::Tensor& dw, bool accumulate) {
  CHECK_CUDA_F32(partial);
  c10::cuda::CUDAGuard guard(partial.device());
  check(olb_colsum_finalize(partial.data_ptr<float>(), static_cast<int>(nparts), static_cast<int>(dw.numel()),
                            dw.data_ptr(), dw.scalar_type() == at::kFloat, accumulate, cur_stream()),
        "olb_colsum_finalize");
}

void layernorm_fwd(const at::Tensor& x, at::Tensor& y, at::Tensor& mean, at::Tensor& rstd, double eps) {
  CHECK_CUDA_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = x.size(-1);
  const int rows = x.numel() / cols;
  check(olb_layernorm_fwd(x.data_ptr(), y.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), rows, cols,
                          static_cast<float>(eps), cur_stream()),
        "olb_layernorm_fwd");
}

void layernorm_bwd(const at::Tensor& dy, const at::Tensor& x, const at::Tensor& mean, const at::Tensor& rstd,
                   at::Tensor& dx) {
  CHECK_CUDA_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  const int cols = x.size(-1);
  const int rows = x.numel() / cols;
  check(olb_layernorm_bwd(dy.data_ptr(), x.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), dx.data_ptr(),
                          rows, cols, cur_stream()),
        "olb_layernorm_bwd");
}

// g, u, act: 2D bf16 views with unit inner stride.
void swiglu_fwd(const at::Tensor& g, const at::Tensor& u, at::Tensor& act) {
  CHECK_CUDA_BF16(g);
  c10::cuda::CUDAGuard guard(g.device());
  check(olb_swiglu_fwd(g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0), act.data_ptr(), act.stride(0), g.size(0),
                       static_cast<int>(g.size(1)), cur_stream()),
        "olb_swiglu_fwd");
}

void swiglu_bwd(const at::Tensor& dact, const at::Tensor& g, const at::Tensor& u, at::Tensor& dg, at::Tensor& du) {
  CHECK_CUDA_BF16(g);
  c10::cuda::CUDAGuard guard(g.device());
  check(olb_swiglu_bwd(dact.data_ptr(), dact.stride(0), g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0),
                       dg.data_ptr(), dg.stride(0), du.data_ptr(), du.stride(0), g.size(0), static_cast<int>(g.size(1)),
                       cur_stream()),
        "olb_swiglu_bwd");
}

void swiglu_rowscale_fwd(const at::Tensor& g, const at::Tensor& u, const at::Tensor& src_of, const at::Tensor& k_of,
                         const at::Tensor& weights, const at::Tensor& meta, at::Tensor& act) {
  CHECK_CUDA_BF16(g);
  CHECK_CUDA_F32(weights);
  c10::cuda::CUDAGuard guard(g.device());
  check(olb_swiglu_rowscale_fwd(g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0), src_of.data_ptr<int>(),
                                k_of.data_ptr<int>(), weights.data_ptr<float>(), static_cast<int>(weights.size(1)),
                                meta.data_ptr<int>(), act.data_ptr(), act.stride(0), static_cast<int>(g.size(0)),
                                static_cast<int>(g.size(1)), cur_stream()),
        "olb_swiglu_rowscale_fwd");
}

void swiglu_rowscale_bwd(const at::Tensor& dact, const at::Tensor& g, const at::Tensor& u, const at::Tensor& src_of,
                         const at::Tensor& k_of, const at::Tensor& weights, const at::Tensor& meta, at::Tensor& dg,
                         at::Tensor& du, const c10::optional<at::Tensor>& dweights) {
  CHECK_CUDA_BF16(g);
  CHECK_CUDA_F32(weights);
  c10::cuda::CUDAGuard guard(g.device());
  check(olb_swiglu_rowscale_bwd(dact.data_ptr(), dact.stride(0), g.data_ptr(), g.stride(0), u.data_ptr(), u.stride(0),
                                src_of.data_ptr<int>(), k_of.data_ptr<int>(), weights.data_ptr<float>(),
                                static_cast<int>(weights.size(1)), meta.data_ptr<int>(), dg.data_ptr(), dg.stride(0),
                                du.data_ptr(), du.stride(0), opt_ptr<float>(dweights), static_cast<int>(g.size(0)),
                                static_cast<int>(g.size(1)), cur_stream()),
        "olb_swiglu_rowscale_bwd");
}

// x: [tokens, heads, head_stride-ish] view: pointer to the first rotated element, explicit strides.
void rope_inplace(at::Tensor& x, int64_t token_stride, int64_t tokens, int64_t heads, int64_t head_stride,
                  int64_t rot_dim, int64_t seq_len, const at::Tensor& cos_tab, const at::Tensor& sin_tab,
                  bool interleaved, bool conj) {
  CHECK_CUDA_BF16(x);
  CHECK_CUDA_F32(cos_tab);
  c10::cuda::CUDAGuard guard(x.device());
  check(olb_rope_inplace(x.data_ptr(), token_stride, static_cast<int>(tokens), static_cast<int>(heads),
                         static_cast<int>(head_stride), static_cast<int>(rot_dim), static_cast<int>(seq_len),
                         cos_tab.data_ptr<float>(), sin_tab.data_ptr<float>(), interleaved, conj, cur_stream()),
        "olb_rope_inplace");
}

int64_t router_blocks(int64_t T) { return olb_router_blocks(static_cast<int>(T)); }

void router_softmax_topk(const at::Tensor& logits, int64_t K, bool renorm, at::Tensor& weights, at::Tensor& indices,
                         const c10::optional<at::Tensor>& cnt_partial, const c10::optional<at::Tensor>& prob_partial,
                         const c10::optional<at::Tensor>& lse_sq_partial) {
  CHECK_CUDA_BF16(logits);
  CHECK_CUDA_F32(weights);
  CHECK_CUDA_I32(indices);
  c10::cuda::CUDAGuard guard(logits.device());
  check(olb_router_softmax_topk(logits.data_ptr(), static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                                static_cast<int>(K), renorm, weights.data_ptr<float>(), indices.data_ptr<int>(),
                                opt_ptr<float>(cnt_partial), opt_ptr<float>(prob_partial),
                                opt_ptr<float>(lse_sq_partial), cur_stream()),
        "olb_router_softmax_topk");
}

void router_bwd(const at::Tensor& logits, const at::Tensor& indices, const c10::optional<at::Tensor>& dweights,
                bool renorm, const c10::optional<at::Tensor>& aux_f, const c10::optional<at::Tensor>& aux_scale_dev,
                double aux_scale, double z_scale, at::Tensor& dlogits) {
  CHECK_CUDA_BF16(logits);
  c10::cuda::CUDAGuard guard(logits.device());
  check(olb_router_bwd_ex(logits.data_ptr(), indices.data_ptr<int>(), opt_ptr<const float>(dweights),
                          static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                          static_cast<int>(indices.size(1)), renorm, opt_ptr<const float>(aux_f),
                          opt_ptr<const float>(aux_scale_dev), static_cast<float>(aux_scale),
                          static_cast<float>(z_scale), dlogits.data_ptr(), cur_stream()),
        "olb_router_bwd");
}

void router_sigmoid_group_topk(const at::Tensor& logits, const c10::optional<at::Tensor>& bias, int64_t K,
                               int64_t n_group, int64_t topk_group, bool renorm, double scale, at::Tensor& weights,
                               at::Tensor& indices) {
  CHECK_CUDA_F32(logits);
  c10::cuda::CUDAGuard guard(logits.device());
  check(olb_router_sigmoid_group_topk(logits.data_ptr<float>(), opt_ptr<const float>(bias),
                                      static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                                      static_cast<int>(K), static_cast<int>(n_group), static_cast<int>(topk_group),
                                      renorm, static_cast<float>(scale), weights.data_ptr<float>(),
                                      indices.data_ptr<int>(), cur_stream()),
        "olb_router_sigmoid_group_topk");
}

void router_sigmoid_bwd(const at::Tensor& logits, const at::Tensor& indices, const at::Tensor& dweights, bool renorm,
                        double scale, at::Tensor& dlogits) {
  CHECK_CUDA_F32(logits);
  c10::cuda::CUDAGuard guard(logits.device());
  check(olb_router_sigmoid_bwd(logits.data_ptr<float>(), indices.data_ptr<int>(), dweights.data_ptr<float>(),
                               static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                               static_cast<int>(indices.size(1)), renorm, static_cast<float>(scale),
                               dlogits.data_ptr<float>(), cur_stream()),
        "olb_router_sigmoid_bwd");
}

int64_t moe_ws_ints(int64_t T, int64_t E_loc) { return olb_moe_ws_ints(static_cast<int>(T), static_cast<int>(E_loc)); }

void moe_build_index(const at::Tensor& indices, int64_t e_start, int64_t E_loc, int64_t cap, at::Tensor& ws,
                     at::Tensor& row_of, at::Tensor& src_of, at::Tensor& k_of, at::Tensor& meta, at::Tensor& offsets,
                     at::Tensor& counts, const c10::optional<at::Tensor>& status, int64_t row_pad) {
  CHECK_CUDA_I32(indices);
  c10::cuda::CUDAGuard guard(indices.device());
  TORCH_CHECK(ws.numel() >= olb_moe_ws_ints(indices.size(0), E_loc), "workspace too small");
  TORCH_CHECK(meta.numel() >= 1 + cap / 128 && src_of.numel() >= cap && k_of.numel() >= cap, "index buffers too small");
  check(olb_moe_build_index(indices.data_ptr<int>(), static_cast<int>(indices.size(0)),
                            static_cast<int>(indices.size(1)), static_cast<int>(e_start), static_cast<int>(E_loc),
                            static_cast<int>(cap), static_cast<int>(row_pad), ws.data_ptr<int>(), row_of.data_ptr<int>(),
                            src_of.data_ptr<int>(),
                            k_of.data_ptr<int>(), meta.data_ptr<int>(), offsets.data_ptr<int>(), counts.data_ptr<int>(),
                            opt_ptr<int>(status), cur_stream()),
        "olb_moe_build_index");
}

void moe_scatter_dweights(const at::Tensor& partial, const at::Tensor& src_of, const at::Tensor& k_of, const at::Tensor& meta,
                          at::Tensor& out) {
  CHECK_CUDA_F32(partial);
  CHECK_CUDA_F32(out);
  TORCH_CHECK(partial.dim() == 2 && partial.is_contiguous() && out.dim() == 2 && out.is_contiguous());
  c10::cuda::CUDAGuard guard(partial.device());
  check(olb_moe_scatter_dweights(partial.data_ptr<float>(), static_cast<int>(partial.size(1)), src_of.data_ptr<int>(),
                                 k_of.data_ptr<int>(), meta.data_ptr<int>(), static_cast<int>(out.size(1)),
                                 out.data_ptr<float>(), static_cast<int>(partial.size(0)), cur_stream()),
        "olb_moe_scatter_dweights");
}

void moe_gather_rows(const at::Tensor& x, const at::Tensor& src_of, const at::Tensor& meta, at::Tensor& out) {
  CHECK_CUDA_BF16(x);
  c10::cuda::CUDAGuard guard(x.device());
  check(olb_moe_gather_rows(x.data_ptr(), src_of.data_ptr<int>(), meta.data_ptr<int>(), out.data_ptr(),
                            static_cast<int>(out.size(0)), static_cast<int>(out.size(1)), cur_stream()),
        "olb_moe_gather_rows");
}

void moe_combine(const at::Tensor& y, const at::Tensor& row_of, const c10::optional<at::Tensor>& w, at::Tensor& out) {
  CHECK_CUDA_BF16(y);
  c10::cuda::CUDAGuard guard(y.device());
  check(olb_moe_combine(y.data_ptr(), row_of.data_ptr<int>(), opt_ptr<const float>(w), out.data_ptr(),
                        static_cast<int>(row_of.size(0)), static_cast<int>(row_of.size(1)),
                        static_cast<int>(out.size(1)), cur_stream()),
        "olb_moe_combine");
}

void moe_combine_bwd(const at::Tensor& dout, const c10::optional<at::Tensor>& y, const at::Tensor& src_of,
                     const at::Tensor& k_of, const at::Tensor& meta, const c10::optional<at::Tensor>& w, at::Tensor& dy,
                     const c10::optional<at::Tensor>& dw, int64_t K) {
  CHECK_CUDA_BF16(dout);
  c10::cuda::CUDAGuard guard(dout.device());
  check(olb_moe_combine_bwd(dout.data_ptr(), opt_ptr<const void>(y), src_of.data_ptr<int>(), k_of.data_ptr<int>(),
                            meta.data_ptr<int>(), opt_ptr<const float>(w), dy.data_ptr(), opt_ptr<float>(dw),
                            static_cast<int>(dy.size(0)), static_cast<int>(K), static_cast<int>(dy.size(1)),
                            cur_stream()),
        "olb_moe_combine_bwd");
}

void ce_fwd(const at::Tensor& logits, const at::Tensor& labels, at::Tensor& loss_row, at::Tensor& lse) {
  CHECK_CUDA_BF16(logits);
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_cuda());
  c10::cuda::CUDAGuard guard(logits.device());
  check(olb_ce_fwd(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), loss_row.data_ptr<float>(),
                   lse.data_ptr<float>(), static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                   cur_stream()),
        "olb_ce_fwd");
}

void ce_bwd(const at::Tensor& logits, const at::Tensor& labels, const at::Tensor& lse, const at::Tensor& scale_dev,
            at::Tensor& dlogits) {
  CHECK_CUDA_BF16(logits);
  CHECK_CUDA_F32(scale_dev);
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(dlogits.stride(0) == logits.stride(0));
  check(olb_ce_bwd(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), lse.data_ptr<float>(),
                   scale_dev.data_ptr<float>(), dlogits.data_ptr(), static_cast<int>(logits.size(0)),
                   static_cast<int>(logits.size(1)), cur_stream()),
        "olb_ce_bwd");
}

void ce_partial_fwd(const at::Tensor& logits, const at::Tensor& labels, int64_t v_start, at::Tensor& part_max,
                    at::Tensor& part_sum, at::Tensor& part_tgt) {
  CHECK_CUDA_BF16(logits);
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_cuda());
  CHECK_CUDA_F32(part_max);
  CHECK_CUDA_F32(part_sum);
  CHECK_CUDA_F32(part_tgt);
  c10::cuda::CUDAGuard guard(logits.device());
  check(olb_ce_partial_fwd(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                           static_cast<int>(v_start), part_max.data_ptr<float>(), part_sum.data_ptr<float>(),
                           part_tgt.data_ptr<float>(), static_cast<int>(logits.size(0)), static_cast<int>(logits.size(1)),
                           cur_stream()),
        "olb_ce_partial_fwd");
}

void ce_partial_bwd(const at::Tensor& logits, const at::Tensor& labels, int64_t v_start, int64_t v_total,
                    const at::Tensor& lse, const at::Tensor& scale_dev, at::Tensor& dlogits) {
  CHECK_CUDA_BF16(logits);
  CHECK_CUDA_F32(scale_dev);
  CHECK_CUDA_F32(lse);
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(dlogits.stride(0) == logits.stride(0));
  check(olb_ce_partial_bwd(logits.data_ptr(), logits.stride(0), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                           static_cast<int>(v_start), static_cast<int>(v_total), lse.data_ptr<float>(),
                           scale_dev.data_ptr<float>(), dlogits.data_ptr(), static_cast<int>(logits.size(0)),
                           static_cast<int>(logits.size(1)), cur_stream()),
        "olb_ce_partial_bwd");
}

int64_t sumsq_blocks(int64_t n) { return olb_sumsq_blocks(n); }

// out[0] (+)= sum((grad*scale)^2); `partial` is scratch of at least sumsq_blocks(n) floats.
void sumsq(const at::Tensor& grad, double grad_scale, at::Tensor& partial, at::Tensor& out, bool accumulate) {
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous());
  c10::cuda::CUDAGuard guard(grad.device());
  const int64_t n = grad.numel();
  const int nb = olb_sumsq_blocks(n);
  TORCH_CHECK(partial.numel() >= nb, "partial buffer too small");
  check(olb_sumsq_partial(grad.data_ptr(), grad.scalar_type() == at::kFloat, n, static_cast<float>(grad_scale),
                          partial.data_ptr<float>(), cur_stream()),
        "olb_sumsq_partial");
  check(olb_sum_finalize(partial.data_ptr<float>(), nb, out.data_ptr<float>(), accumulate, cur_stream()),
        "olb_sum_finalize");
}

void adamw_step(const at::Tensor& grad, at::Tensor& master, at::Tensor& m, at::Tensor& v, at::Tensor& param, double lr,
                double beta1, double beta2, double eps, double weight_decay, int64_t step, double grad_scale,
                const c10::optional<at::Tensor>& clip_coef, bool skip_weight_update,
                const c10::optional<at::Tensor>& norm_out) {
  CHECK_CUDA_F32(master);
  c10::cuda::CUDAGuard guard(master.device());
  // norm_out (optional, 1 fp32 element): += sum((grad * grad_scale)^2), a by-product of the update's pass
  at::Tensor partial;
  const int nb = olb_adamw_blocks(master.numel());
  if (norm_out.has_value()) {
    CHECK_CUDA_F32(*norm_out);
    partial = at::empty({nb}, master.options());
  }
  olb_adamw_hparams hp;
  hp.lr = static_cast<float>(lr);
  hp.beta1 = static_cast<float>(beta1);
  hp.beta2 = static_cast<float>(beta2);
  hp.eps = static_cast<float>(eps);
  hp.weight_decay = static_cast<float>(weight_decay);
  hp.bias_correction1 = static_cast<float>(1.0 - std::pow(beta1, static_cast<double>(step)));
  hp.bias_correction2 = static_cast<float>(1.0 - std::pow(beta2, static_cast<double>(step)));
  hp.grad_scale = static_cast<float>(grad_scale);
  hp.skip_weight_update = skip_weight_update;
  check(olb_adamw_step(grad.data_ptr(), grad.scalar_type() == at::kFloat, master.data_ptr<float>(), m.data_ptr<float>(),
                       v.data_ptr<float>(), param.data_ptr(), param.scalar_type() == at::kFloat, master.numel(), &hp,
                       opt_ptr<const float>(clip_coef), norm_out.has_value() ? partial.data_ptr<float>() : nullptr,
                       cur_stream()),
        "olb_adamw_step");
  if (norm_out.has_value() && master.numel() > 0)
    check(olb_sum_finalize(partial.data_ptr<float>(), nb, norm_out->data_ptr<float>(), 1, cur_stream()), "olb_sum_finalize");
}

void stamp_globaltimer(at::Tensor& slot) {
  // slot: int64 tensor in pinned host memory (device-mapped) or device memory
  check(olb_stamp_globaltimer(reinterpret_cast<unsigned long long*>(slot.data_ptr()), cur_stream()),
        "olb_stamp_globaltimer");
}

}  // namespace

void register_attention(pybind11::module& m);
void register_comm(pybind11::module& m);
void register_customops(pybind11::module& m);

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm, pybind11::arg("a"), pybind11::arg("b"), pybind11::arg("c"), pybind11::arg("M"), pybind11::arg("N"),
        pybind11::arg("K"), pybind11::arg("a_mn_major"), pybind11::arg("b_mn_major"), pybind11::arg("accumulate"),
        pybind11::arg("mode"), pybind11::arg("meta"), pybind11::arg("num_experts"), pybind11::arg("b_expert_rows"),
        pybind11::arg("c_expert_stride"), pybind11::arg("status"), pybind11::arg("block_n"), pybind11::arg("max_ctas"),
        pybind11::arg("b2"), pybind11::arg("k_split"), pybind11::arg("blk_range"), pybind11::arg("pair_rows") = false);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, pybind11::arg("dy"), pybind11::arg("x"), pybind11::arg("w"), pybind11::arg("rstd"),
        pybind11::arg("dx"), pybind11::arg("dw_partial"), pybind11::arg("dres") = pybind11::none());
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("rmsnorm_bwd_blocks", &rmsnorm_bwd_blocks);
  m.def("colsum_finalize", &colsum_finalize);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("swiglu_rowscale_fwd", &swiglu_rowscale_fwd);
  m.def("swiglu_rowscale_bwd", &swiglu_rowscale_bwd);
  m.def("rope_inplace", &rope_inplace);
  m.def("router_blocks", &router_blocks);
  m.def("router_softmax_topk", &router_softmax_topk);
  m.def("router_bwd", &router_bwd);
  m.def("router_sigmoid_group_topk", &router_sigmoid_group_topk);
  m.def("router_sigmoid_bwd", &router_sigmoid_bwd);
  m.def("moe_ws_ints", &moe_ws_ints);
  m.def("moe_build_index", &moe_build_index, pybind11::arg("indices"), pybind11::arg("e_start"), pybind11::arg("E_loc"),
        pybind11::arg("cap"), pybind11::arg("ws"), pybind11::arg("row_of"), pybind11::arg("src_of"), pybind11::arg("k_of"),
        pybind11::arg("meta"), pybind11::arg("offsets"), pybind11::arg("counts"), pybind11::arg("status"),
        pybind11::arg("row_pad") = 128);
  m.def("moe_scatter_dweights", &moe_scatter_dweights);
  m.def("moe_gather_rows", &moe_gather_rows);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_bwd", &moe_combine_bwd);
  m.def("ce_fwd", &ce_fwd);
  m.def("ce_bwd", &ce_bwd);
  m.def("ce_partial_fwd", &ce_partial_fwd);
  m.def("ce_partial_bwd", &ce_partial_bwd);
  m.def("sumsq_blocks", &sumsq_blocks);
  m.def("sumsq", &sumsq);
  m.def("adamw_step", &adamw_step);
  m.def("stamp_globaltimer", &stamp_globaltimer);
  register_attention(m);
  register_comm(m);
  register_customops(m);
}
