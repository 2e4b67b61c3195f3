// Python bindings for the peer-memory kernels (comm_p2p.cu).  Peer pointers arrive as Python
// lists of integers (addresses inside other GPUs' symmetric buffers).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "olb_api.h"

namespace {

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void check(int rc, const char* what) { TORCH_CHECK(rc == 0, what, " failed with code ", rc); }

std::vector<const void*> cptrs(const std::vector<int64_t>& v) {
  std::vector<const void*> out;
  for (auto p : v) out.push_back(reinterpret_cast<const void*>(static_cast<uintptr_t>(p)));
  return out;
}
std::vector<void*> mptrs(const std::vector<int64_t>& v) {
  std::vector<void*> out;
  for (auto p : v) out.push_back(reinterpret_cast<void*>(static_cast<uintptr_t>(p)));
  return out;
}

void symm_barrier(const std::vector<int64_t>& pads, int64_t my_rank, int64_t channel, int64_t epoch,
                  const c10::optional<at::Tensor>& status, int64_t wait_limit_ns) {
  auto p = mptrs(pads);
  check(olb_symm_barrier(p.data(), static_cast<int>(my_rank), static_cast<int>(p.size()), static_cast<int>(channel),
                         static_cast<unsigned>(epoch), status.has_value() ? status->data_ptr<int>() : nullptr,
                         static_cast<unsigned long long>(wait_limit_ns), cur_stream()),
        "olb_symm_barrier");
}

void ep_publish_meta(const std::vector<int64_t>& idx_all, const std::vector<int64_t>& w_all, const at::Tensor& idx,
                     const at::Tensor& w, int64_t off) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kInt && w.scalar_type() == at::kFloat && idx.is_contiguous() &&
              w.is_contiguous() && idx.numel() == w.numel() && idx_all.size() == w_all.size());
  c10::cuda::CUDAGuard guard(idx.device());
  auto pi = mptrs(idx_all);
  auto pw = mptrs(w_all);
  check(olb_ep_publish_meta(pi.data(), pw.data(), static_cast<int>(pi.size()), idx.data_ptr<int>(), w.data_ptr<float>(),
                            off, idx.numel(), cur_stream()),
        "olb_ep_publish_meta");
}

void sum_slots(const at::Tensor& recv, at::Tensor& out) {
  TORCH_CHECK(recv.is_cuda() && recv.scalar_type() == at::kBFloat16 && recv.dim() == 3 && recv.is_contiguous() &&
              out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.size(0) == recv.size(0) &&
              out.size(1) == recv.size(2));
  c10::cuda::CUDAGuard guard(recv.device());
  check(olb_sum_slots(recv.data_ptr(), static_cast<int>(recv.size(0)), static_cast<int>(recv.size(1)),
                      static_cast<int>(recv.size(2)), out.data_ptr(), cur_stream()),
        "olb_sum_slots");
}

void ep_gather_rows(const std::vector<int64_t>& peer_x, int64_t T, const at::Tensor& src_of, const at::Tensor& meta,
                    at::Tensor& out, const c10::optional<at::Tensor>& blk_range) {
  c10::cuda::CUDAGuard guard(out.device());
  auto p = cptrs(peer_x);
  check(olb_ep_gather_rows(p.data(), static_cast<int>(p.size()), static_cast<int>(T), src_of.data_ptr<int>(),
                           meta.data_ptr<int>(), blk_range.has_value() ? blk_range->data_ptr<int>() : nullptr,
                           out.data_ptr(), static_cast<int>(out.size(0)),
                           static_cast<int>(out.size(1)), cur_stream()),
        "olb_ep_gather_rows");
}

void ep_resolve_rows(const std::vector<int64_t>& peer_row_of, const at::Tensor& idx, int64_t my_rank, int64_t E_loc,
                     at::Tensor& rows) {
  c10::cuda::CUDAGuard guard(rows.device());
  auto p = cptrs(peer_row_of);
  check(olb_ep_resolve_rows(p.data(), static_cast<int>(p.size()), idx.data_ptr<int>(), static_cast<int>(my_rank),
                            static_cast<int>(idx.size(0)), static_cast<int>(idx.size(1)), static_cast<int>(E_loc),
                            rows.data_ptr<int>(), cur_stream()),
        "olb_ep_resolve_rows");
}

void ep_combine(const std::vector<int64_t>& peer_y, const at::Tensor& rows, const at::Tensor& idx, int64_t E_loc,
                at::Tensor& out) {
  c10::cuda::CUDAGuard guard(out.device());
  auto py = cptrs(peer_y);
  check(olb_ep_combine(py.data(), static_cast<int>(py.size()), rows.data_ptr<int>(), idx.data_ptr<int>(),
                       static_cast<int>(idx.size(0)), static_cast<int>(idx.size(1)), static_cast<int>(E_loc),
                       out.data_ptr(), static_cast<int>(out.size(1)), cur_stream()),
        "olb_ep_combine");
}

void ep_pull_dweights(const std::vector<int64_t>& peer_dw, const at::Tensor& idx, int64_t my_rank, int64_t E_loc,
                      at::Tensor& dw) {
  c10::cuda::CUDAGuard guard(dw.device());
  auto p = cptrs(peer_dw);
  check(olb_ep_pull_dweights(p.data(), static_cast<int>(p.size()), idx.data_ptr<int>(), static_cast<int>(my_rank),
                             static_cast<int>(idx.size(0)), static_cast<int>(idx.size(1)), static_cast<int>(E_loc),
                             dw.data_ptr<float>(), cur_stream()),
        "olb_ep_pull_dweights");
}

void pull_reduce_rows(const std::vector<int64_t>& peer_partial, int64_t row0, int64_t ld, at::Tensor& out) {
  c10::cuda::CUDAGuard guard(out.device());
  auto p = cptrs(peer_partial);
  check(olb_pull_reduce_rows(p.data(), static_cast<int>(p.size()), row0, static_cast<int>(out.size(0)),
                             static_cast<int>(out.size(1)), ld, out.data_ptr(), cur_stream()),
        "olb_pull_reduce_rows");
}

// All-gather -> GEMM in one kernel: C[M, N] = A B^T (or A B with `b_mn_major`), where A's rows are spread over the
// GPUs of a group.  `a_gathered` [n * rows, K] is this GPU's gathered copy with its own block of rows filled in;
// `a_peers[r]` is the address of peer r's slice [rows, K].  Extra warps of the GEMM copy the other slices into
// `a_gathered` over NVLink while the tiles of the local rows run (csrc/gemm_tcgen05.cu: PeerArg<true>); when the
// call returns to the stream, `a_gathered` is complete and later GEMMs read it locally.
void gemm_peer(at::Tensor& a_gathered, const std::vector<int64_t>& a_peers, const at::Tensor& b, at::Tensor& c,
               int64_t M, int64_t N, int64_t K, bool b_mn_major, int64_t my_peer, at::Tensor& flags,
               const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(a_gathered.is_cuda() && a_gathered.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16,
              "bf16 CUDA operands expected");
  TORCH_CHECK(a_gathered.dim() == 2 && b.dim() == 2 && a_gathered.stride(1) == 1 && b.stride(1) == 1);
  const int64_t n = static_cast<int64_t>(a_peers.size());
  TORCH_CHECK(n >= 1 && n <= 8 && M % n == 0 && a_gathered.size(0) >= M, "bad peer layout");
  TORCH_CHECK(flags.scalar_type() == at::kInt && flags.is_contiguous() && flags.numel() >= (M + 127) / 128,
              "flags: one int per 128-row block");
  c10::cuda::CUDAGuard guard(a_gathered.device());
  flags.zero_();
  auto ap = cptrs(a_peers);
  olb_gemm_desc d{};
  d.A = a_gathered.data_ptr();
  d.B = b.data_ptr();
  d.C = c.data_ptr();
  d.lda = a_gathered.stride(0);
  d.ldb = b.stride(0);
  d.ldc = c.stride(-2);
  d.a_rows = a_gathered.size(0);
  d.b_rows = b.size(0);
  d.M = static_cast<int>(M);
  d.N = static_cast<int>(N);
  d.K = static_cast<int>(K);
  d.a_mn_major = false;
  d.b_mn_major = b_mn_major;
  d.mode = OLB_GEMM_DENSE;
  d.num_experts = 1;
  d.accumulate = false;
  d.out_fp32 = c.scalar_type() == at::kFloat;
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  d.n_peers = static_cast<int>(n);
  d.my_peer = static_cast<int>(my_peer);
  d.A_peers = ap.data();
  d.a_peer_rows = static_cast<int>(M / n);
  d.stage_flags = flags.data_ptr<int>();
  check(olb_gemm_bf16(&d, cur_stream()), "olb_gemm_bf16 (all-gather variant)");
}

// GEMM -> reduce-scatter transport in one kernel: C[M, N] = A B^T (or A B with `b_mn_major`; `b2` / `k_split` as in
// `gemm`) is this GPU's partial of a sum over the group; rows [r * M/n, (r+1) * M/n) belong to peer r.  The kernel
// computes the next peer's rows first and its own last, and extra warps copy every finished row that belongs to
// another peer into `c_peers[r]` (that peer's receive slot for this GPU, [M/n, N], row stride as `c`) with stores
// over NVLink while later tiles run.  After a barrier each GPU sums its slots and its own rows of `c` locally.
void gemm_push(const at::Tensor& a, const at::Tensor& b, const c10::optional<at::Tensor>& b2, int64_t k_split,
               at::Tensor& c, const std::vector<int64_t>& c_peers, int64_t M, int64_t N, int64_t K, bool b_mn_major,
               int64_t my_peer, at::Tensor& flags, const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
                  c.scalar_type() == at::kBFloat16,
              "bf16 CUDA operands expected");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1);
  const int64_t n = static_cast<int64_t>(c_peers.size());
  TORCH_CHECK(n >= 1 && n <= 8 && M % n == 0 && c.size(0) >= M, "bad peer layout");
  TORCH_CHECK(flags.scalar_type() == at::kInt && flags.is_contiguous() && flags.numel() >= (M + 127) / 128,
              "flags: one int per 128-row block");
  c10::cuda::CUDAGuard guard(a.device());
  flags.zero_();
  auto cp = mptrs(c_peers);
  olb_gemm_desc d{};
  d.A = a.data_ptr();
  d.B = b.data_ptr();
  d.C = c.data_ptr();
  d.lda = a.stride(0);
  d.ldb = b.stride(0);
  d.ldc = c.stride(0);
  d.a_rows = a.size(0);
  d.b_rows = b.size(0);
  d.M = static_cast<int>(M);
  d.N = static_cast<int>(N);
  d.K = static_cast<int>(K);
  d.a_mn_major = false;
  d.b_mn_major = b_mn_major;
  d.mode = OLB_GEMM_DENSE;
  d.num_experts = 1;
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  if (b2.has_value() && k_split > 0) {
    TORCH_CHECK(b2->scalar_type() == at::kBFloat16 && b2->stride(0) == b.stride(0) && b2->size(0) == b.size(0));
    d.B2 = b2->data_ptr();
    d.k_split = static_cast<int>(k_split);
  }
  d.n_peers = static_cast<int>(n);
  d.my_peer = static_cast<int>(my_peer);
  d.a_peer_rows = static_cast<int>(M / n);
  d.C_peers = cp.data();
  d.stage_flags = flags.data_ptr<int>();
  check(olb_gemm_bf16(&d, cur_stream()), "olb_gemm_bf16 (reduce-scatter variant)");
}

// Grouped expert GEMM (ragged-M: rows grouped by expert, `meta` as in `gemm`) whose finished rows travel to the owners
// of their tokens inside the kernel: C[u, :] = A[u, :] W[expert(u)]^T, and row u is copied to
// `c_peers[owner]`'s [tokens, topk, N] buffer at (token, k) = (src_of[u] % tokens, k_of[u]) by extra warps while later
// tiles run (the expert-parallel combine's all-to-all).  The owner sums its topk slots locally after a barrier.
void gemm_ep_push(const at::Tensor& a, const at::Tensor& w2d, at::Tensor& c, const std::vector<int64_t>& c_peers,
                  const at::Tensor& meta, const at::Tensor& src_of, const at::Tensor& k_of, int64_t M, int64_t N, int64_t K,
                  int64_t b_expert_rows, int64_t num_experts, int64_t tokens, int64_t topk, int64_t my_peer,
                  at::Tensor& flags, const c10::optional<at::Tensor>& status, bool b_mn_major,
                  const c10::optional<at::Tensor>& w2d_2, int64_t k_split, bool pair_rows) {
  TORCH_CHECK(a.is_cuda() && a.scalar_type() == at::kBFloat16 && w2d.scalar_type() == at::kBFloat16 &&
                  c.scalar_type() == at::kBFloat16,
              "bf16 CUDA operands expected");
  TORCH_CHECK(a.dim() == 2 && w2d.dim() == 2 && c.dim() == 2 && a.stride(1) == 1 && w2d.stride(1) == 1 && c.stride(1) == 1);
  TORCH_CHECK(meta.scalar_type() == at::kInt && src_of.scalar_type() == at::kInt && k_of.scalar_type() == at::kInt);
  TORCH_CHECK(src_of.numel() >= M && k_of.numel() >= M && a.size(0) >= M && c.size(0) >= M);
  const int64_t n = static_cast<int64_t>(c_peers.size());
  TORCH_CHECK(n >= 1 && n <= 8, "bad peer count");
  TORCH_CHECK(flags.scalar_type() == at::kInt && flags.is_contiguous() && flags.numel() >= (M + 127) / 128,
              "flags: one int per 128-row block");
  c10::cuda::CUDAGuard guard(a.device());
  flags.zero_();
  auto cp = mptrs(c_peers);
  olb_gemm_desc d{};
  d.A = a.data_ptr();
  d.B = w2d.data_ptr();
  d.C = c.data_ptr();
  d.lda = a.stride(0);
  d.ldb = w2d.stride(0);
  d.ldc = c.stride(0);
  d.a_rows = a.size(0);
  d.b_rows = w2d.size(0);
  d.M = static_cast<int>(M);
  d.N = static_cast<int>(N);
  d.K = static_cast<int>(K);
  d.mode = OLB_GEMM_RAGGED_M;
  d.b_mn_major = b_mn_major;
  if (w2d_2.has_value() && k_split > 0) {   // K-concatenated B: a[:, :k_split] @ w2d + a[:, k_split:] @ w2d_2
    TORCH_CHECK(w2d_2->scalar_type() == at::kBFloat16 && w2d_2->sizes() == w2d.sizes() && w2d_2->strides() == w2d.strides());
    d.B2 = w2d_2->data_ptr();
    d.k_split = static_cast<int>(k_split);
  }
  d.meta = meta.data_ptr<int>();
  d.num_experts = static_cast<int>(num_experts);
  d.b_expert_rows = static_cast<int>(b_expert_rows);
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  d.n_peers = static_cast<int>(n);
  d.my_peer = static_cast<int>(my_peer);
  d.C_peers = cp.data();
  d.stage_flags = flags.data_ptr<int>();
  d.ep_src_of = src_of.data_ptr<int>();
  d.ep_k_of = k_of.data_ptr<int>();
  d.ep_tokens = static_cast<int>(tokens);
  d.ep_topk = static_cast<int>(topk);
  d.pair_rows = pair_rows;
  check(olb_gemm_bf16(&d, cur_stream()), "olb_gemm_bf16 (expert-parallel combine variant)");
}

// Gate and up projection of a SwiGLU MLP in one launch: h[:, :I] = x Wg^T, h[:, I:] = x Wu^T and
// act = w(row) * silu(h[:, :I]) * h[:, I:] written by the GEMM's epilogue.  `wg2d` / `wu2d` are [E * I, K] (E = 1 for a
// dense MLP).  With `meta` the rows are grouped by expert (ragged-M) and `src_of` / `k_of` / `weights` [tokens, topk]
// give the routing weight of every row.  With `x_peers` (addresses of every rank's token buffer [tokens, K], row
// stride `x_ld`) the operand `xp` is filled inside the kernel: extra warps fetch row u = token src_of[u] from its
// owner (the expert-parallel dispatch; with one entry, the local permutation) while earlier tiles already run.
void gemm_gateup_swiglu(at::Tensor& xp, const at::Tensor& wg2d, const at::Tensor& wu2d, at::Tensor& h, at::Tensor& act,
                        int64_t M, int64_t I, int64_t K, const c10::optional<at::Tensor>& meta,
                        const c10::optional<at::Tensor>& src_of, const c10::optional<at::Tensor>& k_of,
                        const c10::optional<at::Tensor>& weights, int64_t num_experts,
                        const std::vector<int64_t>& x_peers, int64_t x_ld, int64_t tokens,
                        const c10::optional<at::Tensor>& flags, const c10::optional<at::Tensor>& status,
                        bool pair_rows) {
  TORCH_CHECK(xp.is_cuda() && xp.scalar_type() == at::kBFloat16 && wg2d.scalar_type() == at::kBFloat16 &&
                  wu2d.scalar_type() == at::kBFloat16 && h.scalar_type() == at::kBFloat16 &&
                  act.scalar_type() == at::kBFloat16,
              "bf16 CUDA operands expected");
  TORCH_CHECK(xp.dim() == 2 && wg2d.dim() == 2 && h.dim() == 2 && act.dim() == 2 && xp.stride(1) == 1 &&
              wg2d.stride(1) == 1 && h.stride(1) == 1 && act.stride(1) == 1);
  TORCH_CHECK(wu2d.sizes() == wg2d.sizes() && wu2d.strides() == wg2d.strides(), "gate and up weights must share a layout");
  TORCH_CHECK(xp.size(0) >= M && h.size(0) >= M && act.size(0) >= M && h.size(1) == 2 * I && act.size(1) == I);
  c10::cuda::CUDAGuard guard(xp.device());
  olb_gemm_desc d{};
  d.A = xp.data_ptr();
  d.B = wg2d.data_ptr();
  d.B2 = wu2d.data_ptr();
  d.C = h.data_ptr();
  d.C2 = act.data_ptr();
  d.lda = xp.stride(0);
  d.ldb = wg2d.stride(0);
  d.ldc = h.stride(0);
  d.ldc2 = act.stride(0);
  d.a_rows = xp.size(0);
  d.b_rows = wg2d.size(0);
  d.M = static_cast<int>(M);
  d.N = static_cast<int>(I);
  d.K = static_cast<int>(K);
  d.epilogue = OLB_EPI_SWIGLU;
  d.num_experts = static_cast<int>(num_experts);
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  if (meta.has_value()) {
    d.mode = OLB_GEMM_RAGGED_M;
    d.meta = meta->data_ptr<int>();
    d.b_expert_rows = static_cast<int>(I);
  } else {
    d.mode = OLB_GEMM_DENSE;
  }
  if (src_of.has_value() && weights.has_value()) {
    TORCH_CHECK(k_of.has_value() && src_of->scalar_type() == at::kInt && k_of->scalar_type() == at::kInt &&
                weights->scalar_type() == at::kFloat && weights->dim() == 2 && weights->is_contiguous() &&
                src_of->numel() >= M && k_of->numel() >= M);
    d.row_src_of = src_of->data_ptr<int>();
    d.row_k_of = k_of->data_ptr<int>();
    d.row_weights = weights->data_ptr<float>();
    d.row_topk = static_cast<int>(weights->size(1));
  }
  std::vector<const void*> xs;
  if (!x_peers.empty()) {
    TORCH_CHECK(meta.has_value() && src_of.has_value() && flags.has_value() && x_peers.size() <= 8 && tokens > 0);
    TORCH_CHECK(flags->scalar_type() == at::kInt && flags->is_contiguous() && flags->numel() >= (M + 127) / 128,
                "flags: one int per 128-row block");
    flags->zero_();
    xs = cptrs(x_peers);
    d.n_peers = static_cast<int>(xs.size());
    d.A_peers = xs.data();
    d.a_src_ld = x_ld;
    d.stage_flags = flags->data_ptr<int>();
    d.ep_src_of = src_of->data_ptr<int>();
    d.ep_tokens = static_cast<int>(tokens);
  }
  d.pair_rows = pair_rows;
  check(olb_gemm_bf16(&d, cur_stream()), "olb_gemm_bf16 (gate|up + SwiGLU)");
}

// Grouped GEMM whose operand rows are gathered inside the kernel (see gemm_gateup_swiglu): c[u, :] = xp[u, :] W[e(u)]^T
// (or xp W with `b_mn_major`) with xp[u] = x_peers[src_of[u] / tokens][src_of[u] % tokens].  `xp` is left filled.
// With `h` (saved gate | up [rows, 2 N]), `k_of`, `weights` and `dw_partial` the SwiGLU backward runs in the launch's
// epilogue: `c` is then d(gate) | d(up) [rows, 2 N] and `dw_partial` [rows, N / 256] receives the per-tile partials of the
// routing-weight gradient (CTA-pair kernel: rows padded to 256 per expert, N a multiple of 256).
void gemm_ep_gather(at::Tensor& xp, const at::Tensor& w2d, at::Tensor& c, int64_t M, int64_t N, int64_t K, bool b_mn_major,
                    const at::Tensor& meta, const at::Tensor& src_of, int64_t b_expert_rows, int64_t num_experts,
                    const std::vector<int64_t>& x_peers, int64_t x_ld, int64_t tokens, at::Tensor& flags,
                    const c10::optional<at::Tensor>& status, bool pair_rows, const c10::optional<at::Tensor>& h,
                    const c10::optional<at::Tensor>& k_of, const c10::optional<at::Tensor>& weights,
                    const c10::optional<at::Tensor>& dw_partial) {
  TORCH_CHECK(xp.is_cuda() && xp.scalar_type() == at::kBFloat16 && w2d.scalar_type() == at::kBFloat16 &&
                  c.scalar_type() == at::kBFloat16,
              "bf16 CUDA operands expected");
  TORCH_CHECK(xp.dim() == 2 && w2d.dim() == 2 && c.dim() == 2 && xp.stride(1) == 1 && w2d.stride(1) == 1 && c.stride(1) == 1);
  TORCH_CHECK(xp.size(0) >= M && c.size(0) >= M && src_of.scalar_type() == at::kInt && src_of.numel() >= M);
  TORCH_CHECK(!x_peers.empty() && x_peers.size() <= 8 && tokens > 0);
  TORCH_CHECK(flags.scalar_type() == at::kInt && flags.is_contiguous() && flags.numel() >= (M + 127) / 128,
              "flags: one int per 128-row block");
  c10::cuda::CUDAGuard guard(xp.device());
  flags.zero_();
  auto xs = cptrs(x_peers);
  olb_gemm_desc d{};
  d.A = xp.data_ptr();
  d.B = w2d.data_ptr();
  d.C = c.data_ptr();
  d.lda = xp.stride(0);
  d.ldb = w2d.stride(0);
  d.ldc = c.stride(0);
  d.a_rows = xp.size(0);
  d.b_rows = w2d.size(0);
  d.M = static_cast<int>(M);
  d.N = static_cast<int>(N);
  d.K = static_cast<int>(K);
  d.b_mn_major = b_mn_major;
  d.mode = OLB_GEMM_RAGGED_M;
  d.meta = meta.data_ptr<int>();
  d.num_experts = static_cast<int>(num_experts);
  d.b_expert_rows = static_cast<int>(b_expert_rows);
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  d.n_peers = static_cast<int>(xs.size());
  d.A_peers = xs.data();
  d.a_src_ld = x_ld;
  d.stage_flags = flags.data_ptr<int>();
  d.ep_src_of = src_of.data_ptr<int>();
  d.ep_tokens = static_cast<int>(tokens);
  d.pair_rows = pair_rows;
  if (h.has_value()) {
    TORCH_CHECK(k_of.has_value() && weights.has_value() && dw_partial.has_value() && h->scalar_type() == at::kBFloat16 &&
                h->dim() == 2 && h->stride(1) == 1 && h->size(0) >= M && h->size(1) == 2 * N && c.size(1) == 2 * N &&
                weights->scalar_type() == at::kFloat && weights->is_contiguous() && weights->dim() == 2 &&
                k_of->scalar_type() == at::kInt && dw_partial->scalar_type() == at::kFloat && dw_partial->is_contiguous() &&
                dw_partial->numel() >= M * ((N + 255) / 256));
    d.epilogue = OLB_EPI_SWIGLU_BWD;
    d.aux_in = h->data_ptr();
    d.aux_ld = h->stride(0);
    d.aux_out = dw_partial->data_ptr<float>();
    d.row_src_of = src_of.data_ptr<int>();
    d.row_k_of = k_of->data_ptr<int>();
    d.row_weights = weights->data_ptr<float>();
    d.row_topk = static_cast<int>(weights->size(1));
  }
  check(olb_gemm_bf16(&d, cur_stream()), "olb_gemm_bf16 (expert-parallel dispatch variant)");
}

// dst (a CUDA tensor, contiguous) <- `bytes` bytes at address `src` (possibly another GPU's memory).
void peer_copy(int64_t src, at::Tensor& dst, int64_t bytes) {
  c10::cuda::CUDAGuard guard(dst.device());
  TORCH_CHECK(dst.is_contiguous() && bytes <= static_cast<int64_t>(dst.numel() * dst.element_size()));
  check(olb_peer_copy(reinterpret_cast<const void*>(static_cast<uintptr_t>(src)), dst.data_ptr(), bytes, cur_stream()),
        "olb_peer_copy");
}

// y = x w^T where parts of w are fetched from the peers that own their current values while the GEMM runs (the parameter
// all-gather of a sharded optimizer step, fused into the first GEMM that consumes the weight).  `w_peers[r]` is the
// address of w in peer r's memory, `seg` = [lo_0, hi_0, lo_1, hi_1, ...]: elements of w current only on peer r.
void gemm_b_gather(const at::Tensor& x, at::Tensor& w, at::Tensor& y, int64_t M, int64_t N, int64_t K,
                   const std::vector<int64_t>& w_peers, const std::vector<int64_t>& seg, int64_t my_peer, at::Tensor& flags,
                   const c10::optional<at::Tensor>& status) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 &&
                  y.scalar_type() == at::kBFloat16,
              "bf16 CUDA operands expected");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && y.dim() == 2 && x.stride(1) == 1 && w.is_contiguous() && y.stride(1) == 1);
  TORCH_CHECK(w_peers.size() <= 8 && seg.size() == 2 * w_peers.size() && !w_peers.empty());
  TORCH_CHECK(flags.scalar_type() == at::kInt && flags.is_contiguous() && flags.numel() >= (N + 127) / 128);
  c10::cuda::CUDAGuard guard(x.device());
  flags.zero_();
  auto wp = cptrs(w_peers);
  std::vector<long long> sg(seg.begin(), seg.end());
  olb_gemm_desc d{};
  d.A = x.data_ptr();
  d.B = w.data_ptr();
  d.C = y.data_ptr();
  d.lda = x.stride(0);
  d.ldb = w.stride(0);
  d.ldc = y.stride(0);
  d.a_rows = x.size(0);
  d.b_rows = w.size(0);
  d.M = static_cast<int>(M);
  d.N = static_cast<int>(N);
  d.K = static_cast<int>(K);
  d.mode = OLB_GEMM_DENSE;
  d.num_experts = 1;
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  d.n_peers = static_cast<int>(wp.size());
  d.my_peer = static_cast<int>(my_peer);
  d.B_peers = wp.data();
  d.b_seg = sg.data();
  d.stage_flags = flags.data_ptr<int>();
  check(olb_gemm_bf16(&d, cur_stream()), "olb_gemm_bf16 (parameter all-gather variant)");
}

int64_t rs_adamw_blocks(int64_t n) { return olb_rs_adamw_blocks(n); }

void rs_adamw(const std::vector<int64_t>& peer_grad, const std::vector<int64_t>& peer_param, int64_t shard_off,
              at::Tensor& master, at::Tensor& m, at::Tensor& v, double lr, double beta1, double beta2, double eps,
              double weight_decay, int64_t step, double grad_scale, const c10::optional<at::Tensor>& clip_coef,
              at::Tensor& norm_partial, int64_t mode, bool skip_weight_update, int64_t mc_grad, int64_t mc_param,
              const c10::optional<at::Tensor>& local_only, int64_t my_rank) {
  c10::cuda::CUDAGuard guard(master.device());
  const long long* lo_ptr = nullptr;
  int n_lo = 0;
  if (local_only.has_value() && local_only->numel() > 0) {
    TORCH_CHECK(local_only->is_cuda() && local_only->scalar_type() == at::kLong && local_only->is_contiguous() &&
                local_only->dim() == 2 && local_only->size(1) == 2, "local_only: int64 CUDA tensor [n, 2]");
    lo_ptr = reinterpret_cast<const long long*>(local_only->data_ptr<int64_t>());
    n_lo = static_cast<int>(local_only->size(0));
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
  auto pg = cptrs(peer_grad);
  auto pp = mptrs(peer_param);
  TORCH_CHECK(norm_partial.numel() >= olb_rs_adamw_blocks(master.numel()), "norm_partial too small");
  check(olb_rs_adamw_ex(pg.data(), pp.data(), static_cast<int>(pg.size()), shard_off, master.numel(),
                        master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), &hp,
                        clip_coef.has_value() ? clip_coef->data_ptr<float>() : nullptr, norm_partial.data_ptr<float>(),
                        static_cast<int>(mode), reinterpret_cast<const void*>(static_cast<uintptr_t>(mc_grad)),
                        reinterpret_cast<void*>(static_cast<uintptr_t>(mc_param)), lo_ptr, n_lo, static_cast<int>(my_rank),
                        cur_stream()),
        "olb_rs_adamw");
}

}  // namespace

void register_comm(pybind11::module& m) {
  namespace py = pybind11;
  m.def("symm_barrier", &symm_barrier, py::arg("pads"), py::arg("my_rank"), py::arg("channel"), py::arg("epoch"),
        py::arg("status"), py::arg("wait_limit_ns") = 0);
  m.def("ep_publish_meta", &ep_publish_meta);
  m.def("sum_slots", &sum_slots);
  m.def("ep_gather_rows", &ep_gather_rows);
  m.def("ep_resolve_rows", &ep_resolve_rows);
  m.def("ep_combine", &ep_combine);
  m.def("ep_pull_dweights", &ep_pull_dweights);
  m.def("pull_reduce_rows", &pull_reduce_rows);
  m.def("gemm_peer", &gemm_peer);
  m.def("gemm_push", &gemm_push);
  m.def("gemm_ep_push", &gemm_ep_push, py::arg("a"), py::arg("w2d"), py::arg("c"), py::arg("c_peers"), py::arg("meta"),
        py::arg("src_of"), py::arg("k_of"), py::arg("M"), py::arg("N"), py::arg("K"), py::arg("b_expert_rows"),
        py::arg("num_experts"), py::arg("tokens"), py::arg("topk"), py::arg("my_peer"), py::arg("flags"),
        py::arg("status"), py::arg("b_mn_major") = false, py::arg("w2d_2") = py::none(), py::arg("k_split") = 0,
        py::arg("pair_rows") = false);
  m.def("gemm_gateup_swiglu", &gemm_gateup_swiglu, py::arg("xp"), py::arg("wg2d"), py::arg("wu2d"), py::arg("h"),
        py::arg("act"), py::arg("M"), py::arg("I"), py::arg("K"), py::arg("meta"), py::arg("src_of"), py::arg("k_of"),
        py::arg("weights"), py::arg("num_experts"), py::arg("x_peers"), py::arg("x_ld"), py::arg("tokens"),
        py::arg("flags"), py::arg("status"), py::arg("pair_rows") = false);
  m.def("gemm_ep_gather", &gemm_ep_gather, py::arg("xp"), py::arg("w2d"), py::arg("c"), py::arg("M"), py::arg("N"),
        py::arg("K"), py::arg("b_mn_major"), py::arg("meta"), py::arg("src_of"), py::arg("b_expert_rows"),
        py::arg("num_experts"), py::arg("x_peers"), py::arg("x_ld"), py::arg("tokens"), py::arg("flags"),
        py::arg("status"), py::arg("pair_rows") = false, py::arg("h") = py::none(), py::arg("k_of") = py::none(),
        py::arg("weights") = py::none(), py::arg("dw_partial") = py::none());
  m.def("rs_adamw_blocks", &rs_adamw_blocks);
  m.def("rs_adamw", &rs_adamw, py::arg("peer_grad"), py::arg("peer_param"), py::arg("shard_off"), py::arg("master"),
        py::arg("m"), py::arg("v"), py::arg("lr"), py::arg("beta1"), py::arg("beta2"), py::arg("eps"),
        py::arg("weight_decay"), py::arg("step"), py::arg("grad_scale"), py::arg("clip_coef"), py::arg("norm_partial"),
        py::arg("mode"), py::arg("skip_weight_update"), py::arg("mc_grad") = 0, py::arg("mc_param") = 0,
        py::arg("local_only") = py::none(), py::arg("my_rank") = 0);
  m.def("peer_copy", &peer_copy);
  m.def("gemm_b_gather", &gemm_b_gather);
}
