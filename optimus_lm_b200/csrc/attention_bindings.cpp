// Python bindings for the attention kernels (attention.cu, attention_bwd.cu).
// q, k, v, o: bf16 [B, S, H, Dh] views with unit inner stride (any batch / sequence / head strides).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "olb_api.h"

namespace {

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check4(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 4 && t.stride(3) == 1, name,
              " must be a CUDA bf16 [B, S, H, D] tensor with unit inner stride");
}

void attn_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, at::Tensor& o, at::Tensor& lse,
              double scale, const c10::optional<at::Tensor>& status, int64_t variant) {
  check4(q, "q");
  check4(k, "k");
  check4(v, "v");
  check4(o, "o");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse must be contiguous fp32 [B, H, S]");
  c10::cuda::CUDAGuard guard(q.device());
  olb_attn_fwd_desc d{};
  d.q = q.data_ptr();
  d.k = k.data_ptr();
  d.v = v.data_ptr();
  d.o = o.data_ptr();
  d.lse = lse.data_ptr<float>();
  d.q_bs = q.stride(0); d.q_ss = q.stride(1); d.q_hs = q.stride(2);
  d.k_bs = k.stride(0); d.k_ss = k.stride(1); d.k_hs = k.stride(2);
  d.v_bs = v.stride(0); d.v_ss = v.stride(1); d.v_hs = v.stride(2);
  d.o_bs = o.stride(0); d.o_ss = o.stride(1); d.o_hs = o.stride(2);
  d.B = static_cast<int>(q.size(0));
  d.S = static_cast<int>(q.size(1));
  d.Hq = static_cast<int>(q.size(2));
  d.Hkv = static_cast<int>(k.size(2));
  d.D = static_cast<int>(q.size(3));
  d.Dv = static_cast<int>(v.size(3));
  d.scale = static_cast<float>(scale);
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  d.variant = static_cast<int>(variant);
  const int rc = olb_attn_fwd(&d, cur_stream());
  TORCH_CHECK(rc == 0, "olb_attn_fwd failed with code ", rc);
}

}  // namespace

void register_attention_bwd(pybind11::module& m);

void register_attention(pybind11::module& m) {
  m.def("attn_fwd", &attn_fwd, pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"), pybind11::arg("o"),
        pybind11::arg("lse"), pybind11::arg("scale"), pybind11::arg("status"), pybind11::arg("variant") = 0);
  register_attention_bwd(m);
}
