// Python bindings for the attention backward kernels (attention_bwd.cu).
// All tensors are bf16 [B, S, H, Dh] views with unit inner stride; lse is fp32 [B, Hq, S].
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "olb_api.h"

namespace {

void check4b(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 4 && t.stride(3) == 1, name,
              " must be a CUDA bf16 [B, S, H, D] tensor with unit inner stride");
}

void attn_bwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, const at::Tensor& o, const at::Tensor& lse,
              const at::Tensor& dout, at::Tensor& dq, at::Tensor& dk, at::Tensor& dv, double scale,
              const c10::optional<at::Tensor>& status) {
  check4b(q, "q"); check4b(k, "k"); check4b(v, "v"); check4b(o, "o"); check4b(dout, "dout");
  check4b(dq, "dq"); check4b(dk, "dk"); check4b(dv, "dv");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous(), "lse must be contiguous fp32 [B, H, S]");
  c10::cuda::CUDAGuard guard(q.device());
  // scratch: delta and the base-2 log-sum-exp, [2, B, Hq, S] fp32
  at::Tensor scratch = at::empty({2, q.size(0), q.size(2), q.size(1)}, lse.options());
  olb_attn_bwd_desc d{};
  d.q = q.data_ptr(); d.k = k.data_ptr(); d.v = v.data_ptr(); d.o = o.data_ptr(); d.dout = dout.data_ptr();
  d.lse = lse.data_ptr<float>();
  d.dq = dq.data_ptr(); d.dk = dk.data_ptr(); d.dv = dv.data_ptr();
  d.dq_acc = nullptr;
  d.delta = scratch.data_ptr<float>();
  d.q_bs = q.stride(0); d.q_ss = q.stride(1); d.q_hs = q.stride(2);
  d.k_bs = k.stride(0); d.k_ss = k.stride(1); d.k_hs = k.stride(2);
  d.v_bs = v.stride(0); d.v_ss = v.stride(1); d.v_hs = v.stride(2);
  d.o_bs = o.stride(0); d.o_ss = o.stride(1); d.o_hs = o.stride(2);
  d.do_bs = dout.stride(0); d.do_ss = dout.stride(1); d.do_hs = dout.stride(2);
  d.dq_bs = dq.stride(0); d.dq_ss = dq.stride(1); d.dq_hs = dq.stride(2);
  d.dk_bs = dk.stride(0); d.dk_ss = dk.stride(1); d.dk_hs = dk.stride(2);
  d.dv_bs = dv.stride(0); d.dv_ss = dv.stride(1); d.dv_hs = dv.stride(2);
  d.B = static_cast<int>(q.size(0));
  d.S = static_cast<int>(q.size(1));
  d.Hq = static_cast<int>(q.size(2));
  d.Hkv = static_cast<int>(k.size(2));
  d.D = static_cast<int>(q.size(3));
  d.Dv = static_cast<int>(v.size(3));
  d.scale = static_cast<float>(scale);
  d.status = status.has_value() ? status->data_ptr<int>() : nullptr;
  const int rc = olb_attn_bwd(&d, at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "olb_attn_bwd failed with code ", rc);
}

}  // namespace

void register_attention_bwd(pybind11::module& m) { m.def("attn_bwd", &attn_bwd); }
