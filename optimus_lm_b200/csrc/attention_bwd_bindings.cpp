// Python bindings for the attention backward kernels (attention_bwd.cu).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "olb_api.h"

void register_attention_bwd(pybind11::module& m) { (void)m; }
