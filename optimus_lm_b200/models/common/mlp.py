"""Plain SwiGLU MLP: ``down(silu(gate(x)) * up(x))`` with bias-free projections (reference
optimus/models/common/mlp.py:4-15).  The three GEMMs and the activation run on the framework's kernels for bf16
CUDA tensors; the tensor-parallel version is ``dense_decoder.ParallelMLP``."""
import torch.nn as nn

from ...ops import functional as OF


class MLP(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.intermediate_size = config.intermediate_size
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=False)

    def forward(self, x):
        h = OF.swiglu(OF.linear(x, self.gate_proj.weight), OF.linear(x, self.up_proj.weight))
        return OF.linear(h, self.down_proj.weight)
