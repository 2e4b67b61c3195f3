"""Normalisation modules backed by the fused kernels.

``RMSNorm`` has the reference's semantics and parameter name ``weight``
(optimus/models/common/norm_modules.py:4-43, optimus/models/olmoe/modeling_olmoe.py:93-104);
``NonParametricLayerNorm`` is OLMo's fp32 LayerNorm without affine parameters
(optimus/models/olmo/modeling_olmo.py:19-30).
"""
import torch
from torch import nn

from ...ops import functional as OF


class RMSNorm(nn.Module):
    def __init__(self, hidden_size, eps=1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size))
        self.variance_epsilon = eps

    def forward(self, hidden_states):
        return OF.rms_norm(hidden_states, self.weight, self.variance_epsilon)

    def forward_add(self, hidden_states, residual):
        """``(hidden_states + residual, norm(hidden_states + residual))`` in one kernel."""
        return OF.add_rms_norm(hidden_states, residual, self.weight, self.variance_epsilon)

    def extra_repr(self):
        return f"{tuple(self.weight.shape)}, eps={self.variance_epsilon}"


# Name used by the reference's shared modules.
PclLlamaRMSNorm = RMSNorm


class NonParametricLayerNorm(nn.Module):
    def __init__(self, hidden_size=None, eps=1e-5):
        super().__init__()
        self.eps = eps

    def forward(self, x):
        return OF.layer_norm_noaffine(x, self.eps)
