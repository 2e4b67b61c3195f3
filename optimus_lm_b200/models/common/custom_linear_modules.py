"""Linear layers for tensor parallelism on the tcgen05 GEMM (reference
optimus/models/common/custom_linear_modules.py:8-131: ``PclLinear``, ``ColumnLinear``, ``RowLinear``)."""
import torch
from torch import nn

from ...ops import functional as OF


class PclLinear(nn.Linear):
    """``nn.Linear`` whose matmul runs on the kernel path."""

    def forward(self, x):
        y = OF.linear(x, self.weight)
        return y if self.bias is None else y + self.bias


class ColumnLinear(PclLinear):
    """Holds ``out_features / TP`` output rows."""

    def __init__(self, in_features, out_features, bias=False, tensor_parallelism=1, tp_ind=0):
        assert out_features % tensor_parallelism == 0
        super().__init__(in_features, out_features // tensor_parallelism, bias=bias)
        self.tensor_parallelism, self.tp_ind = tensor_parallelism, tp_ind
        self.full_out_features = out_features


class RowLinear(PclLinear):
    """Holds ``in_features / TP`` input columns; outputs are partial sums."""

    def __init__(self, in_features, out_features, bias=False, tensor_parallelism=1, tp_ind=0):
        assert in_features % tensor_parallelism == 0
        super().__init__(in_features // tensor_parallelism, out_features, bias=bias)
        self.tensor_parallelism, self.tp_ind = tensor_parallelism, tp_ind
        self.full_in_features = in_features
