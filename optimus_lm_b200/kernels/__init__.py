"""Kernel entry points under the names of the reference's ``optimus/kernels`` modules.

The reference ships one Triton file per GEMM flavour (``gemm.py`` NN, ``gemm_trans.py`` NT, ``linear_forward.py``,
``linear_backward_input[_add].py``, ``linear_backward_weight.py``, ``grouped_linear_*.py`` with pointer-array
weights, ``merged_mlp_triton_kernels.py`` with ``[E, N, K]`` weights) and ``moe_nongemm.py`` for the permutation
kernels.  Here one persistent tcgen05 kernel (``csrc/gemm_tcgen05.cu``) covers all GEMM flavours through operand
majorness, an accumulate flag and the ragged-M / ragged-K modes; these wrappers give each flavour its reference
name.  All take bf16 CUDA tensors.  ``python -m optimus_lm_b200.kernels`` runs the micro-benchmarks
(``ops/bench_kernels.py``), the counterpart of the reference files' ``__main__`` blocks.
"""
from __future__ import annotations

import torch

from ..ops import functional as OF
from .. import custom_ops as moe_nongemm  # noqa: F401  (K1-K6 entry points with the reference's argument lists)


def gemm(a: torch.Tensor, b: torch.Tensor, out=None, accumulate=False):
    """``a [M, K] @ b [K, N]`` (NN; reference kernels/gemm.py)."""
    M, K = a.shape
    return OF.gemm(a, b, M, b.shape[1], K, b_mn_major=True, out=out, accumulate=accumulate)


def gemm_trans(a: torch.Tensor, b: torch.Tensor, out=None, accumulate=False):
    """``a [M, K] @ b [N, K].T`` (NT; reference kernels/gemm_trans.py)."""
    M, K = a.shape
    return OF.gemm(a, b, M, b.shape[0], K, out=out, accumulate=accumulate)


def linear_forward(x, w, out=None):
    """``y = x @ w.T`` with ``w [N, K]`` (reference kernels/linear_forward.py)."""
    return gemm_trans(x, w, out=out)


def linear_backward_input(dy, w, out=None):
    """``dx = dy @ w`` (reference kernels/linear_backward_input.py)."""
    return OF.gemm(dy, w, dy.shape[0], w.shape[1], w.shape[0], b_mn_major=True, out=out)


def linear_backward_input_add(dy, w, dx):
    """``dx += dy @ w`` (read-modify-write epilogue; reference kernels/linear_backward_input_add.py)."""
    return OF.gemm(dy, w, dy.shape[0], w.shape[1], w.shape[0], b_mn_major=True, out=dx, accumulate=True)


def linear_backward_weight(dy, x, out=None, accumulate=False):
    """``dw = dy.T @ x`` (TN; reference kernels/linear_backward_weight.py)."""
    return OF.gemm(dy, x, dy.shape[1], x.shape[1], dy.shape[0], a_mn_major=True, b_mn_major=True, out=out,
                   accumulate=accumulate)


# Expert-grouped variants.  The reference passes cumulative token counts and either a pointer array of per-expert
# weights or one merged [E, N, K] tensor; here the rows are grouped and 128-padded by ``OF.MoEIndex`` and the
# weights are always the merged tensor (per-expert modules are stacked views of it).
def grouped_linear_forward(xp, w_merged, index: "OF.MoEIndex", out=None):
    return OF.grouped_linear_fwd(xp, w_merged, index, out=out)


def grouped_linear_backward_input(dy, w_merged, index: "OF.MoEIndex", out=None):
    return OF.grouped_linear_dgrad(dy, w_merged, index, out=out)


def grouped_linear_backward_input_add(dy, w_merged, index: "OF.MoEIndex", dx):
    return OF.grouped_linear_dgrad(dy, w_merged, index, out=dx, accumulate=True)


def grouped_linear_backward_weight(dy, xp, index: "OF.MoEIndex"):
    return OF.grouped_linear_wgrad(dy, xp, index, dy.shape[1], xp.shape[1])


merged_grouped_linear_forward = grouped_linear_forward
merged_grouped_linear_backward_input = grouped_linear_backward_input
merged_grouped_linear_backward_weight = grouped_linear_backward_weight
