"""Tensor-parallel SwiGLU MLP with the collectives folded into the GEMMs over peer memory.

Sequence-sharded input ``x [T_loc, H]``, column-sharded gate / up weights ``[I_loc, H]``, row-sharded down weight
``[H, I_loc]`` - the layout of DeepSeek-V3's dense MLP sharded over the expert-parallel group and of a
sequence-parallel TP block.  The reference runs all-gather -> three GEMMs -> reduce-scatter as separate
collectives and library GEMMs (optimus/models/deepseek_v3/modeling_deepseek_v3.py:90-118 with
comms_ptfunctions.py:118-156).  Here:

* **all-gather -> GEMM**: every rank publishes its ``x`` rows in a symmetric buffer; the gate / up GEMMs read the
  row blocks of ``A`` straight from the owners' memories with TMA loads over NVLink (per-peer tensor maps inside
  the tcgen05 GEMM kernel, row-block order rotated so that a rank starts on its own rows).  No gathered copy of
  the activations exists in the forward; the backward re-publishes the saved local ``x`` for the weight gradients.
* **GEMM -> reduce-scatter**: the down projection writes this rank's partial ``[T, H]`` into a symmetric buffer;
  after a device-side barrier each rank pulls and sums (fp32) only its own rows from all peers.

The backward mirrors it (all-gather of ``dout`` inside the dgrad / wgrad GEMMs - the K rows of ``dout^T`` and of
``x`` are read from the peers - and a pull-reduce of ``dx``).  All waits are bounded device barriers.
"""
from __future__ import annotations

import os

import torch

from ..ops import functional as OF
from ..ops._ext import extension, use_kernels
from .symm import SymmGroup, peer_access_ok

_CH_X, _CH_Y, _CH_DY, _CH_DX = 8, 9, 10, 11   # barrier channels (the EP kernels use 0-3)
_PEER_OK = {}


def usable(x, group, weights=()) -> bool:
    """True when the fused peer-memory path can run for ``x [T_loc, H]`` on ``group``."""
    if os.environ.get("OLB_DISABLE_TP_FUSED") or not x.is_cuda or x.dtype != torch.bfloat16 or not use_kernels(x):
        return False
    if x.dim() != 2 or x.shape[0] % 128 or x.shape[1] % 64:
        return False
    for w in weights:
        if w.dtype != torch.bfloat16 or w.shape[0] % 64 or w.shape[1] % 64:
            return False
    key = id(group)
    if key not in _PEER_OK:
        try:
            _PEER_OK[key] = bool(peer_access_ok(group))
        except Exception:  # noqa: BLE001 - no peer access means no fused path
            _PEER_OK[key] = False
    return _PEER_OK[key]


class _AGSwiGLURSFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, wg, wu, wd, rank, n, sg: SymmGroup, holders):
        C = extension()
        T_loc, H = x.shape
        I = wg.shape[0]
        T = n * T_loc
        st = OF.status_word(x.device)
        xs = sg.named("tp_x", (T_loc, H), x.dtype)
        xs.local.copy_(x)
        sg.barrier(_CH_X)
        gu = torch.empty((T, 2 * I), dtype=x.dtype, device=x.device)
        # all-gather -> GEMM: A row blocks come from the peers' copies of x
        C.gemm_peer(xs.local, xs.ptrs, wg, [], gu[:, :I], T, I, H, False, False, rank, False, st)
        C.gemm_peer(xs.local, xs.ptrs, wu, [], gu[:, I:], T, I, H, False, False, rank, False, st)
        act = torch.empty((T, I), dtype=x.dtype, device=x.device)
        C.swiglu_fwd(gu[:, :I], gu[:, I:], act)
        ys = sg.named("tp_y", (T, H), x.dtype)
        OF.gemm(act, wd, T, H, I, out=ys.local)
        sg.barrier(_CH_Y)
        # GEMM -> reduce-scatter: sum my rows of every rank's partial
        out = torch.empty((T_loc, H), dtype=x.dtype, device=x.device)
        C.pull_reduce_rows(ys.ptrs, rank * T_loc, H, out)
        ctx.save_for_backward(x, gu, act, wg, wu, wd)
        ctx.misc = (rank, n, sg, holders)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = extension()
        x, gu, act, wg, wu, wd = ctx.saved_tensors
        rank, n, sg, (hg, hu, hd) = ctx.misc
        T_loc, H = x.shape
        I = wg.shape[0]
        T = n * T_loc
        st = OF.status_word(x.device)
        xs = sg.named("tp_x", (T_loc, H), x.dtype)
        dys = sg.named("tp_dy", (T_loc, H), x.dtype)
        xs.local.copy_(x)                      # the weight gradients need every rank's x again
        dys.local.copy_(dout)
        sg.barrier(_CH_DY)

        def wgrad(holder, a_local, a_ptrs, b_local, b_ptrs, M, N):
            """dW[M, N] = A^T B over all T rows, A / B given row-major [rows, M] / [rows, N] (MN-major operands)."""
            if holder is not None:
                C.gemm_peer(a_local, a_ptrs, b_local, b_ptrs, holder.buf, M, N, T, True, True, rank, holder.ready, st)
                holder.ready = True
                return None
            dw = torch.empty((M, N), dtype=x.dtype, device=x.device)
            C.gemm_peer(a_local, a_ptrs, b_local, b_ptrs, dw, M, N, T, True, True, rank, False, st)
            return dw

        # d(act) = dout_full @ wd : A rows (dout) from the peers, B = wd read MN-major
        dact = torch.empty((T, I), dtype=x.dtype, device=x.device)
        C.gemm_peer(dys.local, dys.ptrs, wd, [], dact, T, I, H, False, True, rank, False, st)
        # d(wd)[H, I] = dout_full^T @ act : the K rows of A come from the peers
        dwd = wgrad(hd, dys.local, dys.ptrs, act, [], H, I) if ctx.needs_input_grad[3] else None
        dgu = torch.empty_like(gu)
        C.swiglu_bwd(dact, gu[:, :I], gu[:, I:], dgu[:, :I], dgu[:, I:])
        del dact
        # d(wg)[I, H] = dg^T @ x_full : the K rows of B come from the peers
        dwg = wgrad(hg, dgu[:, :I], [], xs.local, xs.ptrs, I, H) if ctx.needs_input_grad[1] else None
        dwu = wgrad(hu, dgu[:, I:], [], xs.local, xs.ptrs, I, H) if ctx.needs_input_grad[2] else None
        # d(x_full) = dg @ wg + du @ wu in one launch, then reduce-scatter by peer pulls
        dxs = sg.named("tp_y", (T, H), x.dtype)
        OF.gemm(dgu, wg, T, H, 2 * I, b_mn_major=True, out=dxs.local, b2=wu, k_split=I)
        sg.barrier(_CH_DX)
        dx = torch.empty((T_loc, H), dtype=x.dtype, device=x.device)
        C.pull_reduce_rows(dxs.ptrs, rank * T_loc, H, dx)
        return dx, dwg, dwu, dwd, None, None, None, None


def ag_swiglu_mlp_rs(x, wg, wu, wd, rank, n, group):
    """``reduce_scatter(swiglu(all_gather(x) @ wg.T, all_gather(x) @ wu.T) @ wd.T)`` for row-sharded ``x``."""
    sg = SymmGroup.get(group)
    holders = (OF._holder(wg), OF._holder(wu), OF._holder(wd))
    return _AGSwiGLURSFn.apply(x.contiguous(), wg, wu, wd, rank, n, sg, holders)
