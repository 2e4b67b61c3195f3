"""Tensor-parallel SwiGLU MLP with the collectives folded into the GEMMs over peer memory.

Sequence-sharded input ``x [T_loc, H]``, column-sharded gate / up weights ``[I_loc, H]``, row-sharded down weight
``[H, I_loc]`` - the layout of DeepSeek-V3's dense MLP sharded over the expert-parallel group and of a
sequence-parallel TP block.  The reference runs all-gather -> three GEMMs -> reduce-scatter as separate
collectives and library GEMMs (optimus/models/deepseek_v3/modeling_deepseek_v3.py:90-118 with
comms_ptfunctions.py:118-156).  Here:

* **all-gather -> GEMM**: every rank publishes its ``x`` rows in a symmetric buffer.  The gate GEMM is launched on
  a gathered copy ``[T, H]`` that holds only the local rows; extra warps of each of its CTAs copy the other
  ranks' rows in over NVLink (plain peer loads, each row crosses once) and count them per 128-row block, and the
  TMA producer waits for a block's count before loading its tiles.  The tile order starts on the local rows, so the
  copy runs underneath the math.  The up GEMM and the backward's weight gradients read the gathered copy locally.
* **GEMM -> reduce-scatter**: the down projection computes this rank's partial ``[T, H]`` with the next rank's rows
  first and its own last; its epilogue counts finished tiles per row block, and the same extra warps copy each
  finished row of another rank's block into that rank's receive slot with stores over NVLink while later tiles run.
  After a device-side barrier each rank sums its slots and its own rows (fp32, fixed rank order) from local memory.

The backward mirrors it (all-gather of ``dout`` inside the first dgrad GEMM, the same push for ``dx``).  All waits
are bounded: device barriers, the producer's wait for a staged row block, the stagers' wait for finished tiles.
"""
from __future__ import annotations

import os

import torch

from ..ops import functional as OF
from ..ops._ext import extension, use_kernels
from .symm import SymmGroup, peer_access_ok

_CH_X, _CH_Y, _CH_DY = 8, 9, 10   # barrier channels (the EP kernels use 0-3)
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


def _flags(sg: SymmGroup, T: int) -> torch.Tensor:
    f = getattr(sg, "_tp_flags", None)
    if f is None or f.numel() < T // 128:
        f = sg._tp_flags = torch.zeros(max(T // 128, 1), dtype=torch.int32, device=sg.device)
    return f


def _gemm_reduce_scatter(sg: SymmGroup, a, b, T, N, K, rank, n, b_mn_major=False, b2=None, k_split=0):
    """``reduce_scatter(a @ b^T)`` over the group: returns this rank's ``[T / n, N]`` rows of the sum."""
    C = extension()
    T_loc = T // n
    part = getattr(sg, "_tp_part", None)
    if part is None or part.shape != (T, N) or part.dtype != a.dtype:
        part = sg._tp_part = torch.empty((T, N), dtype=a.dtype, device=a.device)
    recv = sg.named("tp_recv", (n, T_loc, N), a.dtype)       # slot s: rank s's partial of my rows
    slot_bytes = T_loc * N * a.element_size()
    C.gemm_push(a, b, b2, k_split, part, [ptr + rank * slot_bytes for ptr in recv.ptrs], T, N, K, b_mn_major, rank,
                _flags(sg, T), OF.status_word(a.device))
    sg.barrier(_CH_Y)
    out = torch.empty((T_loc, N), dtype=a.dtype, device=a.device)
    mine = part.data_ptr() + rank * slot_bytes
    C.pull_reduce_rows([mine if s == rank else recv.local.data_ptr() + s * slot_bytes for s in range(n)], 0, N, out)
    return out


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
        xg = torch.empty((T, H), dtype=x.dtype, device=x.device)       # gathered x, kept for the weight gradients
        xg[rank * T_loc:(rank + 1) * T_loc].copy_(x)
        sg.barrier(_CH_X)
        gu = torch.empty((T, 2 * I), dtype=x.dtype, device=x.device)
        # all-gather -> GEMM: the gate projection brings the peers' rows into xg while it computes
        C.gemm_peer(xg, xs.ptrs, wg, gu[:, :I], T, I, H, False, rank, _flags(sg, T), st)
        OF.gemm(xg, wu, T, I, H, out=gu[:, I:])
        act = torch.empty((T, I), dtype=x.dtype, device=x.device)
        C.swiglu_fwd(gu[:, :I], gu[:, I:], act)
        # GEMM -> reduce-scatter: finished rows travel to their owners while the down projection is still running
        out = _gemm_reduce_scatter(sg, act, wd, T, H, I, rank, n)
        ctx.save_for_backward(xg, gu, act, wg, wu, wd)
        ctx.misc = (rank, n, sg, holders, T_loc)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = extension()
        xg, gu, act, wg, wu, wd = ctx.saved_tensors
        rank, n, sg, (hg, hu, hd), T_loc = ctx.misc
        T, H = xg.shape
        I = wg.shape[0]
        st = OF.status_word(xg.device)
        dys = sg.named("tp_dy", (T_loc, H), xg.dtype)
        dys.local.copy_(dout)
        dyg = torch.empty((T, H), dtype=xg.dtype, device=xg.device)
        dyg[rank * T_loc:(rank + 1) * T_loc].copy_(dout)
        sg.barrier(_CH_DY)

        def wgrad(holder, a, b, M, N):
            """dW[M, N] = a^T b over all T rows; a / b row-major [T, M] / [T, N] (MN-major operands)."""
            if holder is not None:
                OF.gemm(a, b, M, N, T, a_mn_major=True, b_mn_major=True, out=holder.buf, accumulate=holder.ready)
                holder.ready = True
                return None
            return OF.gemm(a, b, M, N, T, a_mn_major=True, b_mn_major=True)

        # d(act) = dout_full @ wd: the all-gather of dout happens inside this GEMM (B = wd read MN-major)
        dact = torch.empty((T, I), dtype=xg.dtype, device=xg.device)
        C.gemm_peer(dyg, dys.ptrs, wd, dact, T, I, H, True, rank, _flags(sg, T), st)
        dwd = wgrad(hd, dyg, act, H, I) if ctx.needs_input_grad[3] else None
        dgu = torch.empty_like(gu)
        C.swiglu_bwd(dact, gu[:, :I], gu[:, I:], dgu[:, :I], dgu[:, I:])
        del dact
        dwg = wgrad(hg, dgu[:, :I], xg, I, H) if ctx.needs_input_grad[1] else None
        dwu = wgrad(hu, dgu[:, I:], xg, I, H) if ctx.needs_input_grad[2] else None
        # d(x_full) = dg @ wg + du @ wu in one launch, reduce-scattered the same way
        dx = _gemm_reduce_scatter(sg, dgu, wg, T, H, 2 * I, rank, n, b_mn_major=True, b2=wu, k_split=I)
        return dx, dwg, dwu, dwd, None, None, None, None


def ag_swiglu_mlp_rs(x, wg, wu, wd, rank, n, group):
    """``reduce_scatter(swiglu(all_gather(x) @ wg.T, all_gather(x) @ wu.T) @ wd.T)`` for row-sharded ``x``."""
    sg = SymmGroup.get(group)
    holders = (OF._holder(wg), OF._holder(wu), OF._holder(wd))
    return _AGSwiGLURSFn.apply(x.contiguous(), wg, wu, wd, rank, n, sg, holders)


# ----------------------------------------------------------------------------- sequence-parallel building blocks
class _AGLinearFn(torch.autograd.Function):
    """``[all_gather(x) @ w.T for w in weights]`` for row-sharded ``x [T_loc, H]`` and column-parallel weights
    (q / k / v, or gate / up).  The first product's launch gathers the peers' rows (all-gather -> GEMM); the others
    read the gathered copy.  Backward: ``dx = reduce_scatter(sum_i dy_i @ w_i)`` as one K-concatenated
    GEMM -> reduce-scatter launch, ``dw_i = dy_i.T @ all_gather(x)``."""

    @staticmethod
    def forward(ctx, x, rank, n, sg, holders, lead, *weights):
        C = extension()
        T_loc, H = x.shape
        T = n * T_loc
        lead = tuple(lead) if lead else (T,)
        st = OF.status_word(x.device)
        xs = sg.named("tp_x", (T_loc, H), x.dtype)
        xs.local.copy_(x)
        xg = torch.empty((T, H), dtype=x.dtype, device=x.device)
        xg[rank * T_loc:(rank + 1) * T_loc].copy_(x)
        sg.barrier(_CH_X)
        outs = []
        for i, w in enumerate(weights):
            # allocated in its final shape: a later in-place op (RoPE) then works on the output itself, not on a view
            y = torch.empty(lead + (w.shape[0],), dtype=x.dtype, device=x.device)
            y2 = y.view(T, w.shape[0])
            if i == 0:
                C.gemm_peer(xg, xs.ptrs, w, y2, T, w.shape[0], H, False, rank, _flags(sg, T), st)
            else:
                OF.gemm(xg, w, T, w.shape[0], H, out=y2)
            outs.append(y)
        ctx.save_for_backward(xg, *weights)
        ctx.misc = (rank, n, sg, holders)
        return tuple(outs)

    @staticmethod
    def backward(ctx, *douts):
        xg, *weights = ctx.saved_tensors
        rank, n, sg, holders = ctx.misc
        T, H = xg.shape
        dws = []
        for i, (dy, w) in enumerate(zip(douts, weights)):
            dw = None
            if ctx.needs_input_grad[6 + i]:
                dy2 = dy.contiguous().view(T, w.shape[0])
                h = holders[i]
                if h is not None:
                    OF.gemm(dy2, xg, w.shape[0], H, T, a_mn_major=True, b_mn_major=True, out=h.buf, accumulate=h.ready)
                    h.ready = True
                else:
                    dw = OF.gemm(dy2, xg, w.shape[0], H, T, a_mn_major=True, b_mn_major=True)
            dws.append(dw)
        # dx_full = [dy_0 | dy_1 | ...] @ [w_0; w_1; ...]: one GEMM whose rows go to their owners as they finish
        d2 = [d.contiguous().view(T, w.shape[0]) for d, w in zip(douts, weights)]
        dcat = d2[0] if len(d2) == 1 else torch.cat(d2, dim=1)
        wcat = weights[0] if len(weights) == 1 else _stacked(weights)
        dx = _gemm_reduce_scatter(sg, dcat, wcat, T, H, dcat.shape[1], rank, n, b_mn_major=True)
        return (dx, None, None, None, None, None) + tuple(dws)


def _stacked(weights):
    """``[w_0; w_1; ...]`` as one matrix: a view when the weights sit back to back in memory (parameters of a flat
    optimizer buffer in registration order), else a copy."""
    w0 = weights[0]
    end = w0.data_ptr() + w0.numel() * w0.element_size()
    ok = w0.is_contiguous()
    for w in weights[1:]:
        ok = ok and w.is_contiguous() and w.data_ptr() == end and w.shape[1] == w0.shape[1]
        end = w.data_ptr() + w.numel() * w.element_size()
    rows = sum(w.shape[0] for w in weights)
    if ok:
        return torch.as_strided(w0, (rows, w0.shape[1]), (w0.shape[1], 1))
    return torch.cat(list(weights), dim=0)


class _LinearRSFn(torch.autograd.Function):
    """``reduce_scatter(a @ w.T)`` for a row-parallel weight (o / down): the GEMM pushes finished rows to their owners
    (GEMM -> reduce-scatter).  Backward: ``da = all_gather(dout) @ w`` with the gather inside the launch,
    ``dw = all_gather(dout).T @ a``."""

    @staticmethod
    def forward(ctx, a, w, rank, n, sg, holder):
        T, K = a.shape
        out = _gemm_reduce_scatter(sg, a, w, T, w.shape[0], K, rank, n)
        ctx.save_for_backward(a, w)
        ctx.misc = (rank, n, sg, holder)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = extension()
        a, w = ctx.saved_tensors
        rank, n, sg, holder = ctx.misc
        T, K = a.shape
        H = w.shape[0]
        T_loc = T // n
        st = OF.status_word(a.device)
        dys = sg.named("tp_dy", (T_loc, H), a.dtype)
        dys.local.copy_(dout)
        dyg = torch.empty((T, H), dtype=a.dtype, device=a.device)
        dyg[rank * T_loc:(rank + 1) * T_loc].copy_(dout)
        sg.barrier(_CH_DY)
        da = torch.empty((T, K), dtype=a.dtype, device=a.device)
        C.gemm_peer(dyg, dys.ptrs, w, da, T, K, H, True, rank, _flags(sg, T), st)
        dw = None
        if ctx.needs_input_grad[1]:
            if holder is not None:
                OF.gemm(dyg, a, H, K, T, a_mn_major=True, b_mn_major=True, out=holder.buf, accumulate=holder.ready)
                holder.ready = True
            else:
                dw = OF.gemm(dyg, a, H, K, T, a_mn_major=True, b_mn_major=True)
        return da, dw, None, None, None, None


def ag_linear(x, weights, rank, n, group, lead=None):
    """Column-parallel projections of a row-sharded activation: returns ``all_gather(x) @ w.T`` for every ``w``, shaped
    ``lead + (w.shape[0],)`` (default ``[T, N]``)."""
    sg = SymmGroup.get(group)
    return _AGLinearFn.apply(x.contiguous(), rank, n, sg, tuple(OF._holder(w) for w in weights), lead, *weights)


def linear_rs(a, w, rank, n, group):
    """Row-parallel projection whose partial sums are reduce-scattered over the rows: ``[T / n, N]`` of the sum."""
    sg = SymmGroup.get(group)
    return _LinearRSFn.apply(a.contiguous(), w, rank, n, sg, OF._holder(w))


class _GradAllReduceFn(torch.autograd.Function):
    """Identity on a parameter that every rank of ``group`` holds; its gradient is summed over the group.  With
    sequence-sharded activations a replicated weight (a norm's scale) sees only this rank's rows."""

    @staticmethod
    def forward(ctx, w, group):
        ctx.group = group
        return w.view_as(w)

    @staticmethod
    def backward(ctx, g):
        import torch.distributed as dist
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


def replicated_weight(w, group):
    return _GradAllReduceFn.apply(w, group)
