"""Expert-parallel MoE with the token exchange inside the grouped GEMM kernels.

The reference all-gathers every token, routing weight and index over the EP group, runs the
local experts over all gathered tokens and reduce-scatters a ``[EP*T, H]`` buffer
(optimus/models/olmoe/modeling_olmoe.py:305-341, optimus/models/common/moe.py:477-608).  Here no
collective library call is on the path.  Per layer and direction there are two device-side
barriers and these launches:

* publish   - the token rows are copied into this rank's symmetric buffer and the ``[T, K]`` routing
  indices / weights are stored into every peer's gathered arrays by a small kernel (all-gather by
  stores, ~1 MB); barrier;
* dispatch + gate|up + activation - one grouped tcgen05 GEMM launch: extra warps of every CTA fetch the
  routed token rows from their owners over NVLink straight into the expert-grouped operand and count them
  per 128-row block, the TMA producer starts on a block as soon as it is complete, and the epilogue writes
  ``gate | up`` and the routing-weighted SwiGLU;
* down + combine - the down projection's launch sends every finished output row to slot ``[token, k]`` of
  the token owner's receive buffer with stores over NVLink while its later tiles run; barrier; the owner sums
  its K slots from local memory in fp32.

The backward pass mirrors it: the output gradients are gathered inside the down projection's input-gradient
launch, the gate/up input gradient is one K-concatenated launch that pushes its rows back to the tokens'
owners, and the barrier + sum run on a side stream underneath the three weight-gradient GEMMs.  All waits
are bounded and report into the device status word.
"""
from __future__ import annotations

import torch

from ..ops import functional as OF
from ..ops._ext import extension
from .symm import SymmGroup


def _scratch(sg: SymmGroup, name: str, shape, dtype) -> torch.Tensor:
    t = getattr(sg, name, None)
    if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
        t = torch.empty(shape, dtype=dtype, device=sg.device)
        setattr(sg, name, t)
    return t


class _FusedEPMoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topk_w, topk_idx, wg, wu, wd, sg: SymmGroup, e_start, cap, exact, holders=(None, None, None)):
        C = extension()
        ctx.holders = holders
        n, rank = sg.size, sg.rank
        T, H = x.shape
        E_loc, I, _ = wg.shape
        K = topk_idx.shape[1]
        topk_idx = topk_idx.contiguous()
        topk_w = topk_w.contiguous().float()
        status = OF.status_word(x.device)

        # publish: token rows into this rank's symmetric buffer, routing metadata into every peer's gathered arrays
        xs = sg.named("ep_rows", (T, H), x.dtype)
        xs.local.copy_(x)
        idx_all = sg.named("ep_idx", (n * T, K), torch.int32)
        w_sym = sg.named("ep_w", (n * T, K), torch.float32)
        C.ep_publish_meta(idx_all.ptrs, w_sym.ptrs, topk_idx, topk_w, rank * T * K)
        sg.barrier(0)

        index = OF.MoEIndex(idx_all.local, e_start, E_loc, cap, exact)
        w_all = w_sym.local.clone()        # the backward needs it; the symmetric copy is rewritten by the next layer
        # dispatch + gate|up + activation: one launch (rows arrive over NVLink while the first tiles run)
        xp, h, act = OF.grouped_gateup_swiglu(xs.ptrs, H, T, w_all, wg, wu, index)
        # down projection with the combine's transport: finished rows go to slot [token, k] of the token owner's
        # receive buffer from inside the kernel
        rows = index.rows
        ys = torch.empty((rows, H), dtype=x.dtype, device=x.device)
        recv = sg.named("ep_recv", (T, K, H), x.dtype)
        C.gemm_ep_push(act, wd.view(E_loc * H, I), ys, recv.ptrs, index.meta, index.src_of, index.k_of, rows, H, I, H,
                       E_loc, T, K, rank, OF.stage_flags(x.device, rows), status, pair_rows=index.pair)
        del ys
        sg.barrier(1)
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
        C.sum_slots(recv.local, out)

        ctx.save_for_backward(xp, h, act, w_all, wg, wu, wd, topk_idx)
        ctx.index, ctx.sg = index, sg
        ctx.dims = (T, H, I, E_loc, K)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = extension()
        xp, h, act, w_all, wg, wu, wd, topk_idx = ctx.saved_tensors
        index, sg = ctx.index, ctx.sg
        T, H, I, E_loc, K = ctx.dims
        n, rank = sg.size, sg.rank
        rows = index.rows
        status = OF.status_word(dout.device)

        ds = sg.named("ep_rows", (T, H), dout.dtype)
        ds.local.copy_(dout)
        sg.barrier(2)

        hg, hu, hd = ctx.holders
        # Critical path first: the input-gradient chain up to the rows that go back to the tokens' owners.
        # dispatch of the output gradients inside the down projection's input-gradient launch
        # ... with the activation's backward in its epilogue (d(act) never goes to memory)
        dwt = sg.named("ep_dw", (n * T, K), torch.float32)
        dwt.local.zero_()
        dyp, dh = OF.grouped_down_dgrad_swiglu_bwd(ds.ptrs, H, T, wd, h, w_all, index, dwt.local)
        # input gradient of gate and up in one K-concatenated launch that also sends every finished row to slot
        # [token, k] of the token owner's receive buffer
        dxp = torch.empty((rows, H), dtype=dout.dtype, device=dout.device)
        recv = sg.named("ep_recv", (T, K, H), dout.dtype)
        C.gemm_ep_push(dh, wg.view(E_loc * I, H), dxp, recv.ptrs, index.meta, index.src_of, index.k_of, rows, H, 2 * I, I,
                       E_loc, T, K, rank, OF.stage_flags(dout.device, rows), status, True, wu.view(E_loc * I, H), I,
                       index.pair)
        del dxp
        dx = torch.empty((T, H), dtype=dout.dtype, device=dout.device)
        dtopk = torch.empty((T, K), dtype=torch.float32, device=dout.device)
        # ... then the barrier and the owner's sum run on a side stream underneath the three weight-gradient GEMMs,
        # which nothing downstream waits for.
        main = torch.cuda.current_stream()
        side = sg.side_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(side):
            side.wait_event(ready)
            sg.barrier(3)
            C.sum_slots(recv.local, dx)
            C.ep_pull_dweights(dwt.ptrs, topk_idx, rank, E_loc, dtopk)
            done = torch.cuda.Event()
            done.record(side)
        dwd = OF.grouped_linear_wgrad(dyp, act, index, H, I, hd) if ctx.needs_input_grad[5] else None
        del dyp
        dwg = OF.grouped_linear_wgrad(dh[:, :I], xp, index, I, H, hg) if ctx.needs_input_grad[3] else None
        dwu = OF.grouped_linear_wgrad(dh[:, I:], xp, index, I, H, hu) if ctx.needs_input_grad[4] else None
        main.wait_event(done)
        return dx, dtopk, None, dwg, dwu, dwd, None, None, None, None, None


def fused_ep_moe(block, x, w, idx):
    """MoE forward of ``block`` (a ``SparseMoeBlock``-like module with merged experts) for the
    local tokens ``x [T, H]`` with routing weights ``w [T, K]`` and global expert ids ``idx``."""
    pmap = block.pmap
    sg = SymmGroup.get(pmap.ep_group)
    wg, wu, wd = block.experts.weights()
    T = x.shape[0]
    ep = pmap.expert_parallelism
    # capacity factor 0 (default): index arrays for the worst case, activation buffers sized from the routed counts
    # (no routed pair can be dropped); > 0: everything sized for that multiple of the balanced share, no host read,
    # and a rank that receives more raises ST_OVERFLOW in the device status word
    exact = not block.capacity_factor
    cap = OF.moe_capacity_rows(T * ep, block.num_experts_per_tok, block.num_experts_per_rank, ep, block.capacity_factor)
    return _FusedEPMoEFn.apply(x.contiguous(), w.float(), idx, wg, wu, wd, sg, block.expert_start_idx, cap, exact,
                               (OF._holder(wg), OF._holder(wu), OF._holder(wd)))
