"""Expert-parallel MoE with the token exchange fused into the permutation kernels.

The reference all-gathers every token, routing weight and index over the EP group, runs the
local experts over all gathered tokens and reduce-scatters a ``[EP*T, H]`` buffer
(optimus/models/olmoe/modeling_olmoe.py:305-341, optimus/models/common/moe.py:477-608).  Here only
the routing metadata (``[T, K]`` indices and weights, ~1 MB) is all-gathered with NCCL; the token
rows themselves never go through a collective:

* dispatch  - each rank builds the expert-grouped row layout of *its* experts from the gathered
  indices and its gather kernel pulls exactly the routed rows from the owners' activation buffers
  over NVLink, straight into the grouped-GEMM operand (dispatch all-to-all + permutation, one
  kernel, no staging copy of all tokens);
* experts   - grouped tcgen05 GEMMs with the routing weight folded into the activation;
* combine   - forward: the down projection's GEMM kernel sends every finished output row to the owner of
  its token with stores over NVLink from extra warps of each CTA, while its later tiles are still running
  (combine all-to-all inside the grouped GEMM); after a barrier the owner sums the K slots of each token from
  local memory in fp32.  Backward: each rank's combine kernel pulls the K input-gradient rows of each of its
  tokens from the owners' buffers on a side stream underneath the weight-gradient GEMMs.

The backward pass is the mirror image (gather of output gradients, combine of input gradients,
pull of the routing-weight gradients).  Two device-side barriers per direction order the buffer
reuse; all waits are bounded.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops._ext import extension
from .symm import SymmGroup


def _all_gather_rows(t: torch.Tensor, n: int, group) -> torch.Tensor:
    out = torch.empty((n * t.shape[0],) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out, t.contiguous(), group=group)
    return out


def _parts(E_loc: int) -> int:
    """Groups of local experts the dispatch is pipelined over (OLB_EP_PARTS, default 4, 1 = no pipelining)."""
    return max(1, min(int(os.environ.get("OLB_EP_PARTS", "4")), E_loc))


def _push_combine(n: int) -> bool:
    """Forward combine as stores from the down projection's kernel instead of pulls after it.  ``OLB_EP_PUSH`` = 1 / 0
    forces it on / off; by default it is used from 4 ranks on: with 2 ranks half of a token's rows are local and the
    pull (205.4 ms/step) beats the push and its extra pass through the receive buffer (208.8 ms/step)."""
    v = os.environ.get("OLB_EP_PUSH", "auto")
    return n >= 4 if v == "auto" else v != "0"


def _scratch(sg: SymmGroup, name: str, shape, dtype) -> torch.Tensor:
    t = getattr(sg, name, None)
    if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
        t = torch.empty(shape, dtype=dtype, device=sg.device)
        setattr(sg, name, t)
    return t


def _slot_ids(sg: SymmGroup, T: int, K: int) -> torch.Tensor:
    t = getattr(sg, "_ep_slot_ids", None)
    if t is None or tuple(t.shape) != (T, K):
        t = sg._ep_slot_ids = torch.arange(T * K, dtype=torch.int32, device=sg.device).view(T, K)
    return t


def _pipelined_gather(sg: SymmGroup, peer_ptrs, T, index, out, parts: int):
    """Pull the routed rows of ``out`` from their owners in ``parts`` groups of experts on the side stream.
    Returns ``(ranges, events)``: the consumer waits for ``events[p]`` on its own stream before touching the row
    blocks ``ranges[p]``, so the first experts' GEMMs run while the later experts' rows still cross NVLink."""
    C = extension()
    if parts <= 1:
        C.ep_gather_rows(peer_ptrs, T, index.src_of, index.meta, out, None)
        return None, None
    ranges = index.part_ranges(parts)
    main, side = torch.cuda.current_stream(), sg.side_stream()
    start = torch.cuda.Event()
    start.record(main)
    events = []
    with torch.cuda.stream(side):
        side.wait_event(start)
        for p in range(parts):
            C.ep_gather_rows(peer_ptrs, T, index.src_of, index.meta, out, ranges[p])
            ev = torch.cuda.Event()
            ev.record(side)
            events.append(ev)
    return ranges, events


class _FusedEPMoEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, topk_w, topk_idx, wg, wu, wd, sg: SymmGroup, e_start, cap, holders=(None, None, None)):
        C = extension()
        ctx.holders = holders
        n, rank = sg.size, sg.rank
        T, H = x.shape
        E_loc, I, _ = wg.shape
        K = topk_idx.shape[1]
        topk_idx = topk_idx.contiguous()
        topk_w = topk_w.contiguous().float()

        xs = sg.named("ep_rows", (T, H), x.dtype)
        xs.local.copy_(x)
        idx_all = _all_gather_rows(topk_idx, n, sg.group)
        w_all = _all_gather_rows(topk_w, n, sg.group)
        sg.barrier(0)

        index = OF.MoEIndex(idx_all, e_start, E_loc, cap)
        xp = torch.empty((cap, H), dtype=x.dtype, device=x.device)
        h = torch.empty((cap, 2 * I), dtype=x.dtype, device=x.device)
        ranges, events = _pipelined_gather(sg, xs.ptrs, T, index, xp, _parts(E_loc))
        main = torch.cuda.current_stream()
        for p in range(len(events) if events else 1):
            r = None
            if events:
                main.wait_event(events[p])
                r = ranges[p]
            OF.grouped_linear_fwd(xp, wg, index, out=h[:, :I], blk_range=r)
            OF.grouped_linear_fwd(xp, wu, index, out=h[:, I:], blk_range=r)
        act = torch.empty((cap, I), dtype=x.dtype, device=x.device)
        C.swiglu_rowscale_fwd(h[:, :I], h[:, I:], index.src_of, index.k_of, w_all, index.meta, act)
        rt = sg.named("ep_rowof", (n * T, K), torch.int32)
        rt.local.copy_(index.row_of)
        rows = torch.empty((T, K), dtype=torch.int32, device=x.device)
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
        if _push_combine(n):
            # combine all-to-all inside the down projection: its extra warps send every finished row to the owner of
            # its token (slot [token, k] of the owner's receive buffer) while later tiles run
            ys = _scratch(sg, "_ep_ys", (cap, H), x.dtype)
            recv = sg.named("ep_recv", (T, K, H), x.dtype)
            C.gemm_ep_push(act, wd.view(E_loc * H, I), ys, recv.ptrs, index.meta, index.src_of, index.k_of, cap, H, I, H,
                           E_loc, T, K, rank, _scratch(sg, "_ep_flags", (cap // 128 + 1,), torch.int32),
                           OF.status_word(x.device))
            sg.barrier(1)
            C.ep_resolve_rows(rt.ptrs, topk_idx, rank, E_loc, rows)
            slots = torch.where(rows >= 0, _slot_ids(sg, T, K), -1)      # pairs dropped at the owner stay out of the sum
            C.ep_combine([recv.local.data_ptr()] * n, slots, topk_idx, E_loc, out)
        else:
            ys = sg.named("ep_out", (cap, H), x.dtype)
            OF.grouped_linear_fwd(act, wd, index, out=ys.local)
            sg.barrier(1)
            C.ep_resolve_rows(rt.ptrs, topk_idx, rank, E_loc, rows)
            C.ep_combine(ys.ptrs, rows, topk_idx, E_loc, out)

        ctx.save_for_backward(xp, h, act, w_all, wg, wu, wd, rows, topk_idx)
        ctx.index, ctx.sg = index, sg
        ctx.dims = (T, H, I, E_loc, K, cap)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = extension()
        xp, h, act, w_all, wg, wu, wd, rows, topk_idx = ctx.saved_tensors
        index, sg = ctx.index, ctx.sg
        T, H, I, E_loc, K, cap = ctx.dims
        n, rank = sg.size, sg.rank

        ds = sg.named("ep_rows", (T, H), dout.dtype)
        ds.local.copy_(dout)
        sg.barrier(2)

        dyp = torch.empty((cap, H), dtype=dout.dtype, device=dout.device)
        dact = torch.empty((cap, I), dtype=dout.dtype, device=dout.device)
        hg, hu, hd = ctx.holders
        # Critical path first: the input-gradient chain up to the rows the other ranks will pull ...
        ranges, events = _pipelined_gather(sg, ds.ptrs, T, index, dyp, _parts(E_loc))
        main = torch.cuda.current_stream()
        for p in range(len(events) if events else 1):
            r = None
            if events:
                main.wait_event(events[p])
                r = ranges[p]
            OF.grouped_linear_dgrad(dyp, wd, index, out=dact, blk_range=r)
        dh = torch.empty_like(h)
        dwt = sg.named("ep_dw", (n * T, K), torch.float32)
        dwt.local.zero_()
        C.swiglu_rowscale_bwd(dact, h[:, :I], h[:, I:], index.src_of, index.k_of, w_all, index.meta, dh[:, :I],
                              dh[:, I:], dwt.local)
        del dact
        dxp = sg.named("ep_out", (cap, H), dout.dtype)
        if I % 64 == 0:
            OF.grouped_linear_dgrad_pair(dh, wg, wu, index, out=dxp.local)
        else:
            OF.grouped_linear_dgrad(dh[:, :I], wg, index, out=dxp.local)
            OF.grouped_linear_dgrad(dh[:, I:], wu, index, out=dxp.local, accumulate=True)
        dx = torch.empty((T, H), dtype=dout.dtype, device=dout.device)
        dtopk = torch.empty((T, K), dtype=torch.float32, device=dout.device)
        # ... then the combine all-to-all (NVLink-bound pulls) runs on a side stream underneath the three
        # weight-gradient GEMMs, which nothing downstream waits for.
        main = torch.cuda.current_stream()
        side = sg.side_stream()
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(side):
            side.wait_event(ready)
            sg.barrier(3)
            C.ep_combine(dxp.ptrs, rows, topk_idx, E_loc, dx)
            C.ep_pull_dweights(dwt.ptrs, topk_idx, rank, E_loc, dtopk)
            done = torch.cuda.Event()
            done.record(side)
        dwd = OF.grouped_linear_wgrad(dyp, act, index, H, I, hd) if ctx.needs_input_grad[5] else None
        del dyp
        dwg = OF.grouped_linear_wgrad(dh[:, :I], xp, index, I, H, hg) if ctx.needs_input_grad[3] else None
        dwu = OF.grouped_linear_wgrad(dh[:, I:], xp, index, I, H, hu) if ctx.needs_input_grad[4] else None
        main.wait_event(done)
        return dx, dtopk, None, dwg, dwu, dwd, None, None, None, None


def fused_ep_moe(block, x, w, idx):
    """MoE forward of ``block`` (a ``SparseMoeBlock``-like module with merged experts) for the
    local tokens ``x [T, H]`` with routing weights ``w [T, K]`` and global expert ids ``idx``."""
    pmap = block.pmap
    sg = SymmGroup.get(pmap.ep_group)
    wg, wu, wd = block.experts.weights()
    T = x.shape[0]
    cap = OF.moe_capacity_rows(T * pmap.expert_parallelism, block.num_experts_per_tok, block.num_experts_per_rank,
                               pmap.expert_parallelism, block.capacity_factor)
    return _FusedEPMoEFn.apply(x.contiguous(), w.float(), idx, wg, wu, wd, sg, block.expert_start_idx, cap,
                               (OF._holder(wg), OF._holder(wu), OF._holder(wd)))
