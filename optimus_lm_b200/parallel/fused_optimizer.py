"""Optimizer step with the collectives fused into the update kernel.

For every sharded parameter family of a flat-buffer optimizer (``optimizers.py``) the flat
gradient and parameter buffers are moved into symmetric memory.  One kernel
(``csrc/comm_p2p.cu: rs_adamw_kernel``) then does, for the shard this rank owns:

    load the shard of every peer's gradient buffer over NVLink -> sum in fp32 (reduce-scatter; with NVLS one
    ``multimem.ld_reduce`` per 16 bytes does the sum in the switch, and one ``multimem.st`` the all-gather below)
    -> scale by 1/N -> norm partial -> AdamW on the fp32 master / moments
    -> store the updated bf16 parameters into every peer's parameter buffer (all-gather); the attention
       projections and the LM head are left out of this push: every rank fetches the other ranks' parts of such a
       weight inside the first GEMM that consumes it in the next forward (``LazyWeight``), where the transfer
       runs underneath the tiles

which replaces ``reduce_scatter_tensor`` + division + ``get_total_norm`` + ~12 elementwise kernels
+ ``all_gather_into_tensor`` of the reference (optimus/optimizers.py:354-494, 704-928).  Two
device-side barriers bracket the kernel (gradients complete everywhere / parameters written and
gradients consumed everywhere).

Clipping needs the global norm before the update.  While clipping is inactive (the default
"delayed clipping" covers the first ``warmup_steps`` optimizer steps) the norm is a by-product of
the single fused pass; once it is active a first pass computes only the norm partials and the
fused pass follows with the coefficient, at the cost of reading the peers' gradients twice.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional

import torch

from ..ops import functional as OF
from ..ops._ext import extension
from .symm import SymmGroup, SymmTensor, peer_access_ok


def use_multimem(group_size: int) -> bool:
    """NVLS for the optimizer's reduce-scatter and all-gather: ``OLB_MULTIMEM=1`` switches it on, the default is plain
    peer loads and stores.  Measured for 512 Mi parameters (reduce-scatter + AdamW + all-gather, one kernel): 2 ranks
    2.69 ms with NVLS against 1.71 ms plain (the in-switch reduction moves both copies over the links where plain
    loads move one); 8 ranks 3.16 ms against 2.89 ms with one reduced load in flight per thread."""
    return os.environ.get("OLB_MULTIMEM", "0") == "1" and group_size >= 2


_LAZY_NAME = re.compile(r"(^|\.)(q_proj|k_proj|v_proj|o_proj)\.weight$|^lm_head\.weight$")


def lazy_gather_enabled() -> bool:
    """``OLB_PARAM_AG=gemm``: the all-gather of the attention projections' and the LM head's updated weights is left to
    the first GEMM that consumes them; ``push`` (default): the update kernel stores every parameter into every rank's
    buffer.  Measured on OLMoE-1B-7B, expert parallel: 205.2 ms/step against 201.1 ms at 8 GPUs, 188.6 against 186.5 at
    2 GPUs - the 65 gather launches per step cost more than the 1.4 ms of pushes they take out of the update kernel."""
    return os.environ.get("OLB_PARAM_AG", "push") == "gemm"


class LazyWeight:
    """A weight matrix whose all-gather after a sharded optimizer step happens inside the first GEMM that consumes it.

    After the step only the owner of each shard holds the updated values of its part of ``w`` (``segments[r]`` = the
    element range of ``w`` that is current only on rank ``r``).  ``ops.functional.linear`` asks ``gather_gemm`` for the
    forward product while ``stale`` is set: extra warps of that launch copy the segments in over NVLink while tiles whose
    rows of ``w`` are complete already run.  Any other reader calls ``materialize`` first (a plain peer copy)."""

    __slots__ = ("w_ptrs", "segments", "rank", "stale", "numel")

    def __init__(self, w_ptrs, segments, rank, numel):
        self.w_ptrs, self.segments, self.rank, self.numel = list(w_ptrs), list(segments), rank, numel
        self.stale = False

    def _flat_segments(self):
        out = []
        for lo, hi in self.segments:
            out += [lo, hi]
        return out

    def gather_gemm(self, x2, w, y2) -> bool:
        """``y2 = x2 @ w.T`` with the gather inside; False when the shape is not one the fused launch takes."""
        M, K = x2.shape
        N = w.shape[0]
        if not (w.is_contiguous() and M >= 256 and K % 64 == 0 and (N % 256 == 0 or N >= 2048)
                and os.environ.get("OLB_GEMM_PAIR", "1") != "0"):
            return False
        extension().gemm_b_gather(x2, w, y2, M, N, K, self.w_ptrs, self._flat_segments(), self.rank,
                                  OF.stage_flags(w.device, N), OF.status_word(w.device))
        self.stale = False
        return True

    def materialize(self, w):
        C = extension()
        flat = w.view(-1)
        for r, (lo, hi) in enumerate(self.segments):
            if hi > lo:
                C.peer_copy(self.w_ptrs[r] + 2 * lo, flat[lo:hi], 2 * (hi - lo))
        self.stale = False


def slices_aligned(families) -> bool:
    """The fused kernel moves 16-byte vectors of bf16 gradients and parameters and float4 vectors of the fp32 state:
    every slice a rank owns must start at, and cover, a multiple of 8 elements, in the flat buffer and in the state."""
    for fam in families:
        for sl in fam.slices:
            lo, _ = fam._part_range(sl)
            if sl.part % 8 or lo % 8 or sl.state_start % 8:
                return False
    return True


class FusedShardedStep:
    def __init__(self, opt):
        self.opt = opt
        self.device = opt.device
        self.sym: Dict[int, Dict[str, SymmTensor]] = {}
        self.groups: Dict[int, SymmGroup] = {}
        for fi, fam in enumerate(opt.families):
            if not (fam.spec.sharded and fam.spec.num_shards > 1):
                continue
            sg = SymmGroup.get(fam.spec.group)
            self.groups[fi] = sg
            gp = sg.empty((fam.flat_size,), fam.dtype)
            gp.local.copy_(fam.flat_param)
            gg = sg.empty((fam.flat_size,), fam.dtype, zero=True)
            gg.local.copy_(fam.flat_grad)
            fam.flat_param, fam.flat_grad = gp.local, gg.local
            for p, start, size in zip(fam.spec.params, fam.param_start_inds, fam.param_sizes):
                p.data = fam.flat_param[start:start + size].view_as(p.data)
                p.grad = fam.flat_grad[start:start + size].view_as(p.data)
            self.sym[fi] = {"param": gp, "grad": gg}
        if len(opt.families) == 1:
            opt._alias_single()
        else:
            opt._alias_pair()
        self.lazy: Dict[int, List] = {}          # family -> [(param, LazyWeight)]
        self.local_only: Dict[int, torch.Tensor] = {}
        if lazy_gather_enabled():
            self._setup_lazy(opt)
        torch.cuda.synchronize()

    def _setup_lazy(self, opt):
        """Pick the weights whose all-gather moves into their first consuming GEMM: 2D projections that
        ``ops.functional.linear`` consumes (attention q / k / v / o, LM head) of families with one sharded slice."""
        names = {id(p): n for n, p in opt.model.named_parameters()} if getattr(opt, "model", None) is not None else {}
        for fi, fam in enumerate(opt.families):
            if fi not in self.sym or len(fam.slices) != 1:
                continue
            sg = self.groups[fi]
            n, part = sg.size, fam.slices[0].part
            ranges, entries = [], []
            for p, start, size in zip(fam.spec.params, fam.param_start_inds, fam.param_sizes):
                name = names.get(id(p), "")
                if p.dim() != 2 or not _LAZY_NAME.search(name) or start % 8 or size % 8 or p.shape[1] % 64:
                    continue
                if not (p.shape[0] % 256 == 0 or p.shape[0] >= 2048):
                    continue
                segs = []
                for r in range(n):   # the part of [start, start + size) that rank r owns, relative to the weight
                    lo, hi = max(start, r * part), min(start + size, (r + 1) * part)
                    segs.append((lo - start, hi - start) if (hi > lo and r != sg.rank) else (0, 0))
                if not any(hi > lo for lo, hi in segs):
                    continue             # the whole weight is this rank's own
                lw = LazyWeight(self.sym[fi]["param"].offset_ptrs(start), segs, sg.rank, size)
                p._olb_lazy = lw
                entries.append((p, lw))
                ranges.append((start, start + size))
            if entries:
                self.lazy[fi] = entries
                self.local_only[fi] = torch.tensor(sorted(ranges), dtype=torch.int64, device=self.device)

    def materialize(self):
        """Bring every weight whose gather is still pending up to date (before anything but a forward GEMM reads the
        parameters: checkpoints, evaluation code that bypasses ``ops.functional.linear``)."""
        for entries in self.lazy.values():
            for p, lw in entries:
                if lw.stale:
                    lw.materialize(p.data)

    @staticmethod
    def try_create(opt) -> Optional["FusedShardedStep"]:
        if opt.dtype != torch.bfloat16 or opt.skip_optimizer_step:
            return None
        if opt.opt_use_allreduce_for_param_gather:
            return None
        fams = [f for f in opt.families if f.spec.sharded and f.spec.num_shards > 1]
        if not fams:
            return None
        if any(f.spec.group in (None, -1) for f in fams):
            return None
        if hasattr(opt, "_replicated_param_ranges") and (opt.expert_parallelism > 1 or opt.tensor_parallelism > 1):
            return None  # the "shard" class weights replicated gradients in the norm; keep the NCCL path
        if any(f.spec.num_shards > 16 for f in fams):
            return None
        if not slices_aligned(fams):
            return None  # e.g. sub-sharded chunks at DP 3, 5, 6, 7: the NCCL path has no alignment rule
        if not all(peer_access_ok(f.spec.group) for f in fams):
            return None
        return FusedShardedStep(opt)

    def usable(self, opt) -> bool:
        return True

    def _multicast(self, fi):
        """Multicast addresses of a family's gradient and parameter buffers, or ``(0, 0)``: NVLS is used when the
        symmetric-memory provider bound both buffers to a multicast object (``OLB_MULTIMEM=0`` keeps plain peer
        loads and stores; tests in which a rank may leave must use that, as the pool's notes on NVLS say)."""
        if not use_multimem(self.groups[fi].size):
            return 0, 0
        g, p = self.sym[fi]["grad"].multicast_ptr, self.sym[fi]["param"].multicast_ptr
        return (g, p) if g and p else (0, 0)

    @torch.no_grad()
    def step(self, opt):
        C = extension()
        beta1, beta2 = opt.defaults["betas"]
        eps, wd = opt.defaults["eps"], opt.defaults["weight_decay"]
        lr = opt.param_groups[0]["lr"]
        step_no = opt.step_id + 1
        clipping = opt._clipping_active()
        total_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        early_sq = opt._join_early_updates()      # layers of unreduced families already updated under the backward
        if early_sq is not None:
            total_sq.add_(early_sq)

        for sg in {id(g): g for g in self.groups.values()}.values():
            sg.barrier(8)  # every rank's gradients are complete

        def run(mode, clip_coef):
            for fi, fam in enumerate(opt.families):
                scale = 1.0 / fam.spec.grad_divisor
                for sl in fam.slices:
                    s0, s1 = sl.state_start, sl.state_start + sl.part
                    if fi in self.sym:
                        lo, _ = fam._part_range(sl)
                        nb = C.rs_adamw_blocks(sl.part)
                        partial = torch.empty(nb, dtype=torch.float32, device=self.device)
                        mcg, mcp = self._multicast(fi)
                        C.rs_adamw(self.sym[fi]["grad"].ptrs, self.sym[fi]["param"].ptrs, lo, fam.master[s0:s1],
                                   fam.exp_avg[s0:s1], fam.exp_avg_sq[s0:s1], lr, beta1, beta2, eps, wd, step_no, scale,
                                   clip_coef, partial, mode, opt.skip_optimizer_step_weight_update, mcg, mcp,
                                   self.local_only.get(fi), self.groups[fi].rank)
                        if clip_coef is None:
                            total_sq.add_(partial.sum())
                    else:
                        g, pp = fam.grad_part(sl), fam.param_part(sl)
                        for lo, hi in opt._pending_ranges(fam, sl):
                            if clip_coef is None and mode == 0:
                                OF.sum_of_squares(g[lo:hi], scale, out=total_sq, accumulate=True)
                            if mode == 1:   # without clipping the norm is a by-product of the update's pass
                                OF.adamw_step(g[lo:hi], fam.master[s0 + lo:s0 + hi], fam.exp_avg[s0 + lo:s0 + hi],
                                              fam.exp_avg_sq[s0 + lo:s0 + hi], pp[lo:hi], lr, beta1, beta2, eps, wd,
                                              step_no, grad_scale=scale, clip_coef=clip_coef,
                                              skip_weight_update=opt.skip_optimizer_step_weight_update,
                                              norm_out=total_sq if clip_coef is None else None)

        if clipping:
            run(0, None)
            grad_norm = opt._global_norm(total_sq).reshape(())
            clip = torch.clamp(opt.max_grad_norm / (grad_norm + 1e-6), max=1.0).reshape(1).float()
            run(1, clip)
        else:
            run(1, None)
            grad_norm = opt._global_norm(total_sq).reshape(())

        for sg in {id(g): g for g in self.groups.values()}.values():
            sg.barrier(9)  # parameters written everywhere, gradients consumed everywhere
        if not opt.skip_optimizer_step_weight_update:
            for entries in self.lazy.values():      # their other ranks' parts arrive with the next forward's GEMMs
                for _p, lw in entries:
                    lw.stale = True
        return grad_norm
