"""Router auxiliary loss split into per-stage parts, for pipeline parallelism.

The reference computes the *global* load-balance loss under PP by shipping the concatenated
router logits of all earlier stages forward (up to 32 MiB per hop) and their gradients backward
(optimus/training.py:101-190).  The loss only depends on two per-expert sums,

    aux = E * sum_e f_e * P_e,   f_e = count_e / N,   P_e = sum_tokens p_te / N,   N = tokens x layers,

and its gradient w.r.t. any logit only needs the global ``f``.  So each stage sends its running
sums (``2E+2`` floats) forward with the activation, the last stage forms the loss value and the
global ``f`` and sends ``f`` (``E`` floats) backward with the activation gradient, and every
stage back-propagates ``aux_partial`` - the loss with ``f`` held constant - through its own
layers.  The sum of the stages' partial values is the global loss and the gradients are
identical to the reference's.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F

from . import functional as OF
from ._ext import extension


def stats_width(num_experts: int) -> int:
    """Length of the statistics vector: counts[E], prob sums[E], sum lse^2, layer-level partial."""
    return 2 * num_experts + 2


@torch.no_grad()
def router_stats(logits_list: Sequence[torch.Tensor], idx_list, stats_list, num_experts: int, top_k: int) -> torch.Tensor:
    """Per-layer statistics ``[L, 2E+1]`` (counts, prob sums, sum of lse^2), from the router kernel
    when available, else recomputed from the logits."""
    rows = []
    for i, lg in enumerate(logits_list):
        st = stats_list[i] if stats_list is not None else None
        if st is not None:
            rows.append(st[:2 * num_experts + 1].float())
            continue
        lf = lg.float()
        p = F.softmax(lf, dim=-1)
        idx = idx_list[i].long() if idx_list is not None and idx_list[i] is not None else torch.topk(p, top_k, dim=-1)[1]
        cnt = torch.bincount(idx.reshape(-1), minlength=num_experts).float()
        rows.append(torch.cat([cnt, p.sum(0), torch.logsumexp(lf, -1).pow(2).sum().reshape(1)]))
    return torch.stack(rows, dim=0)


class _AuxPartialFn(torch.autograd.Function):
    """value = sum_l [ a_scale * sum_e f_le * Psum_le + z_scale * lse2_l ] with ``f`` constant;
    gradient via the router backward kernel."""

    @staticmethod
    def forward(ctx, f, stats, a_scale, z_scale, n_layers, *tensors):
        logits, idxs = tensors[:n_layers], tensors[n_layers:2 * n_layers]
        E = f.shape[-1]
        value = (a_scale * (f * stats[:, E:2 * E]).sum() + z_scale * stats[:, 2 * E].sum()).reshape(())
        ctx.save_for_backward(f, *logits, *idxs)
        ctx.cfg = (a_scale, z_scale, n_layers)
        return value

    @staticmethod
    def backward(ctx, g):
        a_scale, z_scale, L = ctx.cfg
        saved = ctx.saved_tensors
        f, logits, idxs = saved[0], saved[1:1 + L], saved[1 + L:1 + 2 * L]
        C = extension()
        g = g.to(torch.float32).reshape(1).contiguous()
        grads = []
        for l in range(L):
            d = torch.empty_like(logits[l])
            C.router_bwd(logits[l], idxs[l], None, False, f[l].contiguous(), g, a_scale, z_scale, d)
            grads.append(d)
        return (None,) * 5 + tuple(grads) + (None,) * L


def aux_partial(logits_list, idx_list, stats, f, *, a_scale: float, z_scale: float):
    """Differentiable partial loss of this stage's layers.

    ``stats`` ``[L, 2E+1]`` from ``router_stats``; ``f`` ``[L, E]`` (constant) - the same global
    vector in every row for the global loss, the per-layer local fractions for the layer-level
    loss.  ``a_scale = coef * E / N_norm`` and ``z_scale = z_coef / (T * L_total)``."""
    L = len(logits_list)
    kernel = (idx_list is not None and all(i is not None and i.dtype == torch.int32 for i in idx_list)
              and OF._kernel_ok(*logits_list))
    if kernel:
        return _AuxPartialFn.apply(f.float().contiguous(), stats, a_scale, z_scale, L, *logits_list, *idx_list)
    total = 0.0
    for l, lg in enumerate(logits_list):
        lf = lg.float()
        p = F.softmax(lf, dim=-1)
        total = total + a_scale * (p.sum(0) * f[l].float()).sum()
        if z_scale:
            total = total + z_scale * torch.logsumexp(lf, -1).pow(2).sum()
    return total
