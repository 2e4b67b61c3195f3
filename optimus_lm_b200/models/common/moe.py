"""Sparse mixture-of-experts block (router + expert-parallel dispatch + experts + combine).

Covers the reference's baseline block (optimus/models/olmoe/modeling_olmoe.py:254-359) and
its FastMoE block with per-expert or merged weights (optimus/models/common/moe.py:379-632)
behind one module.  Parameter names follow the reference so checkpoints are interchangeable:
``gate.weight`` and either ``experts.{e}.{gate,up,down}_proj.weight`` or the merged
``experts.{gate_proj,up_proj}_merged_weight [E_loc, I, H]`` /
``experts.down_proj_merged_weight [E_loc, H, I]``.

Execution:

* routing: fp32 softmax -> top-k (-> renorm) in the router kernel, which also emits the
  statistics of the load-balance loss;
* expert parallelism, two interchangeable transports with the same math:
  - ``allgather`` (reference semantics): all-gather tokens / weights / indices over the EP
    group, run the local experts over all gathered tokens, reduce-scatter the partial
    outputs;
  - ``alltoall`` (default on GPUs): the fused dispatch/combine kernels of
    ``optimus_lm_b200.parallel.ep_alltoall`` push only the routed rows to the owning rank over
    NVLink peer memory and return the weighted expert outputs to the token's rank;
* experts: merged weights run the grouped tcgen05 GEMM pipeline of
  ``ops.functional.moe_experts``; per-expert ``nn.Linear`` weights run a loop over experts.
"""
from __future__ import annotations

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint as torch_activation_checkpoint

from ...ops import functional as OF
from .comms_ptfunctions import (forward_allgather_backward_reducescatter, forward_allgather_backward_split,
                                forward_identity_backward_synchronize, forward_reducescatter_backward_allgather,
                                forward_synchronize_backward_identity)


class ExpertMLP(nn.Module):
    """One SwiGLU expert with separate projections (reference ``OlmoeParallelMLP``)."""

    def __init__(self, hidden_size, intermediate_size):
        super().__init__()
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=False)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=False)

    def forward(self, x):
        return OF.linear(OF.swiglu(OF.linear(x, self.gate_proj.weight), OF.linear(x, self.up_proj.weight)),
                         self.down_proj.weight)


class MergedMLP(nn.Module):
    """All local experts in three stacked tensors (reference ``MergedMLP``, moe.py:379-405)."""

    def __init__(self, num_local_experts, hidden_size, intermediate_size):
        super().__init__()
        self.num_experts_per_rank = num_local_experts
        self.gate_proj_merged_weight = nn.Parameter(torch.empty((num_local_experts, intermediate_size, hidden_size)))
        self.up_proj_merged_weight = nn.Parameter(torch.empty((num_local_experts, intermediate_size, hidden_size)))
        self.down_proj_merged_weight = nn.Parameter(torch.empty((num_local_experts, hidden_size, intermediate_size)))

    def weights(self):
        return self.gate_proj_merged_weight, self.up_proj_merged_weight, self.down_proj_merged_weight


def _experts_loop(experts, x, topk_w, topk_idx, e_start):
    """Per-expert loop for the ``nn.ModuleList`` layout (the reference's baseline path)."""
    out = torch.zeros_like(x)
    tw = topk_w.to(x.dtype)
    idx = topk_idx.long()
    for le, expert in enumerate(experts):
        tok, kk = torch.where(idx == (e_start + le))
        if tok.numel() == 0:
            continue
        y = expert(x[tok]) * tw[tok, kk, None]
        out = out.index_add(0, tok, y.to(out.dtype))
    return out


class SparseMoeBlock(nn.Module):
    """Router + experts for ``num_experts`` experts of which this rank owns a contiguous block."""

    def __init__(self, config, pmap=None, *, merged: bool, hidden_size=None, intermediate_size=None,
                 num_experts=None, num_experts_per_tok=None):
        super().__init__()
        self.config = config
        self.pmap = pmap
        self.hidden_size = hidden_size or config.hidden_size
        self.intermediate_size = intermediate_size or config.intermediate_size
        self.num_experts = num_experts or config.num_experts
        self.num_experts_per_tok = num_experts_per_tok or config.num_experts_per_tok
        self.norm_topk_prob = config.norm_topk_prob
        self.output_router_logits = getattr(config, "output_router_logits", False)
        ep = pmap.expert_parallelism if pmap is not None else 1
        ep_ind = pmap.ep_ind if pmap is not None else 0
        self.num_experts_per_rank = self.num_experts // ep
        self.expert_start_idx = ep_ind * self.num_experts_per_rank
        self.expert_end_idx = self.expert_start_idx + self.num_experts_per_rank
        self.merged = merged

        self.gate = nn.Linear(self.hidden_size, self.num_experts, bias=False)
        if merged:
            self.experts = MergedMLP(self.num_experts_per_rank, self.hidden_size, self.intermediate_size)
        else:
            self.experts = nn.ModuleList(
                [ExpertMLP(self.hidden_size, self.intermediate_size) for _ in range(self.num_experts_per_rank)])

        self.use_activation_checkpointing_for_moe = bool(
            config.use_activation_checkpointing and (config.activation_checkpointing_level & 1))
        self.force_uniform_routing = getattr(config, "force_uniform_routing", False)
        self.mask = None
        self.use_allreduce_for_reducescatter = False
        self.capacity_factor = float(getattr(config, "moe_capacity_factor", 0.0))
        self.ep_transport = "alltoall" if getattr(config, "use_fused_ep_alltoall", True) else "allgather"
        self._a2a = None  # lazily built fused dispatcher
        self.last_router_stats = None
        self.last_router_indices = None
        self.last_router_logits = None

    # ------------------------------------------------------------------ routing
    def _route(self, hidden2d, sequence_length):
        router_logits = OF.linear(hidden2d, self.gate.weight)
        if self.force_uniform_routing:
            if self.mask is None or self.mask.shape[0] != router_logits.shape[0]:
                from ...utils import get_load_balanced_expert_mask
                ep_ind = self.pmap.ep_ind if self.pmap is not None else 0
                m = get_load_balanced_expert_mask(sequence_length, self.num_experts, self.num_experts_per_tok, ep_ind)
                reps = router_logits.shape[0] // sequence_length
                self.mask = (~m).repeat(reps, 1).to(router_logits.device)
            router_logits = router_logits.masked_fill(self.mask, float("-inf"))
        w, idx, stats = OF.router_softmax_topk(router_logits, self.num_experts_per_tok, self.norm_topk_prob,
                                               want_stats=self.output_router_logits)
        # the reference rounds the routing weights to the activation dtype before using them
        w = w.to(hidden2d.dtype)
        self.last_router_stats, self.last_router_indices, self.last_router_logits = stats, idx, router_logits
        return router_logits, w, idx

    # ------------------------------------------------------------------ experts
    def _local_experts(self, x, w, idx, cap=None, exact=False):
        if self.merged:
            wg, wu, wd = self.experts.weights()
            return OF.moe_experts(x, w.float() if x.is_cuda else w, idx, wg, wu, wd, self.expert_start_idx, cap, exact)
        if self._grouped_per_expert(x):
            # per-expert parameters on the fast path: stack them (about 0.1 ms of copies per layer) and run the grouped
            # GEMM pipeline; autograd hands each expert its slice of the stacked weight gradient.  The reference
            # gives its grouped kernels an array of the experts' weight pointers instead
            # (optimus/kernels/grouped_linear_forward.py:7-102).
            wg = torch.stack([e.gate_proj.weight for e in self.experts])
            wu = torch.stack([e.up_proj.weight for e in self.experts])
            wd = torch.stack([e.down_proj.weight for e in self.experts])
            return OF.moe_experts(x, w.float(), idx, wg, wu, wd, self.expert_start_idx, cap, exact)
        return _experts_loop(self.experts, x, w, idx, self.expert_start_idx)

    def _grouped_per_expert(self, x) -> bool:
        return (getattr(self, "fast", False) and x.is_cuda and x.dtype == torch.bfloat16
                and self.hidden_size % 64 == 0 and self.intermediate_size % 64 == 0 and OF.use_kernels(x))

    def _expert_block(self, hidden2d, idx, w):
        pmap = self.pmap
        ep = pmap.expert_parallelism if pmap is not None else 1
        if ep == 1:
            return self._local_experts(hidden2d, w, idx)
        if self.ep_transport == "alltoall" and self.merged and hidden2d.is_cuda:
            from ...parallel.ep_alltoall import fused_ep_moe
            return fused_ep_moe(self, hidden2d, w, idx)
        # reference transport: all-gather everything, reduce-scatter the partial outputs
        g = pmap.ep_group
        T = hidden2d.shape[0]
        x_all = forward_allgather_backward_reducescatter.apply(hidden2d, pmap.ep_ind, ep, g,
                                                               self.use_allreduce_for_reducescatter)
        w_all = forward_allgather_backward_reducescatter.apply(w, pmap.ep_ind, ep, g,
                                                               self.use_allreduce_for_reducescatter)
        i_all = forward_allgather_backward_split.apply(idx, pmap.ep_ind, ep, g)
        x_all = forward_identity_backward_synchronize.apply(x_all, g)
        cap = None
        if x_all.is_cuda and (self.merged or self._grouped_per_expert(x_all)):
            cap = OF.moe_capacity_rows(T * ep, self.num_experts_per_tok, self.num_experts_per_rank, ep,
                                       self.capacity_factor)
        y_all = self._local_experts(x_all, w_all, i_all, cap, exact=not self.capacity_factor)
        forward_synchronize_backward_identity.apply(g)
        return forward_reducescatter_backward_allgather.apply(y_all, pmap.ep_ind, ep, g,
                                                              self.use_allreduce_for_reducescatter, False)

    def forward(self, hidden_states):
        B, S, H = hidden_states.shape
        x = hidden_states.reshape(-1, H)
        router_logits, w, idx = self._route(x, S)
        if self.use_activation_checkpointing_for_moe and torch.is_grad_enabled():
            out = torch_activation_checkpoint(self._expert_block, x, idx, w, use_reentrant=False)
        else:
            out = self._expert_block(x, idx, w)
        out = out.reshape(B, S, H)
        return out, (router_logits if self.output_router_logits else None)

    # ------------------------------------------------------------------ weight import
    def set_parameters_from_full_module(self, module):
        """Copy this rank's slice from an unsharded block (HF-style ``gate`` + ``experts``)."""
        self.gate.load_state_dict(module.gate.state_dict())
        src = module.experts
        for le in range(self.num_experts_per_rank):
            ge = self.expert_start_idx + le
            if hasattr(src, "gate_up_proj"):  # fused HF layout: gate_up_proj [E, 2I, H], down_proj [E, H, I]
                I = self.intermediate_size
                g_w, u_w, d_w = src.gate_up_proj[ge, :I], src.gate_up_proj[ge, I:], src.down_proj[ge]
            elif isinstance(src, MergedMLP):
                g_w, u_w, d_w = (src.gate_proj_merged_weight[ge], src.up_proj_merged_weight[ge],
                                 src.down_proj_merged_weight[ge])
            else:
                g_w, u_w, d_w = src[ge].gate_proj.weight, src[ge].up_proj.weight, src[ge].down_proj.weight
            with torch.no_grad():
                if self.merged:
                    self.experts.gate_proj_merged_weight[le].copy_(g_w)
                    self.experts.up_proj_merged_weight[le].copy_(u_w)
                    self.experts.down_proj_merged_weight[le].copy_(d_w)
                else:
                    self.experts[le].gate_proj.weight.copy_(g_w)
                    self.experts[le].up_proj.weight.copy_(u_w)
                    self.experts[le].down_proj.weight.copy_(d_w)


class OlmoeParallelSparseMoeBlock(SparseMoeBlock):
    """Baseline layout: one ``nn.Linear`` triple per local expert."""

    def __init__(self, config, pmap=None):
        super().__init__(config, pmap, merged=False)


class FastOlmoeParallelSparseMoeBlock(SparseMoeBlock):
    """``--use_fast_moe``: merged weights with ``--use_merged_mlp_in_fast_moe``, else per-expert."""

    def __init__(self, config, pmap=None):
        super().__init__(config, pmap, merged=bool(config.use_merged_mlp_in_fast_moe))
        self.fast = True
