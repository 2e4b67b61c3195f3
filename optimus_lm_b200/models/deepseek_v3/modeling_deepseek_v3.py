"""DeepSeek-V3: multi-head latent attention (MLA) + shared/routed experts, pipeline- and
expert-parallel.

Architecture, forward math and state-dict keys of the reference
(optimus/models/deepseek_v3/modeling_deepseek_v3.py:29-643):

* MLA: ``q_a_proj -> RMSNorm -> q_b_proj`` gives per-head ``[nope 128 | rope 64]`` queries;
  ``kv_a_proj_with_mqa`` gives a 512-wide latent (-> RMSNorm -> ``kv_b_proj`` -> per-head
  ``[k_nope 128 | v 128]``) plus one 64-wide rope key shared by all heads.  Interleaved RoPE with
  YaRN frequencies on the rope parts; softmax scale ``qk_head_dim^-0.5 * mscale^2``.  The
  reference materialises the ``S x S`` scores; here the flash-attention op runs with
  ``d_qk = 192, d_v = 128``.
* Router: fp32 sigmoid scores, group-limited top-k on ``score + e_score_correction_bias`` (8 groups,
  best 4 by their top-2 sum, then top-8), weights = unbiased scores renormalised (+1e-20) and
  scaled by 2.5.  No auxiliary loss.  The bias is a zero buffer unless ``update_router_bias``.
* Routed experts partitioned contiguously over EP ranks; one shared expert on local tokens.
* The first ``first_k_dense_replace`` layers use a dense SwiGLU MLP whose intermediate dimension
  is sharded over the EP group like tensor parallelism (all-gather tokens -> partial MLP ->
  reduce-scatter).

``merged_experts`` (default: on for GPUs) stores the local routed experts as three stacked
tensors and runs the grouped tcgen05 GEMM pipeline; ``state_dict`` still exposes the reference's
per-expert keys ``mlp.experts.{e}.{gate,up,down}_proj.weight``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn
from torch.utils.checkpoint import checkpoint as torch_activation_checkpoint

from ...ops import functional as OF
from ...ops._ext import use_kernels
from ..common.comms_ptfunctions import (forward_allgather_backward_reducescatter,
                                        forward_reducescatter_backward_allgather)
from ..common.modeling_rope_utils import RotaryEmbedding, yarn_get_mscale
from ..common.moe import MergedMLP, SparseMoeBlock
from ..common.norm_modules import RMSNorm
from ..common.parallel_converter_utils import populate_ColumnLinear_from_Linear, populate_RowLinear_from_Linear


class DeepseekV3ParallelOutput:
    def __init__(self, loss=None, logits=None):
        self.loss = loss
        self.logits = logits


DeepseekV3ParallelRMSNorm = RMSNorm


class DeepseekV3ParallelRotaryEmbedding(RotaryEmbedding):
    """YaRN table over the 64 rope dims (reference :46-77 with rope_utils.py:5-72)."""


class DeepseekV3ParallelMLP(nn.Module):
    """SwiGLU MLP.  With ``pmap`` (dense layers) the intermediate dimension is split over the EP
    group; without it (routed / shared experts) it is whole."""

    def __init__(self, config, hidden_size=None, intermediate_size=None, pmap=None):
        super().__init__()
        self.config, self.pmap = config, pmap
        self.hidden_size = config.hidden_size if hidden_size is None else hidden_size
        self.intermediate_size = config.intermediate_size if intermediate_size is None else intermediate_size
        if pmap is None:
            self.intermediate_size_per_rank = self.intermediate_size
        else:
            self.intermediate_size_per_rank = config.intermediate_size // pmap.expert_parallelism
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size_per_rank, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size_per_rank, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size_per_rank, self.hidden_size, bias=False)
        self.use_allreduce_for_reducescatter = False
        self.ckpt = bool(config.use_activation_checkpointing and (config.activation_checkpointing_level & 1))

    def _block(self, x):
        p = self.pmap
        sharded = p is not None and p.expert_parallelism > 1
        shape = x.shape
        if sharded:
            x = x.reshape(-1, shape[-1])
            from ...parallel import tp_fused
            if tp_fused.usable(x, p.ep_group, (self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight)):
                y = tp_fused.ag_swiglu_mlp_rs(x, self.gate_proj.weight, self.up_proj.weight, self.down_proj.weight,
                                              p.ep_ind, p.expert_parallelism, p.ep_group)
                return y.reshape(shape)
            x = forward_allgather_backward_reducescatter.apply(x, p.ep_ind, p.expert_parallelism, p.ep_group,
                                                               self.use_allreduce_for_reducescatter)
        h = OF.swiglu(OF.linear(x, self.gate_proj.weight), OF.linear(x, self.up_proj.weight))
        y = OF.linear(h, self.down_proj.weight)
        if sharded:
            y = forward_reducescatter_backward_allgather.apply(y, p.ep_ind, p.expert_parallelism, p.ep_group,
                                                               self.use_allreduce_for_reducescatter, False)
            y = y.reshape(shape)
        return y

    def forward(self, hidden_states):
        if self.ckpt and torch.is_grad_enabled():
            return torch_activation_checkpoint(self._block, hidden_states, use_reentrant=False)
        return self._block(hidden_states)

    def set_parameters_from_full_module(self, module):
        if self.pmap is None:
            self.load_state_dict(module.state_dict())
            return
        ep, i = self.pmap.expert_parallelism, self.pmap.ep_ind
        populate_ColumnLinear_from_Linear(module.gate_proj, self.gate_proj, i, tensor_parallelism=ep)
        populate_ColumnLinear_from_Linear(module.up_proj, self.up_proj, i, tensor_parallelism=ep)
        populate_RowLinear_from_Linear(module.down_proj, self.down_proj, i, tensor_parallelism=ep)


def sigmoid_group_topk_reference(logits, bias, top_k, n_group, topk_group, renorm, scale):
    """Reference routing (:150-191) on fp32 logits; returns (weights, indices)."""
    T, E = logits.shape
    scores = logits.sigmoid()
    choice = scores + bias.unsqueeze(0)
    group_scores = choice.view(T, n_group, E // n_group).topk(2, dim=-1)[0].sum(dim=-1)
    group_idx = torch.topk(group_scores, k=topk_group, dim=-1, sorted=False)[1]
    group_mask = torch.zeros_like(group_scores).scatter_(1, group_idx, 1)
    score_mask = group_mask.unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E)
    choice = choice.masked_fill(~score_mask.bool(), 0.0)
    idx = torch.topk(choice, k=top_k, dim=-1, sorted=False)[1]
    w = scores.gather(1, idx)
    if renorm:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    return w * scale, idx


class _SigmoidRouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, bias, top_k, n_group, topk_group, renorm, scale):
        C = OF.extension()
        T, E = logits.shape
        w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
        idx = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
        C.router_sigmoid_group_topk(logits, bias, top_k, n_group, topk_group, renorm, scale, w, idx)
        ctx.save_for_backward(logits, idx)
        ctx.cfg = (renorm, scale)
        ctx.mark_non_differentiable(idx)
        return w, idx

    @staticmethod
    def backward(ctx, dw, _):
        logits, idx = ctx.saved_tensors
        renorm, scale = ctx.cfg
        d = torch.zeros_like(logits)
        OF.extension().router_sigmoid_bwd(logits, idx, dw.contiguous(), renorm, scale, d)
        return d, None, None, None, None, None, None


class DeepseekV3ParallelTopkRouter(nn.Module):
    def __init__(self, config, pmap=None):
        super().__init__()
        self.config, self.pmap = config, pmap
        self.top_k = config.num_experts_per_tok
        self.n_routed_experts = config.n_routed_experts
        self.routed_scaling_factor = config.routed_scaling_factor
        self.n_group, self.topk_group = config.n_group, config.topk_group
        self.norm_topk_prob = config.norm_topk_prob
        self.weight = nn.Parameter(torch.empty((self.n_routed_experts, config.hidden_size)))
        self.register_buffer("e_score_correction_bias", torch.zeros(self.n_routed_experts, dtype=torch.float32))
        self.mask = None
        self.force_uniform_routing = config.force_uniform_routing
        self.last_indices = None

    def forward(self, hidden_states):
        x = hidden_states.reshape(-1, self.config.hidden_size)
        # fp32 logits as in the reference; the bf16 GEMM with fp32 output keeps the accumulation in fp32
        if x.is_cuda and x.dtype == torch.bfloat16 and use_kernels(x) and self.n_routed_experts % 8 == 0:
            logits = _Fp32LogitsFn.apply(x, self.weight)
        else:
            logits = F.linear(x.float(), self.weight.float())
        if self.force_uniform_routing:
            if self.mask is None or self.mask.shape[0] != logits.shape[0]:
                from ...utils import get_load_balanced_expert_mask
                ep_ind = self.pmap.ep_ind if self.pmap is not None else 0
                m = get_load_balanced_expert_mask(logits.shape[0], self.n_routed_experts, self.top_k, ep_ind)
                self.mask = (~m).to(logits.device)
            scores = logits.sigmoid()
            idx = torch.topk(scores.masked_fill(self.mask, float("-inf")), k=self.top_k, dim=-1, sorted=False)[1]
            w = scores.gather(1, idx)
            if self.norm_topk_prob:
                w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
            w = w * self.routed_scaling_factor
            idx = idx.to(torch.int32) if x.is_cuda else idx
        elif logits.is_cuda and use_kernels(logits) and self.n_routed_experts <= 256:
            w, idx = _SigmoidRouterFn.apply(logits.contiguous(), self.e_score_correction_bias.float(), self.top_k,
                                            self.n_group, self.topk_group, self.norm_topk_prob,
                                            self.routed_scaling_factor)
        else:
            w, idx = sigmoid_group_topk_reference(logits, self.e_score_correction_bias.float(), self.top_k,
                                                  self.n_group, self.topk_group, self.norm_topk_prob,
                                                  self.routed_scaling_factor)
        self.last_indices = idx
        return idx, w


class _Fp32LogitsFn(torch.autograd.Function):
    """Router logits: bf16 operands, fp32 result (tcgen05 GEMM with an fp32 epilogue)."""

    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        return OF.gemm(x, w, x.shape[0], w.shape[0], x.shape[1], out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, d):
        x, w = ctx.saved_tensors
        db = d.to(torch.bfloat16)
        dx = OF.gemm(db, w, x.shape[0], x.shape[1], w.shape[0], b_mn_major=True)
        dw = OF.gemm(db, x, w.shape[0], x.shape[1], x.shape[0], a_mn_major=True, b_mn_major=True)
        return dx, dw


class DeepseekV3ParallelMoE(nn.Module):
    """Routed experts (EP-partitioned) + shared expert.  Module order (experts, gate,
    shared_experts) follows the reference so that ``named_parameters()`` lines up."""

    def __init__(self, config, pmap=None):
        super().__init__()
        self.config, self.pmap = config, pmap
        ep = config.expert_parallelism
        self.num_experts = config.n_routed_experts
        self.num_experts_per_tok = config.num_experts_per_tok
        self.n_routed_experts_per_rank = self.num_experts_per_rank = config.n_routed_experts // ep
        self.expert_start_idx = pmap.ep_ind * self.num_experts_per_rank
        self.expert_end_idx = self.expert_start_idx + self.num_experts_per_rank
        self.hidden_size, self.intermediate_size = config.hidden_size, config.moe_intermediate_size
        self.merged = bool(getattr(config, "merged_experts", torch.cuda.is_available()))
        if self.merged:
            self.experts = MergedMLP(self.num_experts_per_rank, config.hidden_size, config.moe_intermediate_size)
        else:
            self.experts = nn.ModuleList([DeepseekV3ParallelMLP(config, intermediate_size=config.moe_intermediate_size)
                                          for _ in range(self.num_experts_per_rank)])
        self.gate = DeepseekV3ParallelTopkRouter(config, pmap=pmap)
        self.shared_experts = DeepseekV3ParallelMLP(
            config=config, intermediate_size=config.moe_intermediate_size * config.n_shared_experts)
        self.use_allreduce_for_reducescatter = False
        self.ckpt = bool(config.use_activation_checkpointing and (config.activation_checkpointing_level & 1))
        self.capacity_factor = float(getattr(config, "moe_capacity_factor", 0.0))
        self.ep_transport = "alltoall" if getattr(config, "use_fused_ep_alltoall", True) else "allgather"
        self._a2a = None
        if self.merged:
            self._register_state_dict_hook(self._split_experts_on_save)
            self._register_load_state_dict_pre_hook(self._merge_experts_on_load)

    # routed-expert execution and EP transports are shared with the OLMoE block
    _local_experts = SparseMoeBlock._local_experts
    _expert_block = SparseMoeBlock._expert_block
    _grouped_per_expert = SparseMoeBlock._grouped_per_expert

    def _block(self, hidden_states, topk_indices, topk_weights):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        routed = self._expert_block(x, topk_indices, topk_weights.to(x.dtype) if not x.is_cuda else topk_weights)
        return routed.reshape(shape) + self.shared_experts(hidden_states)

    def forward(self, hidden_states):
        topk_indices, topk_weights = self.gate(hidden_states)
        if self.ckpt and torch.is_grad_enabled():
            return torch_activation_checkpoint(self._block, hidden_states, topk_indices, topk_weights,
                                               use_reentrant=False)
        return self._block(hidden_states, topk_indices, topk_weights)

    # ------------------------------------------------------------------ checkpoint key translation
    @staticmethod
    def _split_experts_on_save(module, state_dict, prefix, local_metadata):
        names = (("gate_proj_merged_weight", "gate_proj"), ("up_proj_merged_weight", "up_proj"),
                 ("down_proj_merged_weight", "down_proj"))
        for merged_name, proj in names:
            t = state_dict.pop(f"{prefix}experts.{merged_name}")
            for e in range(t.shape[0]):
                state_dict[f"{prefix}experts.{e}.{proj}.weight"] = t[e]
        return state_dict

    def _merge_experts_on_load(self, state_dict, prefix, *args):
        if f"{prefix}experts.0.gate_proj.weight" not in state_dict:
            return
        for merged_name, proj in (("gate_proj_merged_weight", "gate_proj"), ("up_proj_merged_weight", "up_proj"),
                                  ("down_proj_merged_weight", "down_proj")):
            parts = [state_dict.pop(f"{prefix}experts.{e}.{proj}.weight") for e in range(self.num_experts_per_rank)]
            state_dict[f"{prefix}experts.{merged_name}"] = torch.stack(parts, dim=0)

    def set_parameters_from_full_module(self, module):
        self.gate.load_state_dict(module.gate.state_dict())
        for le in range(self.num_experts_per_rank):
            src = module.experts[self.expert_start_idx + le]
            with torch.no_grad():
                if self.merged:
                    self.experts.gate_proj_merged_weight[le].copy_(src.gate_proj.weight)
                    self.experts.up_proj_merged_weight[le].copy_(src.up_proj.weight)
                    self.experts.down_proj_merged_weight[le].copy_(src.down_proj.weight)
                else:
                    self.experts[le].load_state_dict(src.state_dict())
        self.shared_experts.load_state_dict(module.shared_experts.state_dict())

    @torch.no_grad()
    def update_router_bias(self, speed: float):
        """Auxiliary-loss-free balancing step (an addition, off by default): raise the bias of
        under-loaded experts and lower it for over-loaded ones by ``speed``."""
        idx = self.gate.last_indices
        if idx is None:
            return
        load = torch.bincount(idx.reshape(-1).long(), minlength=self.num_experts).float()
        if torch.distributed.is_initialized() and self.pmap is not None and self.pmap.dpep_group not in (None, -1):
            torch.distributed.all_reduce(load, group=self.pmap.dpep_group)
        self.gate.e_score_correction_bias.add_(speed * torch.sign(load.mean() - load))


class DeepseekV3ParallelAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        assert config.num_attention_heads == config.num_key_value_heads
        assert config.q_lora_rank is not None and config.rope_interleave
        self.num_heads = config.num_attention_heads
        self.q_lora_rank, self.kv_lora_rank = config.q_lora_rank, config.kv_lora_rank
        self.qk_rope_head_dim, self.qk_nope_head_dim = config.qk_rope_head_dim, config.qk_nope_head_dim
        self.v_head_dim, self.qk_head_dim = config.v_head_dim, config.qk_head_dim
        self.q_a_proj = nn.Linear(config.hidden_size, config.q_lora_rank, bias=False)
        self.q_a_layernorm = RMSNorm(config.q_lora_rank, eps=1e-6)
        self.q_b_proj = nn.Linear(config.q_lora_rank, self.num_heads * self.qk_head_dim, bias=False)
        self.kv_a_proj_with_mqa = nn.Linear(config.hidden_size, self.kv_lora_rank + self.qk_rope_head_dim, bias=False)
        self.kv_a_layernorm = RMSNorm(self.kv_lora_rank, eps=1e-6)
        self.kv_b_proj = nn.Linear(self.kv_lora_rank, self.num_heads * (self.qk_nope_head_dim + self.v_head_dim),
                                   bias=False)
        self.o_proj = nn.Linear(self.num_heads * self.v_head_dim, config.hidden_size, bias=False)
        self.scaling = self.qk_head_dim ** (-0.5)
        mscale_all_dim = config.rope_scaling.get("mscale_all_dim", 0)
        if mscale_all_dim:
            m = yarn_get_mscale(config.rope_scaling["factor"], mscale_all_dim)
            self.scaling = self.scaling * m * m

    def forward(self, hidden_states, position_embeddings):
        B, S, _ = hidden_states.shape
        H, dn, dr, dv = self.num_heads, self.qk_nope_head_dim, self.qk_rope_head_dim, self.v_head_dim
        cos, sin = position_embeddings
        q = OF.linear(self.q_a_layernorm(OF.linear(hidden_states, self.q_a_proj.weight)), self.q_b_proj.weight)
        q = OF.rope(q, cos, sin, rot_offset=dn, rot_dim=dr, interleaved=True, heads=H).view(B, S, H, dn + dr)

        ckv = OF.linear(hidden_states, self.kv_a_proj_with_mqa.weight)
        k_lat, k_rot = ckv[..., :self.kv_lora_rank], ckv[..., self.kv_lora_rank:]
        kv = OF.linear(self.kv_a_layernorm(k_lat.contiguous()), self.kv_b_proj.weight).view(B, S, H, dn + dv)
        k_nope, v = kv[..., :dn], kv[..., dn:]
        k_rot = OF.rope(k_rot.reshape(B, S, 1, dr).contiguous(), cos, sin, interleaved=True)
        k = torch.cat((k_nope, k_rot.expand(B, S, H, dr)), dim=-1)

        o = OF.attention(q, k, v, scale=self.scaling, causal=True)
        return OF.linear(o.reshape(B, S, H * dv), self.o_proj.weight), None

    def set_parameters_from_full_module(self, module):
        self.load_state_dict(module.state_dict())


class DeepseekV3ParallelDecoderLayer(nn.Module):
    def __init__(self, config, layer_idx=0, pmap=None, memory_tracker=None):
        super().__init__()
        self.self_attn = DeepseekV3ParallelAttention(config)
        if layer_idx >= config.first_k_dense_replace:
            self.mlp = DeepseekV3ParallelMoE(config, pmap=pmap)
        else:
            self.mlp = DeepseekV3ParallelMLP(config, pmap=pmap)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.layer_idx, self.memory_tracker = layer_idx, memory_tracker
        lvl = config.activation_checkpointing_level if config.use_activation_checkpointing else 0
        self.ckpt_attn, self.ckpt_norm = bool(lvl & 2), bool(lvl & 4)

    def _log(self, what):
        if self.memory_tracker is not None:
            self.memory_tracker.log(f"L{self.layer_idx} {what}")

    def _ckpt(self, on, fn, *args):
        if on and torch.is_grad_enabled():
            return torch_activation_checkpoint(fn, *args, use_reentrant=False)
        return fn(*args)

    def forward(self, hidden_states, position_embeddings):
        self._log("Before Decoder")
        residual = hidden_states
        h = self._ckpt(self.ckpt_norm, self.input_layernorm, hidden_states)
        h, _ = self._ckpt(self.ckpt_attn, self.self_attn, h, position_embeddings)
        self._log("After Attention")
        hidden_states = residual + h
        residual = hidden_states
        h = self._ckpt(self.ckpt_norm, self.post_attention_layernorm, hidden_states)
        h = self.mlp(h)
        self._log("After MoE")
        return residual + h

    def set_parameters_from_full_module(self, module):
        self.self_attn.set_parameters_from_full_module(module.self_attn)
        self.mlp.set_parameters_from_full_module(module.mlp)
        self.input_layernorm.load_state_dict(module.input_layernorm.state_dict())
        self.post_attention_layernorm.load_state_dict(module.post_attention_layernorm.state_dict())


class DeepseekV3ParallelModel(nn.Module):
    def __init__(self, config, pmap=None, memory_tracker=None):
        super().__init__()
        self.pmap, self.config, self.memory_tracker = pmap, config, memory_tracker
        self.padding_idx = config.pad_token_id
        self.vocab_size = config.vocab_size
        self.embed_tokens = (nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
                             if pmap.is_first_stage_rank else nn.Identity())
        self.num_hidden_layers_per_rank = config.num_hidden_layers // pmap.pipeline_parallelism
        self.layer_start_idx = pmap.pp_ind * self.num_hidden_layers_per_rank
        self.layer_end_idx = self.layer_start_idx + self.num_hidden_layers_per_rank
        self.layers = nn.ModuleList([
            DeepseekV3ParallelDecoderLayer(config, layer_idx=i, pmap=pmap, memory_tracker=memory_tracker)
            for i in range(self.layer_start_idx, self.layer_end_idx)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps) if pmap.is_last_stage_rank else nn.Identity()
        self.rotary_emb = DeepseekV3ParallelRotaryEmbedding(config=config)
        lvl = config.activation_checkpointing_level if config.use_activation_checkpointing else 0
        self.ckpt_norm = bool(lvl & 4)

    def forward(self, input_ids):
        hidden_states = OF.embed(self.embed_tokens, input_ids)
        pos = self.rotary_emb.table(hidden_states.size(1), hidden_states.device)
        for layer in self.layers:
            hidden_states = layer(hidden_states, pos)
        if self.ckpt_norm and torch.is_grad_enabled():
            return torch_activation_checkpoint(self.norm, hidden_states, use_reentrant=False)
        return self.norm(hidden_states)

    def set_parameters_from_full_module(self, module):
        if self.pmap.is_first_stage_rank:
            self.embed_tokens.load_state_dict(module.embed_tokens.state_dict())
        for l in range(self.num_hidden_layers_per_rank):
            self.layers[l].set_parameters_from_full_module(module.layers[self.layer_start_idx + l])
        if self.pmap.is_last_stage_rank:
            self.norm.load_state_dict(module.norm.state_dict())


class DeepseekV3ParallelForCausalLM(nn.Module):
    def __init__(self, config, pmap=None, memory_tracker=None):
        super().__init__()
        if pmap is None:
            from ...mapper import ParallelDpPpEpTpMapper
            pmap = ParallelDpPpEpTpMapper()
        self.config, self.pmap, self.memory_tracker = config, pmap, memory_tracker
        self.vocab_size = config.vocab_size
        self.model = DeepseekV3ParallelModel(config, pmap=pmap, memory_tracker=memory_tracker)
        self.lm_head = (nn.Linear(config.hidden_size, config.vocab_size, bias=False)
                        if pmap.is_last_stage_rank else nn.Identity())
        self.inplace_ce_backward = True

    def loss_function(self, logits, labels, vocab_size=None):
        return OF.shifted_cross_entropy(logits, labels, inplace_backward=self.inplace_ce_backward)

    def forward(self, input_ids, labels=None):
        hidden_states = self.model(input_ids)
        PP = self.pmap.pipeline_parallelism
        if PP > 1 and not self.pmap.is_last_stage_rank:
            return {"output": hidden_states, "router_logits": None}
        logits = OF.linear(hidden_states, self.lm_head.weight)
        if PP > 1:
            return {"output": logits, "router_logits": None}
        loss = self.loss_function(logits, labels, self.vocab_size) if labels is not None else None
        if self.training and getattr(self.config, "update_router_bias", False):
            for layer in self.model.layers:
                if isinstance(layer.mlp, DeepseekV3ParallelMoE):
                    layer.mlp.update_router_bias(self.config.router_bias_update_speed)
        return DeepseekV3ParallelOutput(loss=loss, logits=logits)

    def set_parameters_from_full_module(self, module):
        self.model.set_parameters_from_full_module(module.model)
        if self.pmap.is_last_stage_rank:
            self.lm_head.load_state_dict(module.lm_head.state_dict())

    def get_flops(self, context_size):
        """Analytical training FLOPs per sequence (reference :560-605)."""
        c, S = self.config, context_size
        H = c.num_attention_heads
        attn = 6 * S * c.hidden_size * c.q_lora_rank + 6 * S * c.q_lora_rank * (H * c.qk_head_dim)
        attn += 6 * S * c.hidden_size * (c.kv_lora_rank + c.qk_rope_head_dim)
        attn += 6 * S * c.kv_lora_rank * (H * (c.qk_nope_head_dim + c.v_head_dim))
        attn += 6 * S * (H * c.v_head_dim) * c.hidden_size
        attn += 6 * H * S * S * c.qk_head_dim + 6 * H * S * S * (c.qk_nope_head_dim + c.v_head_dim)
        dense = 3 * 6 * S * c.hidden_size * c.intermediate_size
        moe = 3 * (c.num_experts_per_tok + c.n_shared_experts) * 6 * S * c.hidden_size * c.moe_intermediate_size
        if c.use_activation_checkpointing:
            lvl = c.activation_checkpointing_level
            attn = int((4 / 3) * attn) if lvl & 1 else attn
            dense = int((4 / 3) * dense) if lvl & 2 else dense
            moe = int((4 / 3) * moe) if lvl & 4 else moe
        stack = c.first_k_dense_replace * (attn + dense) + (c.num_hidden_layers - c.first_k_dense_replace) * (attn + moe)
        return (stack + 6 * S * c.hidden_size * c.vocab_size) / self.pmap.pipeline_parallelism

    def get_ep_replicated_param_list(self):
        """Parameters identical on all EP ranks: everything except routed experts and the
        EP-sharded dense MLPs (reference :607-643)."""
        names = []
        if self.pmap.is_first_stage_rank:
            names.append("model.embed_tokens.weight")
        n = len(self.model.layers)
        for i in range(n):
            names += [f"model.layers.{i}.self_attn.{p}.weight" for p in
                      ("q_a_proj", "q_a_layernorm", "q_b_proj", "kv_a_proj_with_mqa", "kv_a_layernorm", "kv_b_proj",
                       "o_proj")]
        for i in range(n):
            if self.model.layer_start_idx + i >= self.config.first_k_dense_replace:
                names.append(f"model.layers.{i}.mlp.gate.weight")
                names += [f"model.layers.{i}.mlp.shared_experts.{p}_proj.weight" for p in ("gate", "up", "down")]
        for i in range(n):
            names += [f"model.layers.{i}.input_layernorm.weight", f"model.layers.{i}.post_attention_layernorm.weight"]
        if self.pmap.is_last_stage_rank:
            names += ["model.norm.weight", "lm_head.weight"]
        return names
