"""Dense decoder shared by the OLMo and Llama families: tensor-, pipeline- and
virtual-pipeline-parallel attention / SwiGLU MLP / decoder layer / model / causal LM.

Behaviour of the reference's two separate implementations (optimus/models/olmo/modeling_olmo.py
:45-525 and optimus/models/llama/modeling_llama.py:24-485), which differ only in the norm
(OLMo: fp32 LayerNorm without parameters, or RMSNorm with the ``RMS`` tag; Llama: RMSNorm with
the config's eps), GQA, selective checkpointing and how pipeline stages hand over tensors.
Megatron-style TP: q/k/v and gate/up are column-parallel, o and down are row-parallel, the
block input is identity-forward / all-reduce-backward and the block output is all-reduced.
"""
from __future__ import annotations

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint as torch_activation_checkpoint

from ...ops import functional as OF
from .comms_ptfunctions import (forward_allgather_backward_split, forward_allreduce_backward_identity,
                                forward_identity_backward_allreduce, forward_split_backward_allgather)
from .modeling_rope_utils import RotaryEmbedding
from .norm_modules import NonParametricLayerNorm, RMSNorm
from .parallel_converter_utils import populate_ColumnLinear_from_Linear, populate_RowLinear_from_Linear
from .parallel_modules import ParallelEmbedding, ParallelLMHead


class CausalLMOutput:
    def __init__(self, loss=None, logits=None):
        self.loss = loss
        self.logits = logits


def _make_norm(config, family):
    if family == "olmo" and not getattr(config, "use_rms_norm", False):
        return NonParametricLayerNorm(config.hidden_size)
    eps = getattr(config, "rms_norm_eps", 1e-5) if family == "llama" else 1e-5
    return RMSNorm(config.hidden_size, eps=eps)


class ParallelMLP(nn.Module):
    def __init__(self, config, pmap=None):
        super().__init__()
        self.config, self.pmap = config, pmap
        tp = pmap.tensor_parallelism
        self.hidden_size, self.intermediate_size = config.hidden_size, config.intermediate_size
        self.intermediate_size_per_rank = config.intermediate_size // tp
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size_per_rank, bias=False)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size_per_rank, bias=False)
        self.down_proj = nn.Linear(self.intermediate_size_per_rank, self.hidden_size, bias=False)

    def forward(self, x, seq_parallel=False):
        tp = self.pmap.tensor_parallelism
        if seq_parallel:
            from ...parallel import tp_fused
            pm = self.pmap
            g, u = tp_fused.ag_linear(x, (self.gate_proj.weight, self.up_proj.weight), pm.tp_ind, tp, pm.tp_group)
            return tp_fused.linear_rs(OF.swiglu(g, u), self.down_proj.weight, pm.tp_ind, tp, pm.tp_group)
        if tp > 1:
            x = forward_identity_backward_allreduce.apply(x, self.pmap.tp_group)
        h = OF.swiglu(OF.linear(x, self.gate_proj.weight), OF.linear(x, self.up_proj.weight))
        y = OF.linear(h, self.down_proj.weight)
        if tp > 1:
            y = forward_allreduce_backward_identity.apply(y, self.pmap.tp_group)
        return y

    def set_parameters_from_full_module(self, module):
        tp, i = self.pmap.tensor_parallelism, self.pmap.tp_ind
        populate_ColumnLinear_from_Linear(module.gate_proj, self.gate_proj, i, tensor_parallelism=tp)
        populate_ColumnLinear_from_Linear(module.up_proj, self.up_proj, i, tensor_parallelism=tp)
        populate_RowLinear_from_Linear(module.down_proj, self.down_proj, i, tensor_parallelism=tp)


class ParallelAttention(nn.Module):
    """Causal self-attention with GQA and optional full-width QK-norm (the reference's shared
    module optimus/models/common/attention_modules.py:30-110 has the same options)."""

    def __init__(self, config, pmap=None):
        super().__init__()
        self.config, self.pmap = config, pmap
        tp = pmap.tensor_parallelism
        self.num_attention_heads_per_rank = config.num_attention_heads // tp
        self.num_key_value_heads_per_rank = config.num_key_value_heads // tp
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        self.num_key_value_groups = config.num_attention_heads // config.num_key_value_heads
        self.scaling = self.head_dim ** -0.5
        bias = getattr(config, "attention_bias", False)
        hq = self.num_attention_heads_per_rank * self.head_dim
        hkv = self.num_key_value_heads_per_rank * self.head_dim
        self.q_proj = nn.Linear(config.hidden_size, hq, bias=bias)
        self.k_proj = nn.Linear(config.hidden_size, hkv, bias=bias)
        self.v_proj = nn.Linear(config.hidden_size, hkv, bias=bias)
        self.o_proj = nn.Linear(hq, config.hidden_size, bias=bias)
        self.use_qk_norm = bool(getattr(config, "use_qk_norm", False)) and not getattr(config, "skip_qk_norm", True)
        if self.use_qk_norm:
            assert tp == 1, "full-width QK-norm needs the whole q/k vector on one rank"
            self.q_norm = RMSNorm(hq, eps=getattr(config, "rms_norm_eps", 1e-5))
            self.k_norm = RMSNorm(hkv, eps=getattr(config, "rms_norm_eps", 1e-5))

    @staticmethod
    def _proj(x, lin):
        y = OF.linear(x, lin.weight)
        return y if lin.bias is None else y + lin.bias

    def forward(self, hidden_states, position_embeddings, seq_parallel=None):
        """``seq_parallel = (B, S)``: ``hidden_states`` holds this rank's ``B * S / TP`` token rows ``[T_loc, H]`` and so
        does the result; the projections carry the all-gather and the reduce-scatter (no biases in this form)."""
        tp = self.pmap.tensor_parallelism
        if seq_parallel is not None:
            from ...parallel import tp_fused
            pm = self.pmap
            B, S = seq_parallel
            q, k, v = tp_fused.ag_linear(hidden_states, (self.q_proj.weight, self.k_proj.weight, self.v_proj.weight),
                                         pm.tp_ind, tp, pm.tp_group, lead=(B, S))
        else:
            if tp > 1:
                hidden_states = forward_identity_backward_allreduce.apply(hidden_states, self.pmap.tp_group)
            B, S, _ = hidden_states.shape
            q = self._proj(hidden_states, self.q_proj)
            k = self._proj(hidden_states, self.k_proj)
            v = self._proj(hidden_states, self.v_proj)
        if self.use_qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        clip = getattr(self.config, "clip_qkv", None)
        if clip is not None:
            q, k, v = q.clamp(-clip, clip), k.clamp(-clip, clip), v.clamp(-clip, clip)
        cos, sin = position_embeddings
        q = OF.rope(q, cos, sin, heads=self.num_attention_heads_per_rank)   # on the projection output, not a view
        k = OF.rope(k, cos, sin, heads=self.num_key_value_heads_per_rank)
        q = q.view(B, S, self.num_attention_heads_per_rank, self.head_dim)
        k = k.view(B, S, self.num_key_value_heads_per_rank, self.head_dim)
        v = v.view(B, S, self.num_key_value_heads_per_rank, self.head_dim)
        o = OF.attention(q, k, v, scale=self.scaling, causal=True)
        if seq_parallel is not None:
            return tp_fused.linear_rs(o.reshape(B * S, self.num_attention_heads_per_rank * self.head_dim),
                                      self.o_proj.weight, pm.tp_ind, tp, pm.tp_group)
        o = self._proj(o.reshape(B, S, self.num_attention_heads_per_rank * self.head_dim), self.o_proj)
        if tp > 1:
            o = forward_allreduce_backward_identity.apply(o, self.pmap.tp_group)
        return o

    def set_parameters_from_full_module(self, module):
        tp, i = self.pmap.tensor_parallelism, self.pmap.tp_ind
        populate_ColumnLinear_from_Linear(module.q_proj, self.q_proj, i, tensor_parallelism=tp)
        populate_ColumnLinear_from_Linear(module.k_proj, self.k_proj, i, tensor_parallelism=tp)
        populate_ColumnLinear_from_Linear(module.v_proj, self.v_proj, i, tensor_parallelism=tp)
        populate_RowLinear_from_Linear(module.o_proj, self.o_proj, i, tensor_parallelism=tp)
        if self.use_qk_norm:
            self.q_norm.load_state_dict(module.q_norm.state_dict())
            self.k_norm.load_state_dict(module.k_norm.state_dict())


def _sp_norm(mod, x, group):
    """A norm applied to sequence-sharded rows: its scale is replicated over the tensor-parallel group, so its
    gradient (a sum over token rows) has to be summed over the group."""
    if isinstance(mod, RMSNorm):
        from ...parallel import tp_fused
        return OF.rms_norm(x, tp_fused.replicated_weight(mod.weight, group), mod.variance_epsilon)
    return mod(x)


class ParallelDecoderLayer(nn.Module):
    def __init__(self, config, layer_idx, pmap=None, family="olmo"):
        super().__init__()
        self.layer_idx = layer_idx
        self.self_attn = ParallelAttention(config, pmap=pmap)
        self.mlp = ParallelMLP(config, pmap=pmap)
        self.input_layernorm = _make_norm(config, family)
        self.post_attention_layernorm = _make_norm(config, family)
        lvl = getattr(config, "activation_checkpointing_level", 0) if getattr(config, "use_activation_checkpointing", False) else 0
        self.ckpt_norm = bool(lvl & 4)

    def _norm(self, mod, x):
        if self.ckpt_norm and torch.is_grad_enabled():
            return torch_activation_checkpoint(mod, x, use_reentrant=False)
        return mod(x)

    def forward_seq_parallel(self, hidden_states, position_embeddings, batch_seq, group):
        """The layer on this rank's token rows ``[T_loc, H]`` (see the module docstring)."""
        h = _sp_norm(self.input_layernorm, hidden_states, group)
        hidden_states = hidden_states + self.self_attn(h, position_embeddings, seq_parallel=batch_seq)
        h = _sp_norm(self.post_attention_layernorm, hidden_states, group)
        return hidden_states + self.mlp(h, seq_parallel=True)

    def forward(self, hidden_states, position_embeddings):
        residual = hidden_states
        h = self.self_attn(self._norm(self.input_layernorm, hidden_states), position_embeddings)
        hidden_states = residual + h
        residual = hidden_states
        h = self.mlp(self._norm(self.post_attention_layernorm, hidden_states))
        return residual + h

    def set_parameters_from_full_module(self, module):
        self.self_attn.set_parameters_from_full_module(module.self_attn)
        self.mlp.set_parameters_from_full_module(module.mlp)
        for name in ("input_layernorm", "post_attention_layernorm"):
            mine = getattr(self, name)
            if isinstance(mine, RMSNorm):
                mine.load_state_dict(getattr(module, name).state_dict())


class ParallelDenseModel(nn.Module):
    def __init__(self, config, pmap=None, family="olmo"):
        super().__init__()
        self.config, self.pmap, self.family = config, pmap, family
        self.num_hidden_layers = config.num_hidden_layers
        self.padding_idx = config.pad_token_id
        self.vocab_size = config.vocab_size
        tp, PP = pmap.tensor_parallelism, pmap.pipeline_parallelism
        self.VPP = getattr(config, "virtual_pipeline_parallelism", 1)
        if pmap.is_first_stage_rank:
            if tp > 1:
                self.embed_tokens = ParallelEmbedding(config.vocab_size, config.hidden_size, self.padding_idx,
                                                      tensor_parallelism=tp, tp_ind=pmap.tp_ind, group=pmap.tp_group)
            else:
                self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        else:
            self.embed_tokens = nn.Identity()
        self.num_hidden_layers_per_rank = config.num_hidden_layers // PP
        self.num_hidden_layers_per_vpp_rank = self.num_hidden_layers_per_rank // self.VPP
        LV = self.num_hidden_layers_per_vpp_rank
        self.layer_ids = [(v * PP + pmap.pp_ind) * LV + l for v in range(self.VPP) for l in range(LV)]
        self.layers = nn.ModuleList([ParallelDecoderLayer(config, self.layer_ids[i], pmap=pmap, family=family)
                                     for i in range(self.num_hidden_layers_per_rank)])
        self.norm = _make_norm(config, family) if pmap.is_last_stage_rank else nn.Identity()
        self.rotary_emb = RotaryEmbedding(config)

    def _seq_parallel_ok(self, hidden_states) -> bool:
        """Sequence-parallel execution with the collectives inside the GEMMs: tensor parallel, bf16 on GPUs with peer
        access, no projection biases, token rows divisible into 128-row blocks per rank."""
        pm = self.pmap
        tp = pm.tensor_parallelism
        if tp <= 1 or not hidden_states.is_cuda or hidden_states.dtype != torch.bfloat16:
            return False
        if getattr(self.config, "attention_bias", False) or hidden_states.dim() != 3:
            return False
        B, S, H = hidden_states.shape
        if (B * S) % (tp * 128) or any(l.ckpt_norm for l in self.layers):
            return False
        from ...parallel import tp_fused
        l0 = self.layers[0]
        ws = (l0.self_attn.q_proj.weight, l0.self_attn.k_proj.weight, l0.self_attn.o_proj.weight,
              l0.mlp.gate_proj.weight, l0.mlp.down_proj.weight)
        return tp_fused.usable(hidden_states.view(B * S, H)[:(B * S) // tp], pm.tp_group, ws)

    def forward(self, input_ids, vp_ind=0):
        hidden_states = OF.embed(self.embed_tokens, input_ids) if vp_ind == 0 else input_ids
        pos = self.rotary_emb.table(hidden_states.size(1), hidden_states.device)
        LV = self.num_hidden_layers_per_vpp_rank
        if self._seq_parallel_ok(hidden_states):
            pm = self.pmap
            B, S, H = hidden_states.shape
            # this rank's rows of the flattened [B * S] token axis; the backward all-gathers the rows' gradients for
            # the (vocabulary-parallel) embedding or the previous pipeline stage
            h = forward_split_backward_allgather.apply(hidden_states.reshape(B * S, H), pm.tp_ind, pm.tensor_parallelism,
                                                       pm.tp_group)
            for i in range(vp_ind * LV, (vp_ind + 1) * LV):
                h = self.layers[i].forward_seq_parallel(h, pos, (B, S), pm.tp_group)
            if vp_ind == self.VPP - 1:
                h = _sp_norm(self.norm, h, pm.tp_group)
            # every rank continues with all rows (the hidden-split LM head, or the next pipeline stage)
            h = forward_allgather_backward_split.apply(h, pm.tp_ind, pm.tensor_parallelism, pm.tp_group)
            return h.view(B, S, H)
        for i in range(vp_ind * LV, (vp_ind + 1) * LV):
            hidden_states = self.layers[i](hidden_states, pos)
        return self.norm(hidden_states) if vp_ind == self.VPP - 1 else hidden_states

    def set_parameters_from_full_module(self, module):
        if self.pmap.is_first_stage_rank:
            if isinstance(self.embed_tokens, ParallelEmbedding):
                self.embed_tokens.set_parameters_from_full_module(module.embed_tokens)
            else:
                self.embed_tokens.load_state_dict(module.embed_tokens.state_dict())
        for i in range(self.num_hidden_layers_per_rank):
            self.layers[i].set_parameters_from_full_module(module.layers[self.layer_ids[i]])
        if self.pmap.is_last_stage_rank and isinstance(self.norm, RMSNorm):
            self.norm.load_state_dict(module.norm.state_dict())


class ParallelDenseForCausalLM(nn.Module):
    """``pp_dict_outputs``: Llama's pipeline stages return ``{"output", "router_logits": None}``
    (old trainer contract), OLMo's return raw tensors (virtual-pipeline trainer contract)."""

    family = "olmo"
    pp_dict_outputs = False
    output_class = CausalLMOutput

    def __init__(self, config, pmap=None, memory_tracker=None):
        super().__init__()
        if pmap is None:
            from ...mapper import ParallelDpPpEpTpMapper
            pmap = ParallelDpPpEpTpMapper()
        self.config, self.pmap = config, pmap
        self.vocab_size = config.vocab_size
        self.model = ParallelDenseModel(config, pmap=pmap, family=self.family)
        if pmap.is_last_stage_rank:
            if pmap.tensor_parallelism > 1:
                self.lm_head = ParallelLMHead(config.hidden_size, config.vocab_size, bias=False,
                                              tensor_parallelism=pmap.tensor_parallelism, tp_ind=pmap.tp_ind,
                                              group=pmap.tp_group)
            else:
                self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        else:
            self.lm_head = nn.Identity()
        self.inplace_ce_backward = True

    def loss_function(self, logits, labels, vocab_size=None):
        return OF.shifted_cross_entropy(logits, labels, inplace_backward=self.inplace_ce_backward)

    def _head(self, hidden_states):
        if isinstance(self.lm_head, ParallelLMHead):
            return self.lm_head(hidden_states)
        return OF.linear(hidden_states, self.lm_head.weight)

    def forward(self, input_ids, vp_ind=0, labels=None):
        if isinstance(vp_ind, torch.Tensor):  # forward(input_ids, labels) positional call
            vp_ind, labels = 0, vp_ind
        hidden_states = self.model(input_ids, vp_ind=vp_ind)
        PP, VPP = self.pmap.pipeline_parallelism, self.model.VPP
        output_stage = self.pmap.is_last_stage_rank and vp_ind == VPP - 1
        if PP > 1 and not output_stage:
            return {"output": hidden_states, "router_logits": None} if self.pp_dict_outputs else hidden_states
        logits = self._head(hidden_states)
        if PP > 1:
            return {"output": logits, "router_logits": None} if self.pp_dict_outputs else logits
        loss = self.loss_function(logits, labels, self.vocab_size) if labels is not None else None
        return self.output_class(loss=loss, logits=logits)

    def set_parameters_from_full_module(self, module):
        self.model.set_parameters_from_full_module(module.model)
        if self.pmap.is_last_stage_rank:
            if isinstance(self.lm_head, ParallelLMHead):
                self.lm_head.set_parameters_from_full_module(module.lm_head)
            else:
                self.lm_head.load_state_dict(module.lm_head.state_dict())

    # ------------------------------------------------------------------ accounting
    def get_flops(self, context_size):
        c, S = self.config, context_size
        hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
        attn = 2 * 6 * S * c.hidden_size * (c.num_attention_heads * hd)
        attn += 2 * 6 * S * c.hidden_size * (c.num_key_value_heads * hd)
        attn += 2 * 6 * c.num_attention_heads * S * S * hd
        mlp = 3 * 6 * S * c.hidden_size * c.intermediate_size
        tp, pp = self.pmap.tensor_parallelism, self.pmap.pipeline_parallelism
        block = attn // tp + mlp // tp
        return (c.num_hidden_layers * block) // pp + (6 * S * c.hidden_size * c.vocab_size) // tp

    def _tp_sharded_names(self):
        names = ["model.embed_tokens.weight", "lm_head.weight"]
        for i in range(len(self.model.layers)):
            names += [f"model.layers.{i}.self_attn.{p}_proj.weight" for p in "qkvo"]
            names += [f"model.layers.{i}.mlp.{p}_proj.weight" for p in ("gate", "up", "down")]
        return set(names)

    def get_tp_replicated_param_list(self):
        """Parameters that are identical on all TP ranks (norm weights, biases)."""
        sharded = self._tp_sharded_names()
        return [n for n, p in self.named_parameters() if n not in sharded]

    def calculate_grad_norm(self, grad_scale: float = 1.0):
        """Global gradient norm under TP: sharded gradients count once per rank, replicated ones
        with weight 1/TP, summed over the TP group (reference modeling_olmo.py:476-525)."""
        import torch.distributed as dist
        sharded = self._tp_sharded_names()
        dev = next(self.parameters()).device
        sq_s = torch.zeros(1, dtype=torch.float32, device=dev)
        sq_r = torch.zeros(1, dtype=torch.float32, device=dev)
        for n, p in self.named_parameters():
            if p.grad is None:
                continue
            OF.sum_of_squares(p.grad.contiguous().view(-1), grad_scale, out=sq_s if n in sharded else sq_r,
                              accumulate=True)
        tp = self.pmap.tensor_parallelism
        if dist.is_initialized() and tp > 1:
            total = sq_s + sq_r / tp
            dist.all_reduce(total, group=self.pmap.tp_group)
        else:
            total = sq_s + sq_r
        return total.sqrt().reshape(())
