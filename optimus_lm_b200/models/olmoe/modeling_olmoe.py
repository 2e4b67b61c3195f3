"""OLMoE decoder with pipeline- and expert-parallel sharding.

Architecture and state-dict keys of the reference (optimus/models/olmoe/modeling_olmoe.py:93-661,
and the virtual-pipeline variant modeling_olmoe_new.py): embed -> N x [RMSNorm -> attention
(q/k/v/o, full-width QK RMSNorm before the head split, optional clip, rotate-half RoPE,
causal attention) + residual -> RMSNorm -> sparse MoE + residual] -> RMSNorm -> lm_head.  First
pipeline stage owns the embedding, last stage the final norm and lm_head; the others hold
``nn.Identity`` there.  Loss = shifted cross entropy + ``router_aux_loss_coef`` x load-balance
loss over the local layers' router logits (+ optional z-loss, off by default).

One class serves both reference files: with ``virtual_pipeline_parallelism == 1`` it behaves
like modeling_olmoe.py, otherwise ``forward(..., vp_ind)`` runs one virtual chunk like
modeling_olmoe_new.py (local layer l of chunk v is global layer ``(v*PP + pp_ind)*LV + l``).
Every hot op goes through ``optimus_lm_b200.ops`` (tcgen05 GEMMs, fused norm/rope/router/MoE/CE
kernels) instead of eager torch ops.
"""
from __future__ import annotations

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint as torch_activation_checkpoint

from ...ops import functional as OF
from ..common.modeling_rope_utils import RotaryEmbedding
from ..common.moe import FastOlmoeParallelSparseMoeBlock, OlmoeParallelSparseMoeBlock
from ..common.norm_modules import RMSNorm


class OlmoeParallelOutput:
    def __init__(self, loss=None, logits=None, aux_loss=None):
        self.loss = loss
        self.logits = logits
        self.aux_loss = aux_loss


OlmoeParallelRMSNorm = RMSNorm
OlmoeParallelRotaryEmbedding = RotaryEmbedding


class OlmoeParallelAttention(nn.Module):
    def __init__(self, config, pmap=None):
        super().__init__()
        self.config = config
        self.pmap = pmap
        self.hidden_size = config.hidden_size
        self.num_attention_heads = config.num_attention_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        self.num_key_value_groups = self.num_attention_heads // self.num_key_value_heads
        hq, hkv = self.num_attention_heads * self.head_dim, self.num_key_value_heads * self.head_dim
        self.q_proj = nn.Linear(self.hidden_size, hq, bias=False)
        self.k_proj = nn.Linear(self.hidden_size, hkv, bias=False)
        self.v_proj = nn.Linear(self.hidden_size, hkv, bias=False)
        self.o_proj = nn.Linear(hq, self.hidden_size, bias=False)
        self.q_norm = RMSNorm(hq, eps=config.rms_norm_eps)
        self.k_norm = RMSNorm(hkv, eps=config.rms_norm_eps)

    def forward(self, hidden_states, position_embeddings):
        B, S, _ = hidden_states.shape
        q = OF.linear(hidden_states, self.q_proj.weight)
        k = OF.linear(hidden_states, self.k_proj.weight)
        v = OF.linear(hidden_states, self.v_proj.weight)
        if not self.config.skip_qk_norm:
            q = self.q_norm(q)
            k = self.k_norm(k)
        if self.config.clip_qkv is not None:
            c = self.config.clip_qkv
            q, k, v = q.clamp(-c, c), k.clamp(-c, c), v.clamp(-c, c)
        cos, sin = position_embeddings
        q = OF.rope(q, cos, sin, heads=self.num_attention_heads)     # on the projection output, not on a view
        k = OF.rope(k, cos, sin, heads=self.num_key_value_heads)
        q = q.view(B, S, self.num_attention_heads, self.head_dim)
        k = k.view(B, S, self.num_key_value_heads, self.head_dim)
        v = v.view(B, S, self.num_key_value_heads, self.head_dim)
        o = OF.attention(q, k, v, causal=True)
        return OF.linear(o.reshape(B, S, self.num_attention_heads * self.head_dim), self.o_proj.weight)

    def set_parameters_from_full_module(self, module):
        self.load_state_dict(module.state_dict())


class OlmoeParallelDecoderLayer(nn.Module):
    def __init__(self, config, layer_idx=0, pmap=None, memory_tracker=None):
        super().__init__()
        self.self_attn = OlmoeParallelAttention(config, pmap=pmap)
        block = FastOlmoeParallelSparseMoeBlock if config.use_fast_moe else OlmoeParallelSparseMoeBlock
        self.mlp = block(config, pmap=pmap)
        self.input_layernorm = RMSNorm(config.hidden_size)
        self.post_attention_layernorm = RMSNorm(config.hidden_size)
        self.layer_idx = layer_idx
        self.memory_tracker = memory_tracker
        self.config = config
        lvl = config.activation_checkpointing_level if config.use_activation_checkpointing else 0
        self.ckpt_attn = bool(lvl & 2)
        self.ckpt_norm = bool(lvl & 4)

    def _log(self, what):
        if self.memory_tracker is not None:
            self.memory_tracker.log(f"L{self.layer_idx} {what}")

    def _maybe_ckpt(self, on, fn, *args):
        if on and torch.is_grad_enabled():
            return torch_activation_checkpoint(fn, *args, use_reentrant=False)
        return fn(*args)

    def forward(self, hidden_states, position_embeddings, residual=None, defer_add=False):
        """One decoder layer.  With ``defer_add`` the layer returns ``(mlp_out, residual, router_logits)`` without the
        last residual add, and accepts such a pair as input: every residual add then runs inside the RMSNorm kernel
        that follows it (the next layer's input norm, or the model's final norm)."""
        self._log("Before Decoder")
        fused = defer_add and not self.ckpt_norm
        if residual is None:
            residual = hidden_states
            h = self._maybe_ckpt(self.ckpt_norm, self.input_layernorm, hidden_states)
        elif fused:
            residual, h = self.input_layernorm.forward_add(hidden_states, residual)
        else:
            residual = hidden_states + residual
            h = self._maybe_ckpt(self.ckpt_norm, self.input_layernorm, residual)
        self._log("Before Attention")
        h = self._maybe_ckpt(self.ckpt_attn, self.self_attn, h, position_embeddings)
        self._log("After Attention")
        if fused:
            residual, h = self.post_attention_layernorm.forward_add(h, residual)
        else:
            residual = h + residual
            h = self._maybe_ckpt(self.ckpt_norm, self.post_attention_layernorm, residual)
        self._log("Before MoE")
        h, router_logits = self.mlp(h)
        self._log("After MoE")
        if defer_add:
            return h, residual, router_logits
        hidden_states = h + residual
        self._log("After decoder")
        return hidden_states, router_logits

    def set_parameters_from_full_module(self, module):
        self.self_attn.set_parameters_from_full_module(module.self_attn)
        self.mlp.set_parameters_from_full_module(module.mlp)
        self.input_layernorm.load_state_dict(module.input_layernorm.state_dict())
        self.post_attention_layernorm.load_state_dict(module.post_attention_layernorm.state_dict())


class OlmoeParallelModel(nn.Module):
    def __init__(self, config, pmap=None, memory_tracker=None):
        super().__init__()
        self.pmap = pmap
        self.config = config
        self.memory_tracker = memory_tracker
        self.num_hidden_layers = config.num_hidden_layers
        self.padding_idx = config.padding_idx
        self.vocab_size = config.vocab_size
        self.hidden_size = config.hidden_size
        PP = pmap.pipeline_parallelism
        self.VPP = getattr(config, "virtual_pipeline_parallelism", 1)

        if pmap.is_first_stage_rank:
            self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        else:
            self.embed_tokens = nn.Identity()

        self.num_hidden_layers_per_rank = config.num_hidden_layers // PP
        self.num_layers_per_virtual_stage = self.num_hidden_layers_per_rank // self.VPP
        self.layer_start_idx = pmap.pp_ind * self.num_hidden_layers_per_rank
        self.layer_end_idx = self.layer_start_idx + self.num_hidden_layers_per_rank
        self.layers = nn.ModuleList([
            OlmoeParallelDecoderLayer(config, layer_idx=self.global_layer_index(l), pmap=pmap,
                                      memory_tracker=memory_tracker)
            for l in range(self.num_hidden_layers_per_rank)])

        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps) if pmap.is_last_stage_rank else nn.Identity()
        self.rotary_emb = RotaryEmbedding(config)
        lvl = config.activation_checkpointing_level if config.use_activation_checkpointing else 0
        self.ckpt_norm = bool(lvl & 4)

    def global_layer_index(self, local_idx: int) -> int:
        """Global index of local layer ``local_idx`` (contiguous block per stage, or round-robin
        chunks of ``LV`` layers under virtual pipelining)."""
        if self.VPP == 1:
            return self.pmap.pp_ind * self.num_hidden_layers_per_rank + local_idx
        LV = self.num_layers_per_virtual_stage
        v, lv = divmod(local_idx, LV)
        return (v * self.pmap.pipeline_parallelism + self.pmap.pp_ind) * LV + lv

    def forward(self, inputs, vp_ind=None):
        first_chunk = vp_ind is None or vp_ind == 0
        last_chunk = vp_ind is None or vp_ind == self.VPP - 1
        hidden_states = OF.embed(self.embed_tokens, inputs) if first_chunk else inputs
        S = hidden_states.size(1)
        position_embeddings = self.rotary_emb.table(S, hidden_states.device)

        layers = self.layers
        if vp_ind is not None and self.VPP > 1:
            LV = self.num_layers_per_virtual_stage
            layers = self.layers[vp_ind * LV:(vp_ind + 1) * LV]
        router_logits = []
        residual = None
        for layer in layers:
            hidden_states, residual, rl = layer(hidden_states, position_embeddings, residual, defer_add=True)
            router_logits.append(rl)
        if last_chunk and isinstance(self.norm, RMSNorm) and residual is not None and not self.ckpt_norm:
            _, hidden_states = self.norm.forward_add(hidden_states, residual)   # last residual add inside the final norm
            return hidden_states, tuple(router_logits)
        if residual is not None:
            hidden_states = hidden_states + residual
        if last_chunk:
            if self.ckpt_norm and torch.is_grad_enabled():
                hidden_states = torch_activation_checkpoint(self.norm, hidden_states, use_reentrant=False)
            else:
                hidden_states = self.norm(hidden_states)
        return hidden_states, tuple(router_logits)

    def set_parameters_from_full_module(self, module):
        if self.pmap.is_first_stage_rank:
            self.embed_tokens.load_state_dict(module.embed_tokens.state_dict())
        for l in range(self.num_hidden_layers_per_rank):
            self.layers[l].set_parameters_from_full_module(module.layers[self.global_layer_index(l)])
        if self.pmap.is_last_stage_rank:
            self.norm.load_state_dict(module.norm.state_dict())


class OlmoeParallelForCausalLM(nn.Module):
    def __init__(self, config, pmap=None, memory_tracker=None):
        super().__init__()
        if pmap is None:
            from ...mapper import ParallelDpPpEpTpMapper
            pmap = ParallelDpPpEpTpMapper()
        self.config = config
        self.pmap = pmap
        self.memory_tracker = memory_tracker
        self.vocab_size = config.vocab_size
        self.num_experts = config.num_experts
        self.num_experts_per_tok = config.num_experts_per_tok
        self.router_aux_loss_coef = config.router_aux_loss_coef
        self.router_z_loss_coef = getattr(config, "router_z_loss_coef", 0.0)
        self.model = OlmoeParallelModel(config, pmap=pmap, memory_tracker=memory_tracker)
        self.lm_head = (nn.Linear(config.hidden_size, config.vocab_size, bias=False)
                        if pmap.is_last_stage_rank else nn.Identity())
        self.output_router_logits = config.output_router_logits
        self.use_local_router_aux_loss = config.use_local_router_aux_loss
        self.VPP = getattr(config, "virtual_pipeline_parallelism", 1)
        self.inplace_ce_backward = True

    def loss_function(self, logits, labels, vocab_size=None):
        return OF.shifted_cross_entropy(logits, labels, inplace_backward=self.inplace_ce_backward)

    def aux_loss_from_router(self, router_logits, layers=None):
        """``coef * load-balance (+ z)`` over the given router logits; uses the router kernels'
        statistics of ``layers`` when they are the producers of ``router_logits``."""
        router_logits = [r for r in router_logits if r is not None]
        if not router_logits:
            return None
        idx = stats = None
        if layers is not None:
            idx = [l.mlp.last_router_indices for l in layers]
            stats = [l.mlp.last_router_stats for l in layers]
            if any(s is None for s in stats) or len(stats) != len(router_logits):
                idx = stats = None
        return OF.router_aux_loss(router_logits, idx, stats, self.num_experts, self.num_experts_per_tok,
                                  layer_level=self.use_local_router_aux_loss, aux_coef=self.router_aux_loss_coef,
                                  z_coef=self.router_z_loss_coef)

    def forward(self, input_ids, labels=None, vp_ind=None):
        hidden_states, router_logits = self.model(input_ids, vp_ind=vp_ind)
        PP = self.pmap.pipeline_parallelism
        last_chunk = vp_ind is None or vp_ind == self.VPP - 1
        is_output_stage = self.pmap.is_last_stage_rank and last_chunk
        if self.VPP > 1 and vp_ind is not None:
            # virtual-pipeline contract: raw tensors between chunks, logits from the last one
            return self.lm_head(hidden_states) if is_output_stage else hidden_states
        if PP > 1 and not self.pmap.is_last_stage_rank:
            return {"output": hidden_states, "router_logits": router_logits}
        logits = OF.linear(hidden_states, self.lm_head.weight)
        if PP > 1:
            return {"output": logits, "router_logits": router_logits}

        loss = None
        if labels is not None:
            loss = self.loss_function(logits, labels, self.vocab_size)
        aux_loss = None
        if self.output_router_logits:
            aux_loss = self.aux_loss_from_router(router_logits, self.model.layers)
            if labels is not None and aux_loss is not None:
                loss = loss + aux_loss.to(loss.dtype)
        return OlmoeParallelOutput(loss=loss, logits=logits, aux_loss=aux_loss)

    def set_parameters_from_full_module(self, module):
        self.model.set_parameters_from_full_module(module.model)
        if self.pmap.is_last_stage_rank:
            self.lm_head.load_state_dict(module.lm_head.state_dict())

    def get_flops(self, context_size):
        """Analytical training FLOPs per sequence for this rank's stage (the reference's model,
        modeling_olmoe.py:580-630, including its factor-6 attention terms)."""
        c = self.config
        hd = getattr(c, "head_dim", None) or c.hidden_size // c.num_attention_heads
        S = context_size
        attn = 6 * S * c.hidden_size * (c.num_attention_heads * hd) * 2          # q and o
        attn += 6 * S * c.hidden_size * (c.num_key_value_heads * hd) * 2         # k and v
        attn += 2 * 6 * c.num_attention_heads * S * S * hd                       # QK^T and PV
        mlp = 3 * c.num_experts_per_tok * 6 * S * c.hidden_size * c.intermediate_size
        if c.use_activation_checkpointing:
            if c.activation_checkpointing_level & 1:
                attn = int((4 / 3) * attn)
            if c.activation_checkpointing_level & 2:
                mlp = int((4 / 3) * mlp)
        total = (c.num_hidden_layers // self.pmap.pipeline_parallelism) * (attn + mlp)
        if self.pmap.is_last_stage_rank:
            total += 6 * S * c.hidden_size * c.vocab_size
        return total

    def get_ep_replicated_param_list(self):
        """Names of the parameters that are identical on all ranks of an EP group (everything
        except the experts), in the reference's order (modeling_olmoe.py:632-661)."""
        names = ["model.embed_tokens.weight"]
        n = len(self.model.layers)
        for i in range(n):
            names += [f"model.layers.{i}.self_attn.{p}.weight" for p in
                      ("q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm")]
        names += [f"model.layers.{i}.mlp.gate.weight" for i in range(n)]
        for i in range(n):
            names += [f"model.layers.{i}.input_layernorm.weight", f"model.layers.{i}.post_attention_layernorm.weight"]
        names += ["model.norm.weight", "lm_head.weight"]
        return names
