"""Llama: dense decoder with RMSNorm (eps from the config), grouped-query attention, SwiGLU;
tensor- and pipeline-parallel.  Reference: optimus/models/llama/modeling_llama.py:24-485.
Pipeline stages return ``{"output": tensor, "router_logits": None}`` (the contract of the
GPipe / 1F1B trainer); activation checkpointing supports level 4 (norms) only."""
from ..common.dense_decoder import (CausalLMOutput, ParallelAttention, ParallelDecoderLayer, ParallelDenseForCausalLM,
                                    ParallelDenseModel, ParallelMLP)
from ..common.norm_modules import RMSNorm as LlamaParallelRMSNorm  # noqa: F401


class LlamaParallelOutput(CausalLMOutput):
    pass


LlamaParallelMLP = ParallelMLP
LlamaParallelAttention = ParallelAttention
LlamaParallelDecoderLayer = ParallelDecoderLayer
LlamaParallelModel = ParallelDenseModel


class LlamaParallelForCausalLM(ParallelDenseForCausalLM):
    family = "llama"
    pp_dict_outputs = True
    output_class = LlamaParallelOutput

    def forward(self, input_ids, labels=None, vp_ind=0):
        return super().forward(input_ids, vp_ind=vp_ind, labels=labels)
