"""OLMo: dense decoder with non-parametric LayerNorm (or RMSNorm via the ``RMS`` tag), SwiGLU,
optional clip_qkv; tensor-, pipeline- and virtual-pipeline parallel.  Reference:
optimus/models/olmo/modeling_olmo.py:19-525.  ``lm_head`` is always its own parameter (no
weight tying, also with the ``TWE`` tag - as in the reference).  Pipeline stages exchange raw
tensors (``forward(input_ids, vp_ind, labels)``)."""
from ..common.dense_decoder import (CausalLMOutput, ParallelAttention, ParallelDecoderLayer, ParallelDenseForCausalLM,
                                    ParallelDenseModel, ParallelMLP)
from ..common.norm_modules import NonParametricLayerNorm as OlmoLayerNorm, RMSNorm as OlmoParallelRMSNorm  # noqa: F401


class OlmoParallelOutput(CausalLMOutput):
    pass


OlmoParallelMLP = ParallelMLP
OlmoParallelAttention = ParallelAttention
OlmoParallelDecoderLayer = ParallelDecoderLayer
OlmoParallelModel = ParallelDenseModel


class OlmoParallelForCausalLM(ParallelDenseForCausalLM):
    family = "olmo"
    pp_dict_outputs = False
    output_class = OlmoParallelOutput
