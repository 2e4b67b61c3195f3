from .configuration_olmoe import OlmoeParallelConfig  # noqa: F401
from .modeling_olmoe import (OlmoeParallelAttention, OlmoeParallelDecoderLayer, OlmoeParallelForCausalLM,  # noqa: F401
                             OlmoeParallelModel, OlmoeParallelRMSNorm)
