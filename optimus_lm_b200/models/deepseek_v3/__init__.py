from .configuration_deepseek_v3 import DeepseekV3ParallelConfig  # noqa: F401
from .modeling_deepseek_v3 import DeepseekV3ParallelForCausalLM, DeepseekV3ParallelModel  # noqa: F401
