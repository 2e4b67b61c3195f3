from .configuration_llama import LlamaParallelConfig  # noqa: F401
from .modeling_llama import LlamaParallelForCausalLM, LlamaParallelModel  # noqa: F401
