from .configuration_olmo import OlmoParallelConfig  # noqa: F401
from .modeling_olmo import OlmoParallelForCausalLM, OlmoParallelModel  # noqa: F401
