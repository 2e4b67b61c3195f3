"""All-gather -> GEMM and GEMM -> reduce-scatter over peer memory for the tensor-parallel style
paths (the EP-sharded dense MLP of DeepSeek-V3, OLMo/Llama TP blocks)."""
from __future__ import annotations


def usable(x, group) -> bool:
    """True when the fused peer-memory path can run for ``x`` on ``group``."""
    return False
