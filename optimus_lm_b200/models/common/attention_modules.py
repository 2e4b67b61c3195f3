"""Shared tensor-parallel attention module and its helpers under the reference's module path
(optimus/models/common/attention_modules.py:10-110).  The implementation is ``dense_decoder.ParallelAttention``
(column-parallel q/k/v, row-parallel o, optional full-width QK norm, fused RoPE and flash-attention kernels)."""
import torch

from .dense_decoder import ParallelAttention  # noqa: F401
from .modeling_rope_utils import apply_rotary_pos_emb, rotate_half  # noqa: F401


def repeat_kv(hidden_states: torch.Tensor, n_rep: int) -> torch.Tensor:
    """``[B, H_kv, S, D] -> [B, H_kv * n_rep, S, D]`` (the attention kernels take grouped heads directly; this is
    for code that materialises the repeated heads)."""
    if n_rep == 1:
        return hidden_states
    b, h, s, d = hidden_states.shape
    return hidden_states[:, :, None, :, :].expand(b, h, n_rep, s, d).reshape(b, h * n_rep, s, d)
