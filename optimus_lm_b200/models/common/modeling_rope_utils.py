"""Rotary position embedding parameters: default, linear, dynamic-NTK and YaRN.

Covers the reference's optimus/models/common/modeling_rope_utils.py:11-194 (inverse
frequency initialisers, config validation, the ``dynamic_rope_update`` decorator) and
optimus/models/deepseek_v3/rope_utils.py:5-96 (YaRN and the interleaved application).

Unlike the reference, which recomputes cos/sin with a matmul on every forward, the
``RotaryEmbedding`` module here caches one ``[max_positions, rot_dim]`` fp32 table per
device (cos and sin) and hands out slices; the fused RoPE kernel reads that table.
"""
from __future__ import annotations

import functools
import math
from typing import Optional, Tuple

import torch
from torch import nn


def _rot_dim(config) -> Tuple[float, int]:
    base = config.rope_theta
    partial = getattr(config, "partial_rotary_factor", 1.0)
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
    return base, int(head_dim * partial)


def _compute_default_rope_parameters(config, device=None, seq_len=None):
    base, dim = _rot_dim(config)
    exponent = torch.arange(0, dim, 2, dtype=torch.int64).to(device=device, dtype=torch.float) / dim
    return 1.0 / (base ** exponent), 1.0


def _compute_linear_scaling_rope_parameters(config, device=None, seq_len=None):
    inv_freq, attention_factor = _compute_default_rope_parameters(config, device, seq_len)
    return inv_freq / config.rope_scaling["factor"], attention_factor


def _compute_dynamic_ntk_parameters(config, device=None, seq_len=None):
    base, dim = _rot_dim(config)
    max_pos = config.max_position_embeddings
    factor = config.rope_scaling["factor"]
    seq_len = max(seq_len, max_pos) if seq_len is not None else max_pos
    base = base * ((factor * seq_len / max_pos) - (factor - 1)) ** (dim / (dim - 2))
    exponent = torch.arange(0, dim, 2, dtype=torch.int64).to(device=device, dtype=torch.float) / dim
    return 1.0 / (base ** exponent), 1.0


def yarn_get_mscale(scale=1, mscale=1):
    if scale <= 1:
        return 1.0
    return 0.1 * mscale * math.log(scale) + 1.0


def _compute_yarn_parameters(config, device=None, seq_len=None):
    base, dim = _rot_dim(config)
    rs = config.rope_scaling
    factor = rs["factor"]
    attention_factor = rs.get("attention_factor")
    mscale, mscale_all_dim = rs.get("mscale"), rs.get("mscale_all_dim")
    orig_max = rs.get("original_max_position_embeddings") or config.max_position_embeddings
    if attention_factor is None:
        if mscale and mscale_all_dim:
            attention_factor = float(yarn_get_mscale(factor, mscale) / yarn_get_mscale(factor, mscale_all_dim))
        else:
            attention_factor = yarn_get_mscale(factor)
    beta_fast = rs.get("beta_fast") or 32
    beta_slow = rs.get("beta_slow") or 1

    def correction_dim(num_rotations):
        return (dim * math.log(orig_max / (num_rotations * 2 * math.pi))) / (2 * math.log(base))

    low, high = correction_dim(beta_fast), correction_dim(beta_slow)
    if rs.get("truncate", True):
        low, high = math.floor(low), math.ceil(high)
    low, high = max(low, 0), min(high, dim - 1)
    if low == high:
        high += 0.001
    ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low), 0, 1)
    extrapolation_weight = (1 - ramp).to(device=device, dtype=torch.float)

    pos_freqs = base ** (torch.arange(0, dim, 2).to(device=device, dtype=torch.float) / dim)
    inv_extra = 1.0 / pos_freqs
    inv_inter = 1.0 / (factor * pos_freqs)
    inv_freq = inv_inter * (1 - extrapolation_weight) + inv_extra * extrapolation_weight
    return inv_freq, attention_factor


ROPE_INIT_FUNCTIONS = {
    "default": _compute_default_rope_parameters,
    "linear": _compute_linear_scaling_rope_parameters,
    "dynamic": _compute_dynamic_ntk_parameters,
    "yarn": _compute_yarn_parameters,
}


def rope_type_of(config) -> str:
    rs = getattr(config, "rope_scaling", None)
    if rs is None:
        return "default"
    return rs.get("rope_type", rs.get("type", "default"))


# ----------------------------------------------------------------------------- validation
def _check_received_keys(rope_type, received, required, optional=None, ignore_keys=None):
    received = set(received)
    if "type" in received:
        received -= {"type"}
        required = set(required) | {"rope_type"} if "rope_type" in received else set(required)
        received |= {"rope_type"}
    if ignore_keys is not None:
        received -= set(ignore_keys)
    missing = set(required) - received
    if missing:
        raise KeyError(f"Missing required keys in `rope_scaling` for 'rope_type'='{rope_type}': {missing}")
    unused = received - set(required) - (set(optional) if optional else set())
    if unused:
        import warnings
        warnings.warn(f"Unrecognized keys in `rope_scaling` for 'rope_type'='{rope_type}': {unused}")


def _validate_default_rope_parameters(config, ignore_keys=None):
    rs = config.rope_scaling
    _check_received_keys(rope_type_of(config), rs.keys(), {"rope_type"}, ignore_keys=ignore_keys)


def _validate_factor(config, ignore_keys, optional=None):
    rs = config.rope_scaling
    _check_received_keys(rope_type_of(config), rs.keys(), {"rope_type", "factor"}, optional, ignore_keys)
    factor = rs["factor"]
    if factor is None or not isinstance(factor, float) or factor < 1.0:
        import warnings
        warnings.warn(f"`rope_scaling`'s factor field must be a float >= 1, got {factor}")


def _validate_linear_scaling_rope_parameters(config, ignore_keys=None):
    _validate_factor(config, ignore_keys)


def _validate_dynamic_scaling_rope_parameters(config, ignore_keys=None):
    _validate_factor(config, ignore_keys, optional={"original_max_position_embeddings"})


def _validate_yarn_parameters(config, ignore_keys=None):
    _validate_factor(config, ignore_keys, optional={"attention_factor", "beta_fast", "beta_slow", "mscale",
                                                    "mscale_all_dim", "original_max_position_embeddings",
                                                    "truncate"})


ROPE_VALIDATION_FUNCTIONS = {
    "default": _validate_default_rope_parameters,
    "linear": _validate_linear_scaling_rope_parameters,
    "dynamic": _validate_dynamic_scaling_rope_parameters,
    "yarn": _validate_yarn_parameters,
}


def rope_config_validation(config, ignore_keys: Optional[set] = None):
    rs = getattr(config, "rope_scaling", None)
    if rs is None:
        return
    fn = ROPE_VALIDATION_FUNCTIONS.get(rope_type_of(config))
    if fn is None:
        import warnings
        warnings.warn(f"Missing validation function mapping in `ROPE_VALIDATION_FUNCTIONS` for '{rope_type_of(config)}'")
        return
    fn(config, ignore_keys=ignore_keys)


# ----------------------------------------------------------------------------- dynamic update
def dynamic_rope_update(rope_forward):
    """Decorator for a rotary module's ``forward(x, position_ids)``: for ``dynamic`` RoPE
    the inverse frequencies grow when a longer sequence shows up and shrink back to the
    original ones afterwards (reference modeling_rope_utils.py:11-43)."""

    @functools.wraps(rope_forward)
    def wrapper(self, x, position_ids):
        if "dynamic" in getattr(self, "rope_type", ""):
            seq_len = int(position_ids.max()) + 1
            if seq_len > self.max_seq_len_cached:
                inv_freq, self.attention_scaling = self.rope_init_fn(self.config, x.device, seq_len=seq_len)
                self.register_buffer("inv_freq", inv_freq, persistent=False)
                self.max_seq_len_cached = seq_len
                self._table = None
            elif seq_len < self.original_max_seq_len < self.max_seq_len_cached:
                self.register_buffer("inv_freq", self.original_inv_freq.to(x.device), persistent=False)
                self.max_seq_len_cached = self.original_max_seq_len
                self._table = None
        return rope_forward(self, x, position_ids)

    return wrapper


class RotaryEmbedding(nn.Module):
    """cos/sin provider with a cached table.

    ``forward(x, position_ids)`` returns ``(cos, sin)`` of shape ``[B, S, rot_dim]`` in
    ``x.dtype`` exactly like the reference rotary modules
    (optimus/models/olmoe/modeling_olmoe.py:130-161); ``table(seq_len, device)`` returns the
    fp32 ``[seq_len, rot_dim]`` pair that the fused kernels consume.
    """

    def __init__(self, config, device=None):
        super().__init__()
        self.config = config
        self.rope_type = rope_type_of(config)
        self.max_seq_len_cached = config.max_position_embeddings
        self.original_max_seq_len = config.max_position_embeddings
        self.rope_init_fn = ROPE_INIT_FUNCTIONS[self.rope_type]
        inv_freq, self.attention_scaling = self.rope_init_fn(config, device)
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self.original_inv_freq = self.inv_freq
        self._table = None

    def table(self, seq_len: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        t = self._table
        if t is None or t[0].shape[0] < seq_len or t[0].device != torch.device(device):
            n = max(seq_len, self.max_seq_len_cached)
            pos = torch.arange(n, device=device, dtype=torch.float32)
            freqs = torch.outer(pos, self.inv_freq.to(device=device, dtype=torch.float32))
            emb = torch.cat((freqs, freqs), dim=-1)
            t = ((emb.cos() * self.attention_scaling).contiguous(), (emb.sin() * self.attention_scaling).contiguous())
            self._table = t
        return t[0][:seq_len], t[1][:seq_len]

    @torch.no_grad()
    @dynamic_rope_update
    def forward(self, x, position_ids):
        seq_len = position_ids.shape[-1]
        cos, sin = self.table(int(self.max_seq_len_cached if seq_len <= self.max_seq_len_cached else seq_len), x.device)
        cos = cos[position_ids].to(x.dtype)
        sin = sin[position_ids].to(x.dtype)
        return cos, sin


def rotate_half(x):
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary_pos_emb(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    """Half-rotate RoPE on ``[B, h, S, d]`` tensors (reference modeling_olmoe.py:107-119)."""
    cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
    return q * cos + rotate_half(q) * sin, k * cos + rotate_half(k) * sin


def deinterleave_last_dim(x):
    """``[x0, x1, x2, x3, ...] -> [x0, x2, ..., x1, x3, ...]`` on the last dim."""
    *lead, d = x.shape
    return x.reshape(*lead, d // 2, 2).transpose(-1, -2).reshape(*lead, d)


def apply_rotary_pos_emb_interleave(q, k, cos, sin, position_ids=None, unsqueeze_dim=1):
    """DeepSeek-V3 RoPE: de-interleave pairs, then half-rotate; the result stays in the
    de-interleaved order (reference deepseek_v3/rope_utils.py:79-91)."""
    return apply_rotary_pos_emb(deinterleave_last_dim(q), deinterleave_last_dim(k), cos, sin,
                                unsqueeze_dim=unsqueeze_dim)
