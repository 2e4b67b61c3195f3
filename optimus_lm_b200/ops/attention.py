"""Causal attention dispatch.

``flash_attention(q, k, v)`` takes ``[B, S, H, D]`` tensors (k/v may have fewer heads - GQA -
and v may have a different head dim - MLA).  bf16 CUDA inputs run the tcgen05 flash-attention
kernels of csrc/attention.cu; anything else runs the eager fp32-softmax oracle, which is how
the reference's DeepSeek-V3 attention is written
(optimus/models/deepseek_v3/modeling_deepseek_v3.py:359-369; OLMoE/OLMo/Llama call
``F.scaled_dot_product_attention(is_causal=True)``, optimus/models/olmoe/modeling_olmoe.py:219-227).
"""
from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from ._ext import extension, use_kernels
from . import functional as OF


def _kernel_supported(q, k, v) -> bool:
    C = extension()
    if not hasattr(C, "attn_fwd"):
        return False
    D, Dv = q.shape[-1], v.shape[-1]
    return (q.dtype == torch.bfloat16 and D in (64, 128, 192) and Dv in (64, 128) and q.shape[1] % 128 == 0
            and os.environ.get("OLB_ATTENTION", "kernel") == "kernel")


class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        C = extension()
        B, S, Hq, D = q.shape
        Dv = v.shape[-1]
        o = torch.empty((B, S, Hq, Dv), dtype=q.dtype, device=q.device)
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)
        C.attn_fwd(q, k, v, o, lse, scale, OF.status_word(q.device))
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        C = extension()
        q, k, v, o, lse = ctx.saved_tensors
        do = do.contiguous()
        if not hasattr(C, "attn_bwd") or os.environ.get("OLB_ATTENTION_BWD", "kernel") != "kernel":
            # library backward (recomputes the forward): used until the backward kernels cover the shape
            with torch.enable_grad():
                qq, kk, vv = (t.detach().requires_grad_() for t in (q, k, v))
                if q.shape[-1] == v.shape[-1]:
                    out = _sdpa(qq, kk, vv, ctx.scale, True)
                else:
                    out = OF.attention_reference(qq, kk, vv, ctx.scale, True)
            return torch.autograd.grad(out, (qq, kk, vv), do) + (None,)
        dq = torch.empty_like(q)
        dk = torch.empty_like(k)
        dv = torch.empty_like(v)
        C.attn_bwd(q, k, v, o, lse, do, dq, dk, dv, ctx.scale, OF.status_word(q.device))
        return dq, dk, dv, None


def _sdpa(q, k, v, scale, causal):
    Hq, Hkv = q.shape[2], k.shape[2]
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if Hq != Hkv:
        kh = kh.repeat_interleave(Hq // Hkv, dim=1)
        vh = vh.repeat_interleave(Hq // Hkv, dim=1)
    o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal, scale=scale)
    return o.transpose(1, 2).contiguous()


def flash_attention(q, k, v, scale=None, causal=True):
    scale = float(scale) if scale is not None else q.shape[-1] ** -0.5
    if q.is_cuda and causal and use_kernels(q, k, v) and _kernel_supported(q, k, v):
        return _FlashAttnFn.apply(q, k, v, scale)
    if q.is_cuda and q.shape[-1] == v.shape[-1]:
        # shapes the kernels do not cover (odd head dims / sequence lengths)
        return _sdpa(q, k, v, scale, causal)
    return OF.attention_reference(q, k, v, scale, causal)
