"""Autograd ops of the framework.

Each op has two implementations with identical semantics:

* the sm_100a kernels of ``optimus_lm_b200._C`` (tcgen05 GEMMs, fused norm / rope / SwiGLU /
  router / MoE permutation / cross-entropy kernels), used for bf16 CUDA tensors;
* a plain PyTorch version written like the reference's modules, used on CPU (gloo tests)
  and for fp32 runs, and serving as the oracle of the kernel tests.

GEMM operand conventions (see csrc/gemm_tcgen05.cu): forward ``Y = X W^T`` is K-major x
K-major; ``dX = dY W`` reads ``W`` MN-major; ``dW = dY^T X`` reads both operands MN-major,
so no transposed copies are ever materialised.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ._ext import extension, use_kernels

GEMM_DENSE, GEMM_RAGGED_M, GEMM_RAGGED_K = 0, 1, 2

# Device status word per GPU: kernels record bounded-wait timeouts / capacity overflow here.
_STATUS = {}


def status_word(device) -> torch.Tensor:
    device = torch.device(device)
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _STATUS[key] = t
    return t


def check_status(device) -> int:
    """Read (and clear) the device status word; non-zero means a kernel reported a problem."""
    t = status_word(device)
    v = int(t.item())
    if v:
        t.zero_()
    return v


def _kernel_ok(*ts) -> bool:
    return all(t is None or t.dtype == torch.bfloat16 for t in ts) and use_kernels(*[t for t in ts if t is not None])


# ------------------------------------------------------------------------------------ GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, M: int, N: int, K: int, *, a_mn_major=False, b_mn_major=False,
         out: Optional[torch.Tensor] = None, accumulate=False, mode=GEMM_DENSE, meta=None, num_experts=1,
         b_expert_rows=0, c_expert_stride=0, out_dtype=torch.bfloat16, block_n=0, max_ctas=0,
         b2: Optional[torch.Tensor] = None, k_split=0, blk_range: Optional[torch.Tensor] = None,
         pair_rows: bool = False) -> torch.Tensor:
    """Raw tcgen05 GEMM on 2D bf16 views (unit inner stride). See csrc/olb_api.h.  With ``b2`` (same
    layout as ``b``) the K range ``[k_split, K)`` is read from ``b2``: one launch for
    ``a[:, :k_split] @ b + a[:, k_split:] @ b2``.  ``blk_range`` (ragged-M, two int32 on the device) restricts the
    launch to the 128-row blocks ``[blk_range[0], blk_range[1])``.  ``pair_rows`` (ragged-M): the expert groups are padded
    to 256 rows, so two CTAs on neighbouring SMs may share a 256-row tile (``cta_group::2``)."""
    if out is None:
        assert not accumulate
        shape = (num_experts, M, N) if mode == GEMM_RAGGED_K else (M, N)
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    extension().gemm(a, b, out, M, N, K, a_mn_major, b_mn_major, accumulate, mode, meta, num_experts,
                     b_expert_rows, c_expert_stride, status_word(a.device), block_n, max_ctas, b2, k_split, blk_range,
                     pair_rows)
    return out


def _as_2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    return x2


class DirectGrad:
    """Gradient buffer of one weight that the weight-gradient GEMMs write (or accumulate into) themselves.

    Autograd's own route - materialise ``dW``, then ``AccumulateGrad`` adds it into a zeroed ``.grad`` - moves
    the weight gradient through memory four times (memset, GEMM store, read-add-write).  With a ``DirectGrad``
    attached to a parameter (``enable_direct_grads``) the GEMM epilogue stores straight into the ``.grad`` view
    of the optimizer's flat buffer: the first gradient of an optimizer step overwrites, later ones (gradient
    accumulation, pipeline micro-batches) accumulate, and the autograd function returns no gradient."""

    __slots__ = ("buf", "ready")

    def __init__(self, buf: torch.Tensor):
        self.buf = buf
        self.ready = False   # False: buffer content is stale, the next gradient overwrites it


def enable_direct_grads(params):
    """Attach a ``DirectGrad`` to every bf16 CUDA weight matrix whose ``.grad`` is preallocated (a view of a flat
    buffer).  Returns (holders, other_grads): the caller resets the holders and zeroes ``other_grads`` at the
    start of an optimizer step instead of zeroing everything."""
    holders, others = [], []
    for p in params:
        if p.grad is None:
            continue
        if p.is_cuda and p.dtype == torch.bfloat16 and p.dim() >= 2 and p.grad.dtype == torch.bfloat16 \
                and p.grad.is_contiguous() and p.grad.data_ptr() % 16 == 0 and getattr(p, "_olb_direct_ok", True):
            h = DirectGrad(p.grad)
            p._olb_direct = h
            holders.append(h)

            # A gradient that still arrives through autograd (a torch op used the weight: embedding lookup,
            # fp32 fall-back, per-expert modules) is added into the buffer by AccumulateGrad; make sure it
            # is added onto zeros, not onto the previous step's data.
            def _guard(grad, h=h):
                if not h.ready:
                    h.buf.zero_()
                    h.ready = True
                return grad

            p.register_hook(_guard)
        else:
            others.append(p.grad)
    return holders, others


def _holder(w):
    return getattr(w, "_olb_direct", None) if torch.is_grad_enabled() else None


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, holder):
        x2 = _as_2d(x)
        M, K = x2.shape
        N = w.shape[0]
        # the result is allocated in its final shape: a view made inside the function could not be modified in
        # place by a later op (the in-place RoPE kernel works on projection outputs)
        y = torch.empty((*x.shape[:-1], N), dtype=x.dtype, device=x.device)
        lazy = getattr(w, "_olb_lazy", None)
        if lazy is not None and lazy.stale:
            # the other ranks' updated parts of this weight come in inside this launch (parameter all-gather fused
            # into the first consuming GEMM), or by a plain copy when the shape is not one the fused launch takes
            if not lazy.gather_gemm(x2, w, y.view(M, N)):
                lazy.materialize(w)
                gemm(x2, w, M, N, K, out=y.view(M, N))
        else:
            gemm(x2, w, M, N, K, out=y.view(M, N))
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        ctx.holder = holder
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        M, K = x2.shape
        N = w.shape[0]
        dy2 = _as_2d(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, M, K, N, b_mn_major=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            h = ctx.holder
            if h is not None:
                gemm(dy2, x2, N, K, M, a_mn_major=True, b_mn_major=True, out=h.buf, accumulate=h.ready)
                h.ready = True
            else:
                dw = gemm(dy2, x2, N, K, M, a_mn_major=True, b_mn_major=True)
        return dx, dw, None


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` for a bias-free projection (reference: nn.Linear -> oneDNN)."""
    if _kernel_ok(x, w) and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0:
        return _LinearFn.apply(x, w, _holder(w))
    lazy = getattr(w, "_olb_lazy", None)
    if lazy is not None and lazy.stale:
        lazy.materialize(w)
    return F.linear(x, w)


# ------------------------------------------------------------------------------------ embedding
class _EmbeddingFn(torch.autograd.Function):
    """Row lookup with an optional vocabulary range (rows outside ``[v_start, v_start + rows)`` give zeros) and a
    deterministic backward that accumulates straight into the weight's gradient buffer when it has one."""

    @staticmethod
    def forward(ctx, ids, w, v_start, padding_idx, holder):
        C = extension()
        flat = ids.reshape(-1).contiguous()
        out = torch.empty((*ids.shape, w.shape[1]), dtype=w.dtype, device=w.device)
        C.embedding_fwd(flat, w, out.view(flat.numel(), w.shape[1]), v_start)
        ctx.save_for_backward(flat)
        ctx.misc = (v_start, -1 if padding_idx is None else int(padding_idx) + v_start, holder, tuple(w.shape))
        return out

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        v_start, pad, holder, wshape = ctx.misc
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        sorted_ids, perm = torch.sort(flat, stable=True)
        C = extension()
        if holder is not None:
            if not holder.ready:
                holder.buf.zero_()
                holder.ready = True
            C.embedding_bwd(sorted_ids, perm, dy2, holder.buf, v_start, pad, True)
            return None, None, None, None, None
        dw = torch.zeros(wshape, dtype=dy.dtype, device=dy.device)
        C.embedding_bwd(sorted_ids, perm, dy2, dw, v_start, pad, False)
        return None, dw, None, None, None


def embedding(ids: torch.Tensor, weight: torch.Tensor, padding_idx=None, v_start: int = 0, masked: bool = False) -> torch.Tensor:
    """``weight[ids - v_start]`` (zeros for ids outside this rank's vocabulary range; ``padding_idx`` is local to the
    weight and receives no gradient; ``masked`` says that ids beyond the weight's rows may occur).  Reference: ``F.embedding`` / ``ParallelEmbedding``
    (optimus/models/common/parallel_modules.py:32-45)."""
    if _kernel_ok(weight) and ids.is_cuda and ids.dtype == torch.long and weight.is_contiguous() \
            and weight.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids, weight, v_start, padding_idx, _holder(weight))
    if v_start == 0 and not masked:
        return F.embedding(ids, weight, padding_idx)
    local = ids - v_start
    outside = (local < 0) | (local >= weight.shape[0])
    out = F.embedding(local.masked_fill(outside, 0), weight, padding_idx)
    return out.masked_fill(outside.unsqueeze(-1), 0.0)


def embed(module, ids):
    """Call an embedding module: ``nn.Embedding`` goes through ``embedding`` (kernel path on bf16 CUDA), anything
    else (``ParallelEmbedding``, ``nn.Identity`` on non-first pipeline stages) is called as is."""
    if isinstance(module, torch.nn.Embedding):
        return embedding(ids, module.weight, module.padding_idx)
    return module(ids)


# ------------------------------------------------------------------------------------ norms
def rms_norm_reference(x, weight, eps):
    """Reference RMSNorm (optimus/models/olmoe/modeling_olmoe.py:93-104)."""
    dt = x.dtype
    h = x.to(torch.float32)
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    h = h.to(dt)
    return weight * h if weight is not None else h


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        C = extension()
        xc = x.contiguous()
        y = torch.empty_like(xc)
        rstd = torch.empty(xc.numel() // xc.shape[-1], dtype=torch.float32, device=x.device)
        C.rmsnorm_fwd(xc, w, y, rstd, eps)
        ctx.save_for_backward(xc, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        C = extension()
        x, w, rstd = ctx.saved_tensors
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        rows, cols = rstd.numel(), x.shape[-1]
        dw = None
        if w is not None and ctx.needs_input_grad[1]:
            nb = C.rmsnorm_bwd_blocks(rows)
            partial = torch.empty((nb, cols), dtype=torch.float32, device=x.device)
            C.rmsnorm_bwd(dy, x, w, rstd, dx, partial)
            dw = torch.empty_like(w)
            C.colsum_finalize(partial, nb, dw, False)
        else:
            C.rmsnorm_bwd(dy, x, w, rstd, dx, None)
        return dx, dw, None


def rms_norm(x, weight, eps=1e-5):
    if _kernel_ok(x, weight) and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, weight, eps)
    return rms_norm_reference(x, weight, eps)


class _AddRMSNormFn(torch.autograd.Function):
    """``h = x + residual`` and ``y = rms_norm(h, w)`` in one kernel; the backward takes the gradients of both outputs and
    returns their combination once: ``d(h) = rmsnorm_bwd(dy) + dh`` is the gradient of ``x`` and of ``residual``."""

    @staticmethod
    def forward(ctx, x, residual, w, eps):
        C = extension()
        xc, rc = x.contiguous(), residual.contiguous()
        h = torch.empty_like(xc)
        y = torch.empty_like(xc)
        rstd = torch.empty(xc.numel() // xc.shape[-1], dtype=torch.float32, device=x.device)
        C.add_rmsnorm_fwd(xc, rc, w, h, y, rstd, eps)
        ctx.save_for_backward(h, w, rstd)
        ctx.set_materialize_grads(False)
        return h, y

    @staticmethod
    def backward(ctx, dh, dy):
        C = extension()
        h, w, rstd = ctx.saved_tensors
        if dy is None:
            return dh, dh, None, None
        dy = dy.contiguous()
        dres = dh.contiguous() if dh is not None else None
        dx = torch.empty_like(h)
        rows, cols = rstd.numel(), h.shape[-1]
        dw = None
        if w is not None and ctx.needs_input_grad[2]:
            nb = C.rmsnorm_bwd_blocks(rows)
            partial = torch.empty((nb, cols), dtype=torch.float32, device=h.device)
            C.rmsnorm_bwd(dy, h, w, rstd, dx, partial, dres)
            dw = torch.empty_like(w)
            C.colsum_finalize(partial, nb, dw, False)
        else:
            C.rmsnorm_bwd(dy, h, w, rstd, dx, None, dres)
        return dx, dx, dw, None


def add_rms_norm(x, residual, weight, eps=1e-5):
    """``(x + residual, rms_norm(x + residual, weight))``: the residual add of a decoder layer fused with the norm that
    follows it (the reference does ``hidden = h + residual`` and the next RMSNorm as separate ops,
    optimus/models/olmoe/modeling_olmoe.py:436-450)."""
    if _kernel_ok(x, residual, weight) and x.shape[-1] % 8 == 0 and x.shape == residual.shape:
        return _AddRMSNormFn.apply(x, residual, weight, eps)
    h = x + residual
    return h, rms_norm_reference(h, weight, eps)


def layer_norm_noaffine_reference(x, eps=1e-5):
    """OLMo's non-parametric LayerNorm in fp32 (optimus/models/olmo/modeling_olmo.py:19-30)."""
    dt = x.dtype
    return F.layer_norm(x.to(torch.float32), (x.shape[-1],), None, None, eps).to(dt)


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, eps):
        C = extension()
        xc = x.contiguous()
        rows = xc.numel() // xc.shape[-1]
        y = torch.empty_like(xc)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        C.layernorm_fwd(xc, y, mean, rstd, eps)
        ctx.save_for_backward(xc, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, mean, rstd = ctx.saved_tensors
        dx = torch.empty_like(x)
        extension().layernorm_bwd(dy.contiguous(), x, mean, rstd, dx)
        return dx, None


def layer_norm_noaffine(x, eps=1e-5):
    if _kernel_ok(x) and x.shape[-1] % 8 == 0:
        return _LayerNormFn.apply(x, eps)
    return layer_norm_noaffine_reference(x, eps)


# ------------------------------------------------------------------------------------ SwiGLU
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        g2, u2 = _as_2d(g), _as_2d(u)
        act = torch.empty((g2.shape[0], g2.shape[1]), dtype=g.dtype, device=g.device)
        extension().swiglu_fwd(g2, u2, act)
        ctx.save_for_backward(g2, u2)
        ctx.shape = g.shape
        return act.view(g.shape)

    @staticmethod
    def backward(ctx, dact):
        g2, u2 = ctx.saved_tensors
        d2 = _as_2d(dact)
        dg = torch.empty((g2.shape[0], g2.shape[1]), dtype=g2.dtype, device=g2.device)
        du = torch.empty_like(dg)
        extension().swiglu_bwd(d2, g2, u2, dg, du)
        return dg.view(ctx.shape), du.view(ctx.shape)


def swiglu(g, u):
    """``silu(g) * u``."""
    if _kernel_ok(g, u) and g.shape[-1] % 8 == 0:
        return _SwiGLUFn.apply(g, u)
    return F.silu(g) * u


# ------------------------------------------------------------------------------------ RoPE
class _RopeFn(torch.autograd.Function):
    """In-place rotary embedding on ``x[..., rot_offset:rot_offset+rot_dim]`` of a ``[B, S, heads, head_dim]``
    tensor, or of a ``[B, S, heads * head_dim]`` tensor when ``heads`` is given.  The second form lets a module
    rotate the projection output itself rather than a view of it: an in-place autograd function on a view makes
    autograd insert a CopySlices node (one more pass over the tensor in the backward)."""

    @staticmethod
    def forward(ctx, x, cos_tab, sin_tab, rot_offset, rot_dim, interleaved, heads):
        x4 = x if heads is None else x.view(x.shape[0], x.shape[1], heads, x.shape[2] // heads)
        B, S, Hn, D = x4.shape
        assert x4.stride(-1) == 1 and x4.stride(2) % 8 == 0 and x4.stride(1) % 8 == 0 and rot_offset % 8 == 0
        assert B == 1 or x4.stride(0) == S * x4.stride(1)
        view = x4[..., rot_offset:]
        extension().rope_inplace(view, x4.stride(1), B * S, Hn, x4.stride(2), rot_dim, S, cos_tab, sin_tab,
                                 interleaved, False)
        ctx.mark_dirty(x)
        ctx.save_for_backward(cos_tab, sin_tab)
        ctx.args = (rot_offset, rot_dim, interleaved, heads)
        return x

    @staticmethod
    def backward(ctx, dy):
        cos_tab, sin_tab = ctx.saved_tensors
        rot_offset, rot_dim, interleaved, heads = ctx.args
        # The incoming gradient is rotated in place when it is a whole contiguous tensor of its own (the usual
        # case: it was just produced by the attention backward and has no other reader); otherwise on a copy.
        own = _ROPE_BWD_INPLACE and dy.is_contiguous() and (dy._base is None or dy._base.numel() == dy.numel())
        dx = dy if own else dy.contiguous().clone()
        d4 = dx if heads is None else dx.view(dx.shape[0], dx.shape[1], heads, dx.shape[2] // heads)
        B, S, Hn, D = d4.shape
        view = d4[..., rot_offset:]
        extension().rope_inplace(view, d4.stride(1), B * S, Hn, d4.stride(2), rot_dim, S, cos_tab, sin_tab,
                                 interleaved, True)
        return dx, None, None, None, None, None, None


_ROPE_BWD_INPLACE = True


def rope_reference(x, cos_tab, sin_tab, rot_offset=0, rot_dim=None, interleaved=False):
    """x: [B, S, heads, head_dim]; cos/sin: [S, rot_dim] fp32."""
    from ..models.common.modeling_rope_utils import deinterleave_last_dim, rotate_half
    rot_dim = rot_dim or (x.shape[-1] - rot_offset)
    xr = x[..., rot_offset:rot_offset + rot_dim]
    if interleaved:
        xr = deinterleave_last_dim(xr)
    cos = cos_tab[None, :, None, :].to(x.dtype)
    sin = sin_tab[None, :, None, :].to(x.dtype)
    out = xr * cos + rotate_half(xr) * sin
    if rot_offset == 0 and rot_dim == x.shape[-1]:
        return out
    return torch.cat([x[..., :rot_offset], out, x[..., rot_offset + rot_dim:]], dim=-1)


def rope(x, cos_tab, sin_tab, rot_offset=0, rot_dim=None, interleaved=False, heads=None):
    """Rotary embedding on a ``[B, S, heads, head_dim]`` tensor, or on ``[B, S, heads * head_dim]`` with ``heads``
    given (returned in the same shape).  May modify ``x`` in place on the kernel path; use the return value."""
    if heads is not None and not (_kernel_ok(x) and cos_tab.is_cuda and x.is_contiguous()):
        B, S, HD = x.shape
        return rope(x.view(B, S, heads, HD // heads), cos_tab, sin_tab, rot_offset, rot_dim, interleaved).reshape(B, S, HD)
    head_dim = x.shape[-1] if heads is None else x.shape[-1] // heads
    rot_dim = rot_dim or (head_dim - rot_offset)
    if _kernel_ok(x) and rot_dim % 16 == 0 and cos_tab.is_cuda:
        return _RopeFn.apply(x, cos_tab.contiguous(), sin_tab.contiguous(), rot_offset, rot_dim, interleaved, heads)
    return rope_reference(x, cos_tab, sin_tab, rot_offset, rot_dim, interleaved)


# ------------------------------------------------------------------------------------ attention
def attention_reference(q, k, v, scale=None, causal=True):
    """q [B,S,Hq,D], k [B,S,Hkv,D], v [B,S,Hkv,Dv] -> [B,S,Hq,Dv]; fp32 softmax, eager."""
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    rep = Hq // Hkv
    scale = scale if scale is not None else D ** -0.5
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if rep > 1:
        kh = kh.repeat_interleave(rep, dim=1)
        vh = vh.repeat_interleave(rep, dim=1)
    s = torch.matmul(qh, kh.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    p = torch.softmax(s, dim=-1, dtype=torch.float32).to(q.dtype)
    return torch.matmul(p, vh).transpose(1, 2).contiguous()


def attention(q, k, v, scale=None, causal=True):
    """Causal attention on ``[B, S, H, D]`` tensors (GQA when ``k`` has fewer heads)."""
    from . import attention as _attn
    return _attn.flash_attention(q, k, v, scale=scale, causal=causal)


# ------------------------------------------------------------------------------------ router
def router_softmax_topk_reference(logits, k, renorm):
    """Reference routing (optimus/models/olmoe/modeling_olmoe.py:295-299); returns fp32 weights
    and int64 indices."""
    p = F.softmax(logits, dim=1, dtype=torch.float)
    w, idx = torch.topk(p, k, dim=-1)
    if renorm:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, idx


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k, renorm, want_stats):
        C = extension()
        T, E = logits.shape
        logits = logits.contiguous()
        w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
        idx = torch.empty((T, k), dtype=torch.int32, device=logits.device)
        if want_stats:
            nb = C.router_blocks(T)
            cnt = torch.empty((nb, E), dtype=torch.float32, device=logits.device)
            prob = torch.empty((nb, E), dtype=torch.float32, device=logits.device)
            lse2 = torch.empty((nb,), dtype=torch.float32, device=logits.device)
            C.router_softmax_topk(logits, k, renorm, w, idx, cnt, prob, lse2)
            stats = torch.cat([cnt.sum(0), prob.sum(0), lse2.sum(0, keepdim=True)])  # [2E+1], fixed order
        else:
            C.router_softmax_topk(logits, k, renorm, w, idx, None, None, None)
            stats = torch.zeros(2 * E + 1, dtype=torch.float32, device=logits.device)
        ctx.save_for_backward(logits, idx)
        ctx.renorm = renorm
        ctx.mark_non_differentiable(idx, stats)
        return w, idx, stats

    @staticmethod
    def backward(ctx, dw, _didx, _dstats):
        logits, idx = ctx.saved_tensors
        dlogits = torch.empty_like(logits)
        extension().router_bwd(logits, idx, dw.contiguous().float(), ctx.renorm, None, None, 0.0, 0.0, dlogits)
        return dlogits, None, None, None


def router_softmax_topk(logits, k, renorm=False, want_stats=True):
    """Returns ``(weights fp32 [T,k], indices [T,k], stats)``.  ``stats`` is a ``[2E+1]`` fp32
    vector (selection counts per expert, summed probabilities per expert, sum of lse^2) on
    the kernel path and ``None`` on the PyTorch path."""
    if _kernel_ok(logits) and logits.shape[1] <= 256 and k <= 16:
        return _RouterFn.apply(logits, k, renorm, want_stats)
    w, idx = router_softmax_topk_reference(logits, k, renorm)
    return w, idx, None


def load_balancing_loss_reference(gate_logits: Sequence[torch.Tensor], num_experts: int, top_k: int):
    """Switch load-balance loss over all layers concatenated
    (optimus/models/olmoe/modeling_olmoe.py:29-85, attention_mask=None)."""
    if gate_logits is None or len(gate_logits) == 0:
        return 0
    cat = torch.cat(list(gate_logits), dim=0)
    rw = F.softmax(cat, dim=-1)
    _, sel = torch.topk(rw, top_k, dim=-1)
    mask = F.one_hot(sel, num_experts)
    tokens_per_expert = torch.mean(mask.float(), dim=0)
    router_prob_per_expert = torch.mean(rw, dim=0)
    return torch.sum(tokens_per_expert * router_prob_per_expert.unsqueeze(0)) * num_experts


def layer_level_load_balancing_loss_reference(gate_logits, num_experts, top_k):
    """Per-layer load-balance loss averaged over layers
    (optimus/models/common/ral_functions.py:6-35)."""
    if gate_logits is None or len(gate_logits) == 0:
        return 0
    st = torch.stack(list(gate_logits), dim=0)  # [L, T, E]
    rw = F.softmax(st, dim=-1)
    _, sel = torch.topk(rw, top_k, dim=-1)
    mask = F.one_hot(sel, num_experts)  # [L, T, k, E]
    tokens_per_expert = torch.mean(mask.float(), dim=1)  # [L, k, E]
    prob = torch.mean(rw, dim=1)  # [L, E]
    per_layer = torch.sum(tokens_per_expert * prob.unsqueeze(1), dim=(1, 2)) * num_experts
    return per_layer.mean()


def z_loss_reference(gate_logits):
    cat = torch.cat(list(gate_logits), dim=0).float()
    return torch.logsumexp(cat, dim=-1).pow(2).mean()


class _AuxLossFn(torch.autograd.Function):
    """Load-balance (+ optional z) loss from the router kernels' statistics.

    forward inputs: ``num_layers`` logits tensors followed by ``num_layers`` index tensors and
    ``num_layers`` stats vectors.  The gradient w.r.t. each layer's logits is
    ``coef*E/N * p o (f - <f,p>)`` (+ z-loss term) computed by the router backward kernel.
    """

    @staticmethod
    def forward(ctx, num_experts, top_k, layer_level, aux_coef, z_coef, n_layers, *tensors):
        logits = tensors[:n_layers]
        idxs = tensors[n_layers:2 * n_layers]
        stats = torch.stack(tensors[2 * n_layers:3 * n_layers], dim=0)  # [L, 2E+1]
        E = num_experts
        T = logits[0].shape[0]
        cnt, prob, lse2 = stats[:, :E], stats[:, E:2 * E], stats[:, 2 * E]
        if layer_level:
            f = cnt / T  # [L, E]
            aux = (E * (f * (prob / T)).sum(dim=1)).mean()
            n_norm = T * n_layers
        else:
            n_norm = T * n_layers
            f = (cnt.sum(0) / n_norm).unsqueeze(0).expand(n_layers, E)
            aux = E * (f[0] * (prob.sum(0) / n_norm)).sum()
        z = lse2.sum() / (T * n_layers)
        ctx.save_for_backward(*logits, *idxs, f.contiguous())
        ctx.cfg = (E, n_layers, aux_coef, z_coef, n_norm, T)
        return aux_coef * aux + z_coef * z

    @staticmethod
    def backward(ctx, g):
        E, L, aux_coef, z_coef, n_norm, T = ctx.cfg
        saved = ctx.saved_tensors
        logits, idxs, f = saved[:L], saved[L:2 * L], saved[2 * L]
        C = extension()
        g = g.to(torch.float32).reshape(1).contiguous()
        grads = []
        for l in range(L):
            d = torch.empty_like(logits[l])
            C.router_bwd(logits[l], idxs[l], None, False, f[l].contiguous(), g, aux_coef * E / n_norm,
                         z_coef / (T * L), d)
            grads.append(d)
        return (None,) * 6 + tuple(grads) + (None,) * (2 * L)


def router_aux_loss(logits_list, idx_list, stats_list, num_experts, top_k, *, layer_level=False, aux_coef=1.0,
                    z_coef=0.0):
    """``aux_coef * load_balance + z_coef * z_loss`` over the given layers' router logits."""
    L = len(logits_list)
    if L == 0:
        return 0
    if stats_list is not None and all(s is not None for s in stats_list) and _kernel_ok(*logits_list):
        return _AuxLossFn.apply(num_experts, top_k, layer_level, aux_coef, z_coef, L, *logits_list, *idx_list,
                                *stats_list)
    fn = layer_level_load_balancing_loss_reference if layer_level else load_balancing_loss_reference
    loss = aux_coef * fn(tuple(logits_list), num_experts, top_k)
    if z_coef:
        loss = loss + z_coef * z_loss_reference(logits_list)
    return loss


# ------------------------------------------------------------------------------------ MoE experts
def moe_experts_reference(x, topk_w, topk_idx, wg, wu, wd, e_start=0):
    """Loop-over-experts oracle (optimus/models/olmoe/modeling_olmoe.py:310-336).

    x [T,H]; topk_w [T,K] (already in x.dtype or fp32); topk_idx [T,K] global expert ids;
    wg/wu [E_loc, I, H]; wd [E_loc, H, I].  Returns [T, H] partial output of the local experts.
    """
    T, H = x.shape
    E_loc = wg.shape[0]
    out = torch.zeros((T, H), dtype=x.dtype, device=x.device)
    tw = topk_w.to(x.dtype)
    for le in range(E_loc):
        tok, kk = torch.where(topk_idx == (e_start + le))
        if tok.numel() == 0:
            continue
        cur = x[tok]
        h = F.silu(F.linear(cur, wg[le])) * F.linear(cur, wu[le])
        y = F.linear(h, wd[le]) * tw[tok, kk, None]
        out.index_add_(0, tok, y)
    return out


ROW_PAD = 256   # every expert's rows start at a multiple of this: a pair of CTAs shares one 256-row GEMM tile


def moe_capacity_rows(T: int, K: int, E_loc: int, ep: int = 1, capacity_factor: float = 0.0) -> int:
    """Row capacity of the expert-grouped buffers: every routed pair plus ``ROW_PAD - 1`` padding rows per
    local expert, rounded to ``ROW_PAD``.  With ``capacity_factor > 0`` (expert parallel receive
    side) the pair count is ``capacity_factor`` x the balanced share instead of the worst case."""
    pairs = T * K
    if capacity_factor and ep > 1:
        pairs = min(pairs, int(math.ceil(capacity_factor * T * K / ep)))
    rows = pairs + E_loc * (ROW_PAD - 1)
    return ((rows + ROW_PAD - 1) // ROW_PAD) * ROW_PAD


_PART_CUTS = {}
_FLAG_SCRATCH = {}
ROW_GRANULE = 2048    # exact-sized expert buffers are rounded up to this many rows (fewer distinct allocation sizes)


def stage_flags(device, rows: int) -> torch.Tensor:
    """Per-device int32 scratch with one counter per 128-row block, for the GEMM variants whose extra warps move rows
    (the bindings zero it before the launch).  Launches on one stream follow each other, so one buffer serves all."""
    need = rows // 128 + 2
    t = _FLAG_SCRATCH.get(device)
    if t is None or t.numel() < need:
        t = _FLAG_SCRATCH[device] = torch.empty(max(need, 1024), dtype=torch.int32, device=device)
    return t


class MoEIndex:
    """Device-resident permutation of routed (token, k) pairs into expert-grouped rows.

    ``cap`` bounds the index arrays.  ``rows`` is what the activation buffers of this layer hold: ``cap`` itself, or,
    with ``exact``, the number of 128-row blocks the routing actually produced (one 4-byte read of the device-side
    count, rounded up to ``ROW_GRANULE``).  With expert parallelism the worst case is every token of every rank
    choosing this rank's experts; sizing the saved activations for that would not fit, sizing them for a fixed
    multiple of the balanced share can overflow, so the count is read instead and no routed pair is ever dropped."""

    __slots__ = ("row_of", "src_of", "k_of", "meta", "offsets", "counts", "cap", "rows", "E_loc", "K", "pair")

    def __init__(self, topk_idx: torch.Tensor, e_start: int, E_loc: int, cap: int, exact: bool = False):
        C = extension()
        T, K = topk_idx.shape
        dev = topk_idx.device
        ws = torch.empty(C.moe_ws_ints(T, E_loc), dtype=torch.int32, device=dev)
        self.row_of = torch.empty((T, K), dtype=torch.int32, device=dev)
        self.src_of = torch.empty(cap, dtype=torch.int32, device=dev)
        self.k_of = torch.empty(cap, dtype=torch.int32, device=dev)
        self.meta = torch.empty(1 + cap // 128, dtype=torch.int32, device=dev)
        self.offsets = torch.empty(E_loc + 1, dtype=torch.int32, device=dev)
        self.counts = torch.empty(E_loc, dtype=torch.int32, device=dev)
        self.cap, self.E_loc, self.K = cap, E_loc, K
        self.pair = cap % ROW_PAD == 0      # expert groups padded to 256 rows: the CTA-pair kernels may take them
        C.moe_build_index(topk_idx.contiguous(), e_start, E_loc, cap, ws, self.row_of, self.src_of, self.k_of,
                          self.meta, self.offsets, self.counts, status_word(dev), ROW_PAD if self.pair else 128)
        self.rows = cap
        if exact:
            used = int(self.meta[0].item()) * 128
            self.rows = min(cap, max(ROW_GRANULE, -(-used // ROW_GRANULE) * ROW_GRANULE))

    def part_ranges(self, parts: int) -> torch.Tensor:
        """``[parts, 2]`` int32 (device): first and one-past-last 128-row block of each group of consecutive local
        experts.  Lets a consumer start on the first experts' rows while the rest is still in flight."""
        parts = max(1, min(parts, self.E_loc))
        key = (self.E_loc, parts, self.offsets.device)
        cuts = _PART_CUTS.get(key)
        if cuts is None:  # built once: a host-to-device copy here would stall the launch queue every layer
            cuts = _PART_CUTS[key] = torch.tensor([(p * self.E_loc) // parts for p in range(parts + 1)],
                                                  device=self.offsets.device)
        b = torch.div(self.offsets[cuts], 128, rounding_mode="floor").to(torch.int32)
        return torch.stack([b[:-1], b[1:]], dim=1).contiguous()


def grouped_linear_fwd(xp, w, index: MoEIndex, out=None, blk_range=None):
    """``y[rows of e] = xp[rows of e] @ w[e].T`` for merged weights ``w [E, N, K]``."""
    E, N, K = w.shape
    return gemm(xp, w.view(E * N, K), index.rows, N, K, mode=GEMM_RAGGED_M, meta=index.meta, b_expert_rows=N, out=out,
                blk_range=blk_range, pair_rows=index.pair)


def grouped_linear_dgrad(dy, w, index: MoEIndex, out=None, accumulate=False, blk_range=None):
    """``dx[rows of e] (+)= dy[rows of e] @ w[e]``."""
    E, N, K = w.shape
    return gemm(dy, w.view(E * N, K), index.rows, K, N, b_mn_major=True, mode=GEMM_RAGGED_M, meta=index.meta,
                b_expert_rows=N, out=out, accumulate=accumulate, blk_range=blk_range, pair_rows=index.pair)


def grouped_linear_dgrad_pair(dh, w1, w2, index: MoEIndex, out=None):
    """``dx[rows of e] = dh[rows of e, :I] @ w1[e] + dh[rows of e, I:] @ w2[e]`` in one launch (the input
    gradient of the gate and up projections, whose output gradients sit side by side in ``dh``)."""
    E, N, K = w1.shape
    assert w2.shape == w1.shape and dh.shape[1] == 2 * N
    return gemm(dh, w1.view(E * N, K), index.rows, K, 2 * N, b_mn_major=True, mode=GEMM_RAGGED_M, meta=index.meta,
                b_expert_rows=N, out=out, b2=w2.view(E * N, K), k_split=N, pair_rows=index.pair)


def grouped_linear_wgrad(dy, xp, index: MoEIndex, N: int, K: int, holder: Optional["DirectGrad"] = None):
    """``dw[e] = dy[rows of e].T @ xp[rows of e]`` -> [E, N, K].  With a ``DirectGrad`` holder the result goes
    (or is added) into the holder's buffer and ``None`` is returned."""
    if holder is not None:
        gemm(dy, xp, N, K, index.rows, a_mn_major=True, b_mn_major=True, mode=GEMM_RAGGED_K, meta=index.offsets,
             num_experts=index.E_loc, c_expert_stride=N * K, out=holder.buf, accumulate=holder.ready)
        holder.ready = True
        return None
    return gemm(dy, xp, N, K, index.rows, a_mn_major=True, b_mn_major=True, mode=GEMM_RAGGED_K, meta=index.offsets,
                num_experts=index.E_loc, c_expert_stride=N * K)


def grouped_gateup_swiglu(x_ptrs, x_ld: int, tokens: int, weights, wg, wu, index: MoEIndex):
    """Gate and up projections of the local experts with the dispatch in front and the activation behind, one launch:
    extra warps of the GEMM fetch token ``src_of[u]`` from ``x_ptrs[src_of[u] // tokens]`` into row ``u`` of the
    expert-grouped operand (over NVLink when the token lives on another GPU), the tensor-core warps start on the first
    row blocks while later ones are still arriving, and the epilogue writes ``gate | up`` and
    ``weights[src, k] * silu(gate) * up``.  Returns ``(xp, h, act)``."""
    C = extension()
    E, I, H = wg.shape
    dev = wg.device
    rows = index.rows
    xp = torch.empty((rows, H), dtype=wg.dtype, device=dev)
    h = torch.empty((rows, 2 * I), dtype=wg.dtype, device=dev)
    act = torch.empty((rows, I), dtype=wg.dtype, device=dev)
    if I % 128:
        # widths the paired gate|up tile does not cover: separate launches (gather, two projections, activation)
        C.ep_gather_rows(list(x_ptrs), tokens, index.src_of, index.meta, xp, None)
        grouped_linear_fwd(xp, wg, index, out=h[:, :I])
        grouped_linear_fwd(xp, wu, index, out=h[:, I:])
        C.swiglu_rowscale_fwd(h[:, :I], h[:, I:], index.src_of, index.k_of, weights, index.meta, act)
        return xp, h, act
    if len(x_ptrs) == 1 and not _GATHER_IN_KERNEL_LOCAL:
        # every token is in this GPU's memory: nothing crosses NVLink that the GEMM could hide, and the gather's traffic
        # through the L2 slows the tiles down by as much as it takes on its own (measured: 1.14 ms fused against
        # 0.15 + 0.88 ms); the permutation runs as its own kernel and the GEMM reads the operand in place
        C.ep_gather_rows(list(x_ptrs), tokens, index.src_of, index.meta, xp, None)
        C.gemm_gateup_swiglu(xp, wg.view(E * I, H), wu.view(E * I, H), h, act, rows, I, H, index.meta, index.src_of,
                             index.k_of, weights, E, [], 0, 0, None, status_word(dev), index.pair)
        return xp, h, act
    C.gemm_gateup_swiglu(xp, wg.view(E * I, H), wu.view(E * I, H), h, act, rows, I, H, index.meta, index.src_of,
                         index.k_of, weights, E, list(x_ptrs), x_ld, tokens, stage_flags(dev, rows), status_word(dev),
                         index.pair)
    return xp, h, act


_GATHER_IN_KERNEL_LOCAL = os.environ.get("OLB_GATHER_IN_KERNEL", "0") == "1"   # also gather local rows inside the GEMM
_FUSE_SWIGLU_BWD = os.environ.get("OLB_FUSE_SWIGLU_BWD", "0") == "1"            # SwiGLU backward in the dgrad epilogue


def grouped_gather_dgrad(y_ptrs, y_ld: int, tokens: int, w, index: MoEIndex):
    """``dyp[u] = dout[src_of[u]]`` gathered inside the launch that computes ``dact = dyp @ w[e]`` (input gradient of
    the down projection, ``w [E, H, I]``).  Returns ``(dyp, dact)``."""
    C = extension()
    E, H, I = w.shape
    dev = w.device
    rows = index.rows
    dyp = torch.empty((rows, H), dtype=w.dtype, device=dev)
    dact = torch.empty((rows, I), dtype=w.dtype, device=dev)
    if len(y_ptrs) == 1 and not _GATHER_IN_KERNEL_LOCAL:
        C.ep_gather_rows(list(y_ptrs), tokens, index.src_of, index.meta, dyp, None)
        grouped_linear_dgrad(dyp, w, index, out=dact)
        return dyp, dact
    C.gemm_ep_gather(dyp, w.view(E * H, I), dact, rows, I, H, True, index.meta, index.src_of, H, E, list(y_ptrs), y_ld,
                     tokens, stage_flags(dev, rows), status_word(dev), index.pair)
    return dyp, dact


def grouped_down_dgrad_swiglu_bwd(y_ptrs, y_ld: int, tokens: int, w, h, weights, index: MoEIndex, dweights_out):
    """Backward of ``act -> y`` and of the routing-weighted SwiGLU in one launch: the output gradients are gathered
    (``dyp[u] = dout[src_of[u]]``) by extra warps, ``d(act) = dyp @ w[e]`` stays in the accumulator, and the epilogue
    turns it into ``d(gate) | d(up)`` with the saved ``h = gate | up`` and the routing weights.  The routing-weight
    gradients ``<d(act), silu(gate) * up>`` are written to ``dweights_out [tokens_total, K]`` (rows of pairs that are
    not local stay untouched).  Returns ``(dyp, dh)``."""
    C = extension()
    E, H, I = w.shape
    dev = w.device
    rows = index.rows
    dh = torch.empty_like(h)
    if not (_FUSE_SWIGLU_BWD and index.pair and I % 256 == 0 and rows % 256 == 0
            and os.environ.get("OLB_GEMM_PAIR", "1") != "0"):
        # default: the product is stored and a separate kernel does the activation's backward.  The fused epilogue
        # (OLB_FUSE_SWIGLU_BWD=1) reads the saved gate | up with one row per lane, which thrashes the small L1 that is
        # left beside 224 KB of shared memory: 1.07 ms against 0.55 + 0.28 ms for the two kernels.
        dyp, dact = grouped_gather_dgrad(y_ptrs, y_ld, tokens, w, index)
        C.swiglu_rowscale_bwd(dact, h[:, :I], h[:, I:], index.src_of, index.k_of, weights, index.meta, dh[:, :I],
                              dh[:, I:], dweights_out)
        return dyp, dh
    dyp = torch.empty((rows, H), dtype=w.dtype, device=dev)
    partial = torch.empty((rows, I // 256), dtype=torch.float32, device=dev)
    C.gemm_ep_gather(dyp, w.view(E * H, I), dh, rows, I, H, True, index.meta, index.src_of, H, E, list(y_ptrs), y_ld,
                     tokens, stage_flags(dev, rows), status_word(dev), index.pair, h, index.k_of, weights, partial)
    C.moe_scatter_dweights(partial, index.src_of, index.k_of, index.meta, dweights_out)
    return dyp, dh


class _MoEExpertsFn(torch.autograd.Function):
    """Local expert computation on expert-grouped rows:
    index build -> [gather + grouped gate|up GEMM + weighted SwiGLU] (one launch) -> grouped down GEMM ->
    unweighted combine.  The routing weight is folded into the activation, so the backward
    needs neither the expert outputs nor a weighted scatter."""

    @staticmethod
    def forward(ctx, x, topk_w, topk_idx, wg, wu, wd, e_start, cap, holders=(None, None, None), exact=False):
        C = extension()
        T, H = x.shape
        E_loc, I, _ = wg.shape
        ctx.holders = holders
        x = x.contiguous()
        topk_w = topk_w.contiguous().float()
        index = MoEIndex(topk_idx, e_start, E_loc, cap, exact)
        xp, h, act = grouped_gateup_swiglu([x.data_ptr()], H, T, topk_w, wg, wu, index)
        y = grouped_linear_fwd(act, wd, index)
        out = torch.empty((T, H), dtype=x.dtype, device=x.device)
        C.moe_combine(y, index.row_of, None, out)
        ctx.save_for_backward(xp, h, act, topk_w, wg, wu, wd)
        ctx.index = index
        ctx.dims = (T, H, I, E_loc)
        return out

    @staticmethod
    def backward(ctx, dout):
        C = extension()
        xp, h, act, topk_w, wg, wu, wd = ctx.saved_tensors
        index = ctx.index
        T, H, I, E_loc = ctx.dims
        dout = dout.contiguous()
        # d(y) = gather of dout (the combine was an unweighted sum), d(act) = d(y) wd and the activation's backward:
        # one launch
        dtopk = torch.zeros_like(topk_w)
        dyp, dh = grouped_down_dgrad_swiglu_bwd([dout.data_ptr()], H, T, wd, h, topk_w, index, dtopk)
        hg, hu, hd = ctx.holders
        dwd = grouped_linear_wgrad(dyp, act, index, H, I, hd) if ctx.needs_input_grad[5] else None
        del dyp
        dwg = grouped_linear_wgrad(dh[:, :I], xp, index, I, H, hg) if ctx.needs_input_grad[3] else None
        dwu = grouped_linear_wgrad(dh[:, I:], xp, index, I, H, hu) if ctx.needs_input_grad[4] else None
        dxp = grouped_linear_dgrad_pair(dh, wg, wu, index)
        dx = torch.empty((T, H), dtype=dout.dtype, device=dout.device)
        C.moe_combine(dxp, index.row_of, None, dx)
        return dx, dtopk, None, dwg, dwu, dwd, None, None, None, None


def moe_experts(x, topk_w, topk_idx, wg, wu, wd, e_start=0, cap: Optional[int] = None, exact: bool = False):
    """Partial MoE output of the local experts for tokens ``x [T,H]``.

    ``topk_idx`` holds global expert ids; pairs routed to other ranks' experts are skipped.
    ``wg/wu [E_loc, I, H]``, ``wd [E_loc, H, I]`` (the merged-MLP layout of the reference,
    optimus/models/common/moe.py:379-405).  ``exact``: ``cap`` is a worst case that is rarely reached (tokens of a
    whole expert-parallel group); size the activation buffers from the routed count instead (see ``MoEIndex``)."""
    E_loc, I, H = wg.shape
    if _kernel_ok(x, wg, wu, wd) and topk_idx.dtype == torch.int32 and H % 64 == 0 and I % 64 == 0 and E_loc <= 256:
        if cap is None:
            cap = moe_capacity_rows(x.shape[0], topk_idx.shape[1], E_loc)
        return _MoEExpertsFn.apply(x, topk_w, topk_idx, wg, wu, wd, e_start, cap,
                                   (_holder(wg), _holder(wu), _holder(wd)), exact)
    return moe_experts_reference(x, topk_w, topk_idx.long(), wg, wu, wd, e_start)


# ------------------------------------------------------------------------------------ cross entropy
class _ShiftedCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits2d, labels1d, inplace_backward):
        C = extension()
        rows = logits2d.shape[0]
        loss_row = torch.empty(rows, dtype=torch.float32, device=logits2d.device)
        lse = torch.empty_like(loss_row)
        C.ce_fwd(logits2d, labels1d, loss_row, lse)
        n_valid = (labels1d >= 0).sum().to(torch.float32)
        ctx.save_for_backward(logits2d, labels1d, lse, n_valid)
        ctx.inplace = inplace_backward
        return loss_row.sum() / n_valid

    @staticmethod
    def backward(ctx, g):
        logits2d, labels1d, lse, n_valid = ctx.saved_tensors
        scale = (g.to(torch.float32) / n_valid).reshape(1).contiguous()
        d = logits2d if ctx.inplace else torch.empty_like(logits2d)
        extension().ce_bwd(logits2d, labels1d, lse, scale, d)
        return d, None, None


def shifted_cross_entropy_reference(logits, labels):
    """Reference loss (optimus/models/olmoe/modeling_olmoe.py:515-524)."""
    V = logits.shape[-1]
    sl = logits[..., :-1, :].contiguous().view(-1, V)
    tl = labels[..., 1:].contiguous().view(-1)
    return F.cross_entropy(sl, tl)


def shifted_cross_entropy(logits, labels, inplace_backward=False):
    """Mean CE of ``logits[:, :-1]`` against ``labels[:, 1:]``.  On the kernel path the full
    ``[B*S, V]`` logits are used with the last position of every sequence ignored, so no
    shifted copy of the logits is made; with ``inplace_backward`` the gradient overwrites the
    logits buffer."""
    if _kernel_ok(logits) and logits.is_contiguous() and logits.shape[-1] % 8 == 0:
        B, S, V = logits.shape
        tgt = torch.full((B, S), -100, dtype=torch.long, device=logits.device)
        tgt[:, :-1] = labels[:, 1:]
        return _ShiftedCEFn.apply(logits.view(B * S, V), tgt.view(-1), inplace_backward)
    return shifted_cross_entropy_reference(logits, labels)


# ------------------------------------------------------------------------------------ vocabulary-parallel CE
def _merge_ce_stats(part_max, part_sum, part_tgt, group):
    """Merge per-slice softmax statistics over ``group``: returns the global log-sum-exp and target logit per row."""
    import torch.distributed as dist
    gmax = part_max.clone()
    multi = group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
    if multi:
        dist.all_reduce(gmax, op=dist.ReduceOp.MAX, group=group)
    both = torch.stack((part_sum * torch.exp(part_max - gmax), part_tgt))
    if multi:
        dist.all_reduce(both, group=group)
    return gmax + torch.log(both[0]), both[1]


class _VocabParallelCEFn(torch.autograd.Function):
    """Mean cross entropy of rows whose logits are split over the ranks of ``group`` along the vocabulary."""

    @staticmethod
    def forward(ctx, logits2d, labels1d, v_start, v_total, group, inplace_backward):
        rows, V = logits2d.shape
        valid = (labels1d >= 0) & (labels1d < v_total)
        if _kernel_ok(logits2d) and logits2d.stride(1) == 1 and logits2d.stride(0) % 8 == 0:
            C = extension()
            pm, ps, pt = (torch.empty(rows, dtype=torch.float32, device=logits2d.device) for _ in range(3))
            C.ce_partial_fwd(logits2d, labels1d, v_start, pm, ps, pt)
            ctx.kernel = True
        else:
            lf = logits2d.float()
            pm = lf.max(dim=1).values
            ps = torch.exp(lf - pm[:, None]).sum(dim=1)
            loc = labels1d - v_start
            mine = valid & (loc >= 0) & (loc < V)
            pt = torch.where(mine, lf.gather(1, loc.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(pm))
            ctx.kernel = False
        lse, tgt = _merge_ce_stats(pm, ps, pt, group)
        n_valid = valid.sum().to(torch.float32)
        ctx.save_for_backward(logits2d, labels1d, lse, n_valid)
        ctx.misc = (v_start, v_total, inplace_backward)
        return torch.where(valid, lse - tgt, torch.zeros_like(lse)).sum() / n_valid

    @staticmethod
    def backward(ctx, g):
        logits2d, labels1d, lse, n_valid = ctx.saved_tensors
        v_start, v_total, inplace = ctx.misc
        scale = (g.to(torch.float32) / n_valid).reshape(1).contiguous()
        if ctx.kernel:
            d = logits2d if inplace else torch.empty_like(logits2d)
            extension().ce_partial_bwd(logits2d, labels1d, v_start, v_total, lse, scale, d)
            return d, None, None, None, None, None
        V = logits2d.shape[1]
        valid = (labels1d >= 0) & (labels1d < v_total)
        p = torch.exp(logits2d.float() - lse[:, None])
        loc = labels1d - v_start
        mine = valid & (loc >= 0) & (loc < V)
        p[mine.nonzero()[:, 0], loc[mine]] -= 1.0
        p = p * (valid[:, None].float() * scale)
        return p.to(logits2d.dtype), None, None, None, None, None


def vocab_parallel_cross_entropy(logits, labels, v_start: int, v_total: int, group=None, inplace_backward=False,
                                 shifted=True):
    """Mean cross entropy for logits ``[B, S, V_local]`` that cover the vocabulary slice ``[v_start, v_start +
    V_local)`` of ``v_total`` entries on this rank of ``group``; ``labels [B, S]`` hold global ids.  With ``shifted``
    position ``s`` is scored against ``labels[:, s + 1]`` (the loss of
    optimus/models/olmoe/modeling_olmoe.py:515-524).  Only ``[rows]``-sized statistics are all-reduced."""
    B, S, V = logits.shape
    if shifted:
        tgt = torch.full((B, S), -100, dtype=torch.long, device=logits.device)
        tgt[:, :-1] = labels[:, 1:]
    else:
        tgt = labels.long()
    return _VocabParallelCEFn.apply(logits.reshape(B * S, V), tgt.reshape(-1), int(v_start), int(v_total), group,
                                    inplace_backward)


# ------------------------------------------------------------------------------------ optimizer kernels
def adamw_step_reference(grad, master, m, v, param, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
                         clip_coef=None, skip_weight_update=False, norm_out=None):
    """The reference update (optimus/optimizers.py:193-205) in plain torch, in place."""
    g = grad.to(torch.float32) * grad_scale
    if norm_out is not None:
        norm_out.add_(g.pow(2).sum())
    if clip_coef is not None:
        g = g * clip_coef
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    if not skip_weight_update:
        mhat = m / (1 - beta1 ** step)
        vhat = v / (1 - beta2 ** step)
        master.sub_(lr * mhat / (vhat.sqrt() + eps))
        master.add_(master, alpha=-lr * weight_decay)
    if param.data_ptr() != master.data_ptr():
        param.copy_(master)


def adamw_step(grad, master, m, v, param, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0,
               clip_coef=None, skip_weight_update=False, norm_out=None):
    """In-place AdamW on one flat range.  ``norm_out`` (1 fp32 element): ``+= sum((grad * grad_scale)^2)``, taken from
    the update's own read of the gradients instead of a separate pass."""
    if master.is_cuda and use_kernels(master) and master.numel() % 4 == 0:
        extension().adamw_step(grad, master, m, v, param, lr, beta1, beta2, eps, weight_decay, step, grad_scale,
                               clip_coef, skip_weight_update, norm_out)
    else:
        adamw_step_reference(grad, master, m, v, param, lr, beta1, beta2, eps, weight_decay, step, grad_scale,
                             clip_coef, skip_weight_update, norm_out)


def sum_of_squares(t: torch.Tensor, scale: float = 1.0, out: Optional[torch.Tensor] = None, accumulate=False):
    """``sum((t*scale)^2)`` as a 1-element fp32 tensor (deterministic reduction on GPU)."""
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=t.device)
        accumulate = False
    if t.is_cuda and use_kernels(t) and t.dtype in (torch.bfloat16, torch.float32) and t.is_contiguous():
        C = extension()
        partial = torch.empty(max(1, C.sumsq_blocks(t.numel())), dtype=torch.float32, device=t.device)
        C.sumsq(t, scale, partial, out, accumulate)
    else:
        s = (t.to(torch.float32) * scale).pow(2).sum().reshape(1)
        if accumulate:
            out.add_(s)
        else:
            out.copy_(s)
    return out
