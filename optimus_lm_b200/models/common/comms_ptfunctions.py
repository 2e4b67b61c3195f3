"""Differentiable collectives used inside the models.

Same names, argument orders and math as the reference's thirteen autograd functions
(optimus/models/common/comms_ptfunctions.py:26-436), so model code written against the
reference runs unchanged.  Differences by design:

* no device synchronise + barrier in front of the collectives (the reference inserts them
  as "jitter" timers, :41-43, :68-70, :124-126); collectives are enqueued on the current
  stream and overlap with whatever the caller schedules around them;
* one ``_Collective`` base supplies the boilerplate, every function states only its forward
  and backward transfer;
* gloo (CPU ranks) lacks reduce-scatter, so ``_reduce_scatter`` falls back to all-reduce +
  slice there - the same substitute the reference offers behind
  ``use_allreduce_for_reducescatter``.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from ...profilers import record_pcl_function


def _shape_tag(t):
    return "x".join(str(d) for d in t.shape)


def _backend_has_reduce_scatter(group) -> bool:
    try:
        return dist.get_backend(group) != "gloo"
    except Exception:
        return True


def _all_gather_dim0(x, n, group):
    x = x.contiguous()
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    with record_pcl_function(f"2su-comms--allgather({_shape_tag(out)})"):
        dist.all_gather_into_tensor(out, x, group=group)
    return out


def _reduce_scatter_dim0(x, pid, n, group, use_allreduce=False):
    x = x.contiguous()
    part = x.shape[0] // n
    if use_allreduce or not _backend_has_reduce_scatter(group):
        with record_pcl_function(f"2su-comms--allreduce({_shape_tag(x)})"):
            dist.all_reduce(x, group=group)
        return x[pid * part:(pid + 1) * part].clone()
    out = torch.empty((part,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    with record_pcl_function(f"2su-comms--reducescatter({_shape_tag(x)})"):
        dist.reduce_scatter_tensor(out, x, group=group)
    return out


def _all_gather_via_allreduce(x, pid, n, group):
    out = torch.zeros((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    out[pid * x.shape[0]:(pid + 1) * x.shape[0]].copy_(x)
    dist.all_reduce(out, group=group)
    return out


# ----------------------------------------------------------------------------- tensor parallel
class forward_identity_backward_allreduce(torch.autograd.Function):
    """Block input of a tensor-parallel region."""

    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        with record_pcl_function(f"2su-comms--2bwd--2allreduce({_shape_tag(grad)})"):
            dist.all_reduce(grad, group=ctx.group)
        return grad, None


class forward_allreduce_backward_identity(torch.autograd.Function):
    """Block output of a tensor-parallel region (row-parallel partial sums)."""

    @staticmethod
    def forward(ctx, x, group=None):
        x = x.contiguous()
        with record_pcl_function(f"2su-comms--1fwd--2allreduce({_shape_tag(x)})"):
            dist.all_reduce(x, group=group)
        ctx.mark_dirty(x)
        return x

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class forward_inner_split_backward_allgather(torch.autograd.Function):
    """Slice the last dim for this rank; backward rebuilds the full last dim."""

    @staticmethod
    def forward(ctx, x, pid=0, num_processes=1, group=None):
        size_p = x.shape[-1] // num_processes
        ctx.args = (pid, num_processes, group, size_p)
        return x[..., pid * size_p:(pid + 1) * size_p].contiguous()

    @staticmethod
    def backward(ctx, grad):
        pid, n, group, size_p = ctx.args
        full = torch.zeros(tuple(grad.shape[:-1]) + (size_p * n,), dtype=grad.dtype, device=grad.device)
        full[..., pid * size_p:(pid + 1) * size_p].copy_(grad)
        dist.all_reduce(full, group=group)
        return full, None, None, None


# ----------------------------------------------------------------------------- expert parallel
class forward_allgather_backward_reducescatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pid=0, num_processes=1, group=None, use_allreduce_for_reducescatter=False):
        ctx.args = (pid, num_processes, group, use_allreduce_for_reducescatter)
        return _all_gather_dim0(x, num_processes, group)

    @staticmethod
    def backward(ctx, grad):
        pid, n, group, use_ar = ctx.args
        return _reduce_scatter_dim0(grad, pid, n, group, use_ar), None, None, None, None


class forward_allgather_backward_split(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pid=0, num_processes=1, group=None):
        ctx.args = (pid, num_processes, x.shape[0])
        return _all_gather_dim0(x, num_processes, group)

    @staticmethod
    def backward(ctx, grad):
        pid, n, part = ctx.args
        return grad[pid * part:(pid + 1) * part], None, None, None


class forward_reducescatter_backward_allgather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pid=0, num_processes=1, group=None, use_allreduce_for_reducescatter=False,
                use_allreduce_for_allgather=False):
        ctx.args = (pid, num_processes, group, use_allreduce_for_allgather)
        return _reduce_scatter_dim0(x, pid, num_processes, group, use_allreduce_for_reducescatter)

    @staticmethod
    def backward(ctx, grad):
        pid, n, group, use_ar = ctx.args
        if use_ar:
            out = _all_gather_via_allreduce(grad.contiguous(), pid, n, group)
        else:
            out = _all_gather_dim0(grad, n, group)
        return out, None, None, None, None, None


class forward_identity_backward_synchronize(torch.autograd.Function):
    """The reference uses this pair as barrier-only "MoE imbalance" timers (:276-299).  Here
    they record a profiler region and otherwise do nothing, unless OLB_MOE_IMBALANCE_BARRIER=1."""

    @staticmethod
    def forward(ctx, x, group=None):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, grad):
        if os.environ.get("OLB_MOE_IMBALANCE_BARRIER", "0") == "1":
            with record_pcl_function("2su-comms--2bwd--moe-imbalance"):
                dist.barrier(group=ctx.group)
        return grad, None


class forward_synchronize_backward_identity(torch.autograd.Function):
    @staticmethod
    def forward(ctx, group=None):
        if os.environ.get("OLB_MOE_IMBALANCE_BARRIER", "0") == "1":
            with record_pcl_function("2su-comms--1fwd--moe-imbalance"):
                dist.barrier(group=group)
        return torch.zeros(())

    @staticmethod
    def backward(ctx, grad):
        return None


class forward_identity_backward_identity(torch.autograd.Function):
    """Debug tap: with ``OLB_DUMP_TENSORS=<dir>`` saves the forward tensor and its gradient as
    ``<dir>/rank{r}_{tag}_{fwd|bwd}.pt`` (reference :303-315 writes to ``tensors/``)."""

    @staticmethod
    def forward(ctx, x, tag=""):
        ctx.tag = tag
        _dump(x, tag, "fwd")
        return x

    @staticmethod
    def backward(ctx, grad):
        _dump(grad, ctx.tag, "bwd")
        return grad, None


def _dump(t, tag, phase):
    d = os.environ.get("OLB_DUMP_TENSORS")
    if not d:
        return
    os.makedirs(d, exist_ok=True)
    r = dist.get_rank() if dist.is_initialized() else 0
    torch.save(t.detach().cpu(), os.path.join(d, f"rank{r}_{tag}_{phase}.pt"))


# ----------------------------------------------------------------------------- split / gather helpers
class forward_split_backward_allgather_pad(torch.autograd.Function):
    """Ceil-divide dim 0 over the ranks (last part may be short); backward gathers with padding."""

    @staticmethod
    def forward(ctx, x, pid=0, num_processes=1, group=None):
        size = x.shape[0]
        size_p = math.ceil(size / num_processes)
        lo, hi = pid * size_p, min((pid + 1) * size_p, size)
        ctx.args = (num_processes, group, size, size_p)
        return x[lo:hi]

    @staticmethod
    def backward(ctx, grad):
        n, group, size, size_p = ctx.args
        if grad.shape[0] != size_p:
            padded = torch.zeros((size_p,) + tuple(grad.shape[1:]), dtype=grad.dtype, device=grad.device)
            padded[:grad.shape[0]].copy_(grad)
            grad = padded
        return _all_gather_dim0(grad, n, group)[:size], None, None, None


class forward_allgather_backward_split_pad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, xp, size, pid=0, num_processes=1, group=None):
        size_p = math.ceil(size / num_processes)
        if xp.shape[0] != size_p:
            padded = torch.zeros((size_p,) + tuple(xp.shape[1:]), dtype=xp.dtype, device=xp.device)
            padded[:xp.shape[0]].copy_(xp)
            xp = padded
        ctx.args = (pid, size, size_p)
        return _all_gather_dim0(xp, num_processes, group)[:size]

    @staticmethod
    def backward(ctx, grad):
        pid, size, size_p = ctx.args
        return grad[pid * size_p:min((pid + 1) * size_p, size)], None, None, None, None


class forward_split_backward_allgather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pid=0, num_processes=1, group=None):
        size_p = x.shape[0] // num_processes
        ctx.args = (num_processes, group)
        return x[pid * size_p:(pid + 1) * size_p]

    @staticmethod
    def backward(ctx, grad):
        n, group = ctx.args
        return _all_gather_dim0(grad, n, group), None, None, None


class forward_allgather_backward_pick(torch.autograd.Function):
    """Gather along the last dim; backward picks this rank's slice."""

    @staticmethod
    def forward(ctx, x, rank=0, world_size=1, group=None):
        parts = [torch.empty_like(x) for _ in range(world_size)]
        dist.all_gather(parts, x.contiguous(), group=group)
        ctx.args = (rank, x.shape[-1])
        return torch.cat(parts, -1)

    @staticmethod
    def backward(ctx, grad):
        rank, width = ctx.args
        return grad[..., rank * width:(rank + 1) * width].contiguous(), None, None, None
