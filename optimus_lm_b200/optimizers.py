"""Flat-buffer mixed-precision AdamW optimizers.

The five optimizer classes of the reference (optimus/optimizers.py:19-1742) with the same
constructor signatures, ``step() -> grad_norm``, ``zero_grad()``, ``state_dict()`` keys and
flat-buffer layouts (so optimizer checkpoints are interchangeable):

=========================================  ==========================================================
``MixedPrecisionAdamW``                    unsharded flat buffers, DP all-reduce of the flat gradient
``ShardedMixedPrecisionAdamW``             ZeRO-1 over DP, shard size rounded up to 512 elements
``ParamGroupShardedMixedPrecisionAdamW``   two families: EP-replicated parameters sharded over the
                                           DP x EP group, expert parameters sharded over DP
``SubShardedMixedPrecisionAdamW``          like "shard" but the flat buffer is cut into chunks of
                                           <= 128Mi elements that are sharded one by one
``ParamGroupSubShardedMixedPrecisionAdamW``  both of the above
=========================================  ==========================================================

They are thin layouts over one engine.  A *family* is a flat parameter buffer + flat
gradient buffer (model dtype) whose elements are owned, slice by slice, by the ranks of one
process group; the owner keeps fp32 master / exp_avg / exp_avg_sq for its slices.  One step:

1. gradient reduction per family slice: reduce-scatter (or all-reduce) over the family's
   group - on GPUs with peer access the reduction, the 1/N scaling, the bf16->fp32 cast, the
   norm partial and the AdamW update run as one kernel pass over peer memory
   (``optimus_lm_b200.parallel.fused_optimizer``);
2. global gradient norm: deterministic sum of squares of the owned slices, all-reduced over
   all ranks; the reference's per-class scaling quirks are kept (see ``_FamilySpec.grad_divisor``
   and the 1/sqrt(EP) weighting of replicated gradients in the "shard" class);
3. clipping to max-norm 1.0, active from optimizer step ``warmup_steps`` on ("delayed
   clipping") - the coefficient stays on the device, there is no host sync;
4. fused AdamW kernel on the owned slices (reference update rule, decay after the Adam step);
5. parameter all-gather per family slice.

``p.data`` and ``p.grad`` of every parameter are views into the flat buffers.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch.optim import Optimizer

from .ops import functional as OF
from .profilers import record_pcl_function

# chunk size of the sub-sharded classes and of the chunked all-reduce (reference: 128Mi elements);
# OLB_OPT_CHUNK_ELEMS overrides it, e.g. to exercise several chunks on a small model
CHUNK_ELEMS = int(os.environ.get("OLB_OPT_CHUNK_ELEMS", str(128 * 1024 * 1024)))


def chunked_allreduce_wrapper(tensor, group=None, barrier=False, chunk=CHUNK_ELEMS):
    """All-reduce ``tensor`` in pieces of at most ``chunk`` elements (reference :11-17)."""
    for part in tensor.view(-1).split(chunk):
        dist.all_reduce(part, group=group)
        if barrier:
            dist.barrier(group=group)


def _group_ok(group) -> bool:
    return dist.is_available() and dist.is_initialized() and group is not None and group != -1


def _has_reduce_scatter(group) -> bool:
    try:
        return dist.get_backend(group if group != -1 else None) != "gloo"
    except Exception:
        return True


@dataclass
class _Slice:
    """One contiguous region of a family's flat buffer that is sharded over the group."""
    flat_start: int      # start of the region in the flat buffer
    length: int          # region length = num_shards * part
    part: int            # elements owned by each rank
    state_start: int     # offset of this rank's part inside its fp32 state tensors


@dataclass
class _FamilySpec:
    name: str                     # "" | "replicated" | "divided"
    params: List[torch.nn.Parameter]
    group: object                 # process group (or None / -1)
    num_shards: int
    shard_id: int
    grad_divisor: float           # gradients are divided by this after the reduction
    chunk_limit: Optional[int] = None   # sub-sharding: max elements per chunk
    chunk_round: int = 1
    sharded: bool = True


class _Family:
    def __init__(self, spec: _FamilySpec, dtype, device, shard_divisible_by, keep_state: bool):
        self.spec = spec
        self.dtype, self.device = dtype, device
        sizes = [p.numel() for p in spec.params]
        self.param_sizes = sizes
        self.param_start_inds = [0] * len(sizes)
        run = 0
        for i, s in enumerate(sizes):
            self.param_start_inds[i] = run
            run += s
        self.numel = run
        n = spec.num_shards if spec.sharded else 1
        self.slices: List[_Slice] = []
        if not spec.sharded:
            self.flat_size = self.numel
            self.shard_size = self.numel
            self.slices.append(_Slice(0, self.numel, self.numel, 0))
        elif spec.chunk_limit is None:
            self.shard_size = int(math.ceil(self.numel / (n * shard_divisible_by))) * shard_divisible_by
            self.flat_size = n * self.shard_size
            self.slices.append(_Slice(0, self.flat_size, self.shard_size, 0))
        else:
            chunk = self._chunk_size(spec, n)
            num_chunks = max(1, int(math.ceil(self.numel / chunk)))
            sub = chunk // n
            self.flat_size = num_chunks * chunk
            self.shard_size = num_chunks * sub
            for c in range(num_chunks):
                self.slices.append(_Slice(c * chunk, chunk, sub, c * sub))
            self.chunk_size, self.num_chunks, self.sub_chunk_size = chunk, num_chunks, sub

        self.flat_param = torch.zeros(self.flat_size, dtype=dtype, device=device)
        self.flat_grad = torch.zeros(self.flat_size, dtype=dtype, device=device)
        for p, start, size in zip(spec.params, self.param_start_inds, sizes):
            view = self.flat_param[start:start + size].view_as(p.data)
            view.copy_(p.data)
            p.data = view
            p.grad = self.flat_grad[start:start + size].view_as(p.data)

        self.exp_avg = self.exp_avg_sq = self.master = None
        if keep_state:
            self.exp_avg = torch.zeros(self.shard_size, dtype=torch.float32, device=device)
            self.exp_avg_sq = torch.zeros(self.shard_size, dtype=torch.float32, device=device)
            if dtype == torch.float32 and not spec.sharded:
                self.master = self.flat_param  # fp32 run: master aliases the parameters
            else:
                self.master = torch.zeros(self.shard_size, dtype=torch.float32, device=device)
                for sl in self.slices:
                    self.master[sl.state_start:sl.state_start + sl.part].copy_(self.param_part(sl))

    @staticmethod
    def _chunk_size(spec: _FamilySpec, n: int) -> int:
        r = spec.chunk_round
        if r <= 1:
            return (spec.chunk_limit // n) * n            # "subshard": floor to a multiple of DP
        return int(math.ceil(spec.chunk_limit / (n * r))) * (n * r)  # "pgsubshard": ceil to n*512

    # views of this rank's part of a slice
    def _part_range(self, sl: _Slice) -> Tuple[int, int]:
        sid = self.spec.shard_id if self.spec.sharded else 0
        lo = sl.flat_start + sid * sl.part
        return lo, lo + sl.part

    def grad_part(self, sl):
        lo, hi = self._part_range(sl)
        return self.flat_grad[lo:hi]

    def param_part(self, sl):
        lo, hi = self._part_range(sl)
        return self.flat_param[lo:hi]

    def grad_region(self, sl):
        return self.flat_grad[sl.flat_start:sl.flat_start + sl.length]

    def param_region(self, sl):
        return self.flat_param[sl.flat_start:sl.flat_start + sl.length]


class _FlatAdamWEngine(Optimizer):
    """Shared implementation; subclasses only describe their families and state-dict keys."""

    opt_key = "flat"

    def _setup(self, params, model, lr, betas, eps, weight_decay, warmup_steps, dtype, device,
               opt_disable_delayed_grad_clipping, profiler, tensor_parallelism, tp_ind, tp_group,
               expert_parallelism, ep_ind, ep_group, dpep_ind, dpep_group, shard_divisible_by,
               opt_use_chunked_allreduce, opt_use_allreduce_for_grad_acc, opt_use_allreduce_for_param_gather,
               skip_optimizer_step, disable_optimizer_state_checkpointing, skip_optimizer_step_weight_update,
               num_shards, shard_id, group, verbose=False):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        Optimizer.__init__(self, params, defaults)
        assert device is not None
        assert len(self.param_groups) == 1, "Only one parameter group is supported"
        self.model = model
        self.warmup_steps = warmup_steps
        self.dtype, self.device = dtype, torch.device(device)
        self.opt_disable_delayed_grad_clipping = opt_disable_delayed_grad_clipping
        self.profiler = profiler
        self.tensor_parallelism, self.tp_ind, self.tp_group = tensor_parallelism, tp_ind, tp_group
        self.expert_parallelism, self.ep_ind, self.ep_group = expert_parallelism, ep_ind, ep_group
        self.dpep_ind, self.dpep_group = dpep_ind, dpep_group
        self.shard_divisible_by = shard_divisible_by
        self.opt_use_chunked_allreduce = opt_use_chunked_allreduce
        self.opt_use_allreduce_for_grad_acc = opt_use_allreduce_for_grad_acc
        self.opt_use_allreduce_for_param_gather = opt_use_allreduce_for_param_gather
        self.skip_optimizer_step = skip_optimizer_step
        self.disable_optimizer_state_checkpointing = disable_optimizer_state_checkpointing
        self.skip_optimizer_step_weight_update = skip_optimizer_step_weight_update
        self.verbose = verbose
        self.data_parallelism = self.num_shards = num_shards
        self.dp_ind = shard_id
        self.dp_group = self.group = group
        self.step_id = 0
        self.max_grad_norm = 1.0
        self.param_list = [p for pg in self.param_groups for p in pg["params"]]
        # set by the driver after construction (reference dist_train.py:572-574)
        self.pmap = None
        self.config = None
        self.dump_weight_gradients = False
        self.families: List[_Family] = []
        self._fused = None  # fused reduce-scatter + AdamW backend, when enabled

    def _add_family(self, spec: _FamilySpec):
        fam = _Family(spec, self.dtype, self.device, self.shard_divisible_by, keep_state=not self.skip_optimizer_step)
        self.families.append(fam)
        return fam

    def _report(self):
        if not (dist.is_available() and dist.is_initialized() and dist.get_rank() == 0):
            return
        bar = "*" * 80
        lines = [bar]
        for fam in self.families:
            n = fam.spec.num_shards if fam.spec.sharded else 1
            ideal = fam.numel // n
            tag = f" ({fam.spec.name})" if fam.spec.name else ""
            lines += [f"Total number of parameters{tag} : {fam.numel}",
                      f"Number of shards           : {n}",
                      f"Ideal shard size           : {ideal}",
                      f"Actual Shard size          : {fam.shard_size} (Padding : {fam.shard_size - ideal})",
                      f"Padding percentage         : {(1.0 - ideal / max(1, fam.shard_size)) * 100:.3f} %",
                      f"Flat parameter size        : {fam.flat_size}"]
        lines.append(bar)
        print("\n".join(lines), flush=True)

    # ------------------------------------------------------------------ public API
    def enable_direct_grads(self):
        """Let the weight-gradient GEMMs store into the ``.grad`` views of the flat buffers themselves
        (``ops.functional.DirectGrad``): ``zero_grad`` then only zeroes the few gradients that still go through
        autograd's accumulation (norm weights, embeddings) instead of the whole flat buffer."""
        params = [p for fam in self.families for p in fam.spec.params]
        self._direct, self._other_grads = OF.enable_direct_grads(params)
        return len(self._direct)

    def _finish_direct_grads(self):
        # a weight that received no gradient in this optimizer step keeps stale data: zero it
        for h in getattr(self, "_direct", ()):
            if not h.ready:
                h.buf.zero_()
                h.ready = True

    def zero_grad(self, set_to_none: bool = False):
        direct = getattr(self, "_direct", None)
        if direct:
            for h in direct:
                h.ready = False
            if self._other_grads:
                torch._foreach_zero_(self._other_grads)
            return
        for fam in self.families:
            fam.flat_grad.zero_()

    # ------------------------------------------------------------------ updates underneath the backward
    def enable_early_updates(self, layers) -> int:
        """Let the AdamW update of a decoder layer run on a side stream as soon as that layer's backward has
        finished, underneath the backward of the layers before it (the update is bound by HBM bandwidth, the
        backward by the tensor cores).  ``layers``: one list of parameters per decoder layer.  Only parameters of
        families that need no gradient reduction (one shard) take part, and only while gradient clipping is
        inactive - with delayed clipping the reference does not clip during the first ``warmup_steps`` optimizer
        steps (optimus/optimizers.py:394-412), so the norm is a by-product there and the update needs no global
        quantity.  Everything else is updated in ``step`` as before.  Returns the number of layers enabled."""
        self._early_layers = []
        if self.device.type != "cuda" or self.skip_optimizer_step or type(self)._norm_sq_local is not _FlatAdamWEngine._norm_sq_local:
            return 0
        for params in layers:
            ids = {id(p) for p in params}
            ranges = []
            for fam in self.families:
                if (_group_ok(fam.spec.group) and fam.spec.num_shards > 1) or len(fam.slices) != 1 or fam.master is None:
                    continue
                idx = [i for i, p in enumerate(fam.spec.params) if id(p) in ids]
                if not idx:
                    continue
                if idx != list(range(idx[0], idx[-1] + 1)):
                    ranges = None  # the layer's parameters are not one run of the flat buffer
                    break
                lo = fam.param_start_inds[idx[0]]
                hi = fam.param_start_inds[idx[-1]] + fam.param_sizes[idx[-1]]
                if lo % 8 or (hi - lo) % 8:
                    ranges = None
                    break
                holders = [h for h in (getattr(fam.spec.params[i], "_olb_direct", None) for i in idx) if h is not None]
                ranges.append((fam, lo, hi, holders))
            self._early_layers.append(ranges or [])
        self._early_stream = torch.cuda.Stream(device=self.device)
        self._early_sq = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._early_done = {}      # id(family) -> [(lo, hi), ...] updated during this step's backward
        self._early_armed = False
        return sum(1 for r in self._early_layers if r)

    def arm_early_updates(self, armed: bool):
        """Called before a forward pass: ``armed`` when its backward is the last one before ``step``."""
        if getattr(self, "_early_layers", None):
            self._early_armed = bool(armed) and not self._clipping_active()

    @torch.no_grad()
    def early_update_layer(self, layer_idx: int):
        """Backward hook: the gradients of layer ``layer_idx`` are final; update its parameters on the side stream."""
        if not getattr(self, "_early_armed", False):
            return
        ranges = self._early_layers[layer_idx]
        if not ranges:
            return
        beta1, beta2 = self.defaults["betas"]
        eps, wd = self.defaults["eps"], self.defaults["weight_decay"]
        lr = self.param_groups[0]["lr"]
        for fam, lo, hi, holders in ranges:
            for h in holders:
                if not h.ready:            # received no gradient in this step
                    h.buf.zero_()
                    h.ready = True
        main = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(main)
        with torch.cuda.stream(self._early_stream):
            self._early_stream.wait_event(ev)
            for fam, lo, hi, _ in ranges:
                if any(lo < b and a < hi for a, b in self._early_done.get(id(fam), ())):
                    continue               # already updated (a hook that fired twice)
                scale = 1.0 / fam.spec.grad_divisor
                OF.sum_of_squares(fam.flat_grad[lo:hi], scale, out=self._early_sq, accumulate=True)
                OF.adamw_step(fam.flat_grad[lo:hi], fam.master[lo:hi], fam.exp_avg[lo:hi], fam.exp_avg_sq[lo:hi],
                              fam.flat_param[lo:hi], lr, beta1, beta2, eps, wd, self.step_id + 1, grad_scale=scale,
                              clip_coef=None, skip_weight_update=self.skip_optimizer_step_weight_update)
                self._early_done.setdefault(id(fam), []).append((lo, hi))

    def _pending_ranges(self, fam: _Family, sl: _Slice):
        """The parts ``(lo, hi)`` of this rank's part of slice ``sl`` (offsets inside the part) that ``step`` still has
        to update: everything, minus what the backward hooks have updated already."""
        done = sorted(getattr(self, "_early_done", {}).get(id(fam), ()))
        if not done:
            return [(0, sl.part)]
        out, cur = [], 0
        for lo, hi in done:
            if lo > cur:
                out.append((cur, lo))
            cur = max(cur, hi)
        if cur < sl.part:
            out.append((cur, sl.part))
        return out

    def _join_early_updates(self):
        """Before ``step`` touches anything: the side stream's updates are ordered before the current stream.
        Returns the sum of squares of the gradients they covered (None when there were none)."""
        if not getattr(self, "_early_done", None):
            return None
        ev = torch.cuda.Event()
        ev.record(self._early_stream)
        torch.cuda.current_stream(self.device).wait_event(ev)
        return self._early_sq

    def _finish_early_updates(self):
        if getattr(self, "_early_done", None):
            self._early_done = {}
            self._early_sq.zero_()
        self._early_armed = False

    def _clipping_active(self) -> bool:
        return self.opt_disable_delayed_grad_clipping or self.step_id >= self.warmup_steps

    def _pre_reduce(self):
        """Hook: per-class work before the family reductions."""

    def _norm_sq_local(self) -> torch.Tensor:
        acc = torch.zeros(1, dtype=torch.float32, device=self.device)
        for fam in self.families:
            scale = 1.0 / fam.spec.grad_divisor
            for sl in fam.slices:
                g = fam.grad_part(sl)
                for lo, hi in self._pending_ranges(fam, sl):
                    OF.sum_of_squares(g[lo:hi], scale, out=acc, accumulate=True)
        return acc

    def _reduce_family(self, fam: _Family):
        spec = fam.spec
        if not (_group_ok(spec.group) and spec.num_shards > 1):
            return
        use_ar = self.opt_use_allreduce_for_grad_acc or not spec.sharded or not _has_reduce_scatter(spec.group)
        for sl in fam.slices:
            region = fam.grad_region(sl)
            name = f"3dp-comms--1grad_acc{('-' + spec.name) if spec.name else ''}"
            with record_pcl_function(name):
                if use_ar:
                    if self.opt_use_chunked_allreduce:
                        chunked_allreduce_wrapper(region, spec.group)
                    else:
                        dist.all_reduce(region, group=spec.group)
                else:
                    dist.reduce_scatter_tensor(fam.grad_part(sl), region, group=spec.group)

    def _gather_family(self, fam: _Family):
        spec = fam.spec
        if not (spec.sharded and _group_ok(spec.group) and spec.num_shards > 1):
            return
        for sl in fam.slices:
            name = f"3dp-comms--2param_gather{('-' + spec.name) if spec.name else ''}"
            with record_pcl_function(name):
                if self.opt_use_allreduce_for_param_gather:
                    region = fam.param_region(sl)
                    lo, hi = fam._part_range(sl)
                    keep = fam.flat_param[lo:hi].clone()
                    region.zero_()
                    fam.flat_param[lo:hi].copy_(keep)
                    if self.opt_use_chunked_allreduce:
                        chunked_allreduce_wrapper(region, spec.group)
                    else:
                        dist.all_reduce(region, group=spec.group)
                else:
                    dist.all_gather_into_tensor(fam.param_region(sl), fam.param_part(sl), group=spec.group)

    def _global_norm(self, norm_sq: torch.Tensor) -> torch.Tensor:
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 and self._norm_is_distributed():
            dist.all_reduce(norm_sq)
        return norm_sq.sqrt()

    def _norm_is_distributed(self) -> bool:
        return any(f.spec.sharded and f.spec.num_shards > 1 for f in self.families) or self.expert_parallelism > 1 \
            or self.tensor_parallelism > 1 or (self.pmap is not None and self.pmap.pipeline_parallelism > 1)

    @torch.no_grad()
    def step(self, closure=None):
        self._finish_direct_grads()
        if self.dump_weight_gradients and self.pmap is not None:
            from .utils import dump_weight_gradients
            dump_weight_gradients(self.model, self.config, self.pmap, self.opt_key, "beforegradacc")

        fused =self._fused if (self._fused is not None and self._fused.usable(self)) else None
        with record_pcl_function("3dp-comms-1grad_acc-block"):
            self._pre_reduce()
            if fused is None:
                for fam in self.families:
                    self._reduce_family(fam)

        if self.dump_weight_gradients and self.pmap is not None:
            from .utils import dump_weight_gradients
            dump_weight_gradients(self.model, self.config, self.pmap, self.opt_key, "aftergradacc")

        if fused is not None:
            grad_norm = fused.step(self)
            self._finish_early_updates()
            self.step_id += 1
            return grad_norm

        with record_pcl_function("4opt-step_grad-clip"):
            early_sq = self._join_early_updates()
            # While clipping is inactive the update does not depend on the norm: the AdamW kernel then sums the
            # squares of the gradients it reads anyway, and the separate pass over the gradients is skipped.
            norm_in_update = (not self._clipping_active() and not self.skip_optimizer_step
                              and type(self)._norm_sq_local is _FlatAdamWEngine._norm_sq_local)
            norm_sq = torch.zeros(1, dtype=torch.float32, device=self.device) if norm_in_update else self._norm_sq_local()
            if early_sq is not None:
                norm_sq = norm_sq + early_sq
            clip_coef = None
            if not norm_in_update:
                grad_norm = self._global_norm(norm_sq).reshape(())
                if self._clipping_active():
                    clip_coef = torch.clamp(self.max_grad_norm / (grad_norm + 1e-6), max=1.0).reshape(1).float()

        if not self.skip_optimizer_step:
            with record_pcl_function("4opt-step_compute"):
                beta1, beta2 = self.defaults["betas"]
                eps, wd = self.defaults["eps"], self.defaults["weight_decay"]
                lr = self.param_groups[0]["lr"]
                for fam in self.families:
                    for sl in fam.slices:
                        g, pp = fam.grad_part(sl), fam.param_part(sl)
                        for lo, hi in self._pending_ranges(fam, sl):
                            s0, s1 = sl.state_start + lo, sl.state_start + hi
                            OF.adamw_step(g[lo:hi], fam.master[s0:s1], fam.exp_avg[s0:s1], fam.exp_avg_sq[s0:s1],
                                          pp[lo:hi], lr, beta1, beta2, eps, wd, self.step_id + 1,
                                          grad_scale=1.0 / fam.spec.grad_divisor, clip_coef=clip_coef,
                                          skip_weight_update=self.skip_optimizer_step_weight_update,
                                          norm_out=norm_sq if norm_in_update else None)
        if norm_in_update:
            grad_norm = self._global_norm(norm_sq).reshape(())
        self._finish_early_updates()
        with record_pcl_function("3dp-comms-2param_gather-block"):
            for fam in self.families:
                self._gather_family(fam)

        self.step_id += 1
        return grad_norm

    # ------------------------------------------------------------------ checkpoint state
    _STATE_SUFFIX = ""  # "" for unsharded keys, "_shard" for sharded ones

    def _state_items(self):
        for fam in self.families:
            tail = self._STATE_SUFFIX + (f"_{fam.spec.name}" if fam.spec.name else "")
            yield f"flat_exp_avg{tail}", fam, "exp_avg"
            yield f"flat_exp_avg_sq{tail}", fam, "exp_avg_sq"
            yield f"flat_fp32_master_param{tail}", fam, "master"

    def state_dict(self):
        out = {}
        if not self.disable_optimizer_state_checkpointing:
            for key, fam, attr in self._state_items():
                out[key] = getattr(fam, attr)
        out["step_id"] = self.step_id
        return out

    def load_state_dict(self, opt_state_dict):
        for key, fam, attr in self._state_items():
            if key in opt_state_dict and getattr(fam, attr) is not None:
                getattr(fam, attr).copy_(opt_state_dict[key].to(self.device))
        self.step_id = opt_state_dict["step_id"]
        for key, fam, attr in self._state_items():
            if attr != "master" or fam.master is None or fam.master is fam.flat_param:
                continue
            for sl in fam.slices:
                m = fam.master[sl.state_start:sl.state_start + sl.part]
                if key in opt_state_dict:
                    fam.param_part(sl).copy_(m)   # parameters follow the restored master weights
                else:
                    m.copy_(fam.param_part(sl))   # no saved state: restart the master from the weights

    # convenient aliases with the reference's attribute names (single-family classes)
    def _alias_single(self):
        fam = self.families[0]
        self.flat_param, self.flat_grad = fam.flat_param, fam.flat_grad
        self.flat_param_size = fam.numel
        self.shard_size = fam.shard_size
        self.flat_buffer_size = fam.flat_size
        sfx = self._STATE_SUFFIX
        setattr(self, f"flat_exp_avg{sfx}", fam.exp_avg)
        setattr(self, f"flat_exp_avg_sq{sfx}", fam.exp_avg_sq)
        setattr(self, f"flat_fp32_master_param{sfx}", fam.master)
        if fam.spec.sharded and len(fam.slices) == 1:
            self.flat_param_shard = fam.param_part(fam.slices[0])
            self.flat_grad_shard = fam.grad_part(fam.slices[0])

    def _alias_pair(self):
        for fam in self.families:
            n = fam.spec.name
            setattr(self, f"flat_param_{n}", fam.flat_param)
            setattr(self, f"flat_grad_{n}", fam.flat_grad)
            setattr(self, f"shard_size_{n}", fam.shard_size)
            setattr(self, f"flat_exp_avg_shard_{n}", fam.exp_avg)
            setattr(self, f"flat_exp_avg_sq_shard_{n}", fam.exp_avg_sq)
            setattr(self, f"flat_fp32_master_param_shard_{n}", fam.master)
            if len(fam.slices) == 1:
                setattr(self, f"flat_param_shard_{n}", fam.param_part(fam.slices[0]))
                setattr(self, f"flat_grad_shard_{n}", fam.grad_part(fam.slices[0]))


# ---------------------------------------------------------------------------------------------
class MixedPrecisionAdamW(_FlatAdamWEngine):
    """Unsharded optimizer (reference :19-225).  ``num_shards``/``group`` name the data-parallel
    group whose flat gradient is all-reduced and averaged.  Clipping uses the norm of the whole
    (already averaged) gradient."""

    opt_key = "unsharded"
    _STATE_SUFFIX = ""

    def __init__(self, params, model, lr=0.001, betas=(0.9, 0.999), eps=1e-08, weight_decay=0.01, warmup_steps=0,
                 dtype=torch.float32, device=None, num_shards=1, shard_id=0, group=None,
                 opt_disable_delayed_grad_clipping=False, opt_use_two_step_grad_clipping=False,
                 opt_use_chunked_allreduce=False, profiler=None, tensor_parallelism=1, tp_ind=0, tp_group=None,
                 expert_parallelism=1, ep_ind=0, ep_group=None, dpep_ind=0, dpep_group=None,
                 skip_optimizer_step=False, **_ignored):
        assert expert_parallelism == 1, "This optimizer does not support expert parallelism."
        self._setup(params, model, lr, betas, eps, weight_decay, warmup_steps, dtype, device,
                    opt_disable_delayed_grad_clipping, profiler, tensor_parallelism, tp_ind, tp_group,
                    expert_parallelism, ep_ind, ep_group, dpep_ind, dpep_group, 512, opt_use_chunked_allreduce,
                    True, False, skip_optimizer_step, False, False, num_shards, shard_id, group)
        self.opt_use_two_step_grad_clipping = opt_use_two_step_grad_clipping
        self._add_family(_FamilySpec("", self.param_list, group, num_shards, shard_id, float(max(1, num_shards)),
                                     sharded=False))
        self._alias_single()

    def _norm_sq_local(self):
        if self.tensor_parallelism > 1 and hasattr(self.model, "calculate_grad_norm"):
            # the model knows which gradients are replicated over the TP group
            n = self.model.calculate_grad_norm(grad_scale=1.0 / self.families[0].spec.grad_divisor)
            return (n.float() ** 2).reshape(1)
        return super()._norm_sq_local()

    def _global_norm(self, norm_sq):
        # every rank holds the full averaged gradient (TP: reduced inside calculate_grad_norm)
        return norm_sq.sqrt()


class ShardedMixedPrecisionAdamW(_FlatAdamWEngine):
    """ZeRO-1 over the data-parallel group (reference :227-522).

    With expert parallelism the EP-replicated gradients are first all-reduced over the EP
    group, and *all* gradients (experts included) are divided by EP - the reference's scaling,
    kept for loss-curve parity.  For the global norm, gradients that are replicated over EP
    (TP) ranks count with weight 1/EP (1/TP)."""

    opt_key = "shard"
    _STATE_SUFFIX = "_shard"

    def __init__(self, params, model, lr=0.001, betas=(0.9, 0.999), eps=1e-08, weight_decay=0.01, warmup_steps=0,
                 dtype=torch.float32, device=None, num_shards=1, shard_id=0, group=None,
                 opt_disable_delayed_grad_clipping=False, profiler=None, tensor_parallelism=1, tp_ind=0,
                 tp_group=None, expert_parallelism=1, ep_ind=0, ep_group=None, dpep_ind=0, dpep_group=None,
                 shard_divisible_by=512, opt_use_chunked_allreduce=False, opt_use_allreduce_for_grad_acc=False,
                 opt_use_allreduce_for_param_gather=False, skip_optimizer_step=False,
                 disable_optimizer_state_checkpointing=False, skip_optimizer_step_weight_update=False,
                 _chunk_limit=None, **_ignored):
        self._setup(params, model, lr, betas, eps, weight_decay, warmup_steps, dtype, device,
                    opt_disable_delayed_grad_clipping, profiler, tensor_parallelism, tp_ind, tp_group,
                    expert_parallelism, ep_ind, ep_group, dpep_ind, dpep_group, shard_divisible_by,
                    opt_use_chunked_allreduce, opt_use_allreduce_for_grad_acc, opt_use_allreduce_for_param_gather,
                    skip_optimizer_step, disable_optimizer_state_checkpointing, skip_optimizer_step_weight_update,
                    num_shards, shard_id, group)
        divisor = float(max(1, num_shards)) * float(max(1, expert_parallelism))
        self._add_family(_FamilySpec("", self.param_list, group, max(1, num_shards), shard_id, divisor,
                                     chunk_limit=_chunk_limit, chunk_round=1))
        self._alias_single()
        self._replicated_ranges = None
        self._report()

    # which flat-buffer ranges hold EP-/TP-replicated parameters (merged into maximal runs)
    def _replicated_param_ranges(self):
        if self._replicated_ranges is not None:
            return self._replicated_ranges
        weights = {}
        names = {id(p): n for n, p in self.model.named_parameters()}
        ep_rep = set(self.model.get_ep_replicated_param_list()) if (
            self.expert_parallelism > 1 and hasattr(self.model, "get_ep_replicated_param_list")) else set()
        tp_rep = set(self.model.get_tp_replicated_param_list()) if (
            self.tensor_parallelism > 1 and hasattr(self.model, "get_tp_replicated_param_list")) else set()
        fam = self.families[0]
        runs = []
        for p, start, size in zip(fam.spec.params, fam.param_start_inds, fam.param_sizes):
            n = names.get(id(p))
            w = 1.0
            if n in ep_rep:
                w /= self.expert_parallelism
            if n in tp_rep:
                w /= self.tensor_parallelism
            if w == 1.0:
                continue
            if runs and runs[-1][1] == start and runs[-1][2] == w:
                runs[-1][1] = start + size
            else:
                runs.append([start, start + size, w])
        self._replicated_ranges = runs
        return runs

    def _pre_reduce(self):
        if self.expert_parallelism > 1 and _group_ok(self.ep_group):
            rep = set(self.model.get_ep_replicated_param_list())
            with record_pcl_function("3dp-comms--0ep_replicated_allreduce"):
                for name, p in self.model.named_parameters():
                    if name in rep:
                        dist.all_reduce(p.grad, group=self.ep_group)

    def _norm_sq_local(self):
        acc = super()._norm_sq_local()
        runs = self._replicated_param_ranges()
        if not runs:
            return acc
        fam = self.families[0]
        scale = 1.0 / fam.spec.grad_divisor
        corr = torch.zeros(1, dtype=torch.float32, device=self.device)
        for sl in fam.slices:
            lo, hi = fam._part_range(sl)
            for a, b, w in runs:
                x, y = max(a, lo), min(b, hi)
                if x < y:
                    # replicated elements count with weight w instead of 1
                    OF.sum_of_squares(fam.flat_grad[x:y].contiguous(), scale * math.sqrt(1.0 - w), out=corr,
                                      accumulate=True)
        return acc - corr


class ParamGroupShardedMixedPrecisionAdamW(_FlatAdamWEngine):
    """Two parameter families (reference :524-961): EP-replicated parameters sharded over the
    DP x EP group (index ``dpep_ind``), expert ("divided") parameters sharded over DP.
    Replicated gradients are averaged over DP*EP, expert gradients over DP only."""

    opt_key = "pgshard"
    _STATE_SUFFIX = "_shard"

    def __init__(self, params, model, lr=0.001, betas=(0.9, 0.999), eps=1e-08, weight_decay=0.01, warmup_steps=0,
                 dtype=torch.float32, device=None, num_shards=1, shard_id=0, group=None,
                 opt_disable_delayed_grad_clipping=False, profiler=None, tensor_parallelism=1, tp_ind=0,
                 tp_group=None, expert_parallelism=1, ep_ind=0, ep_group=None, dpep_ind=0, dpep_group=None,
                 shard_divisible_by=512, opt_use_chunked_allreduce=False, opt_use_allreduce_for_grad_acc=True,
                 opt_use_allreduce_for_param_gather=False, skip_optimizer_step=False, verbose=False,
                 disable_optimizer_state_checkpointing=False, skip_optimizer_step_weight_update=False,
                 _chunk_limit=None, **_ignored):
        assert tensor_parallelism == 1, f"{type(self).__name__} does not support tensor parallelism."
        self._setup(params, model, lr, betas, eps, weight_decay, warmup_steps, dtype, device,
                    opt_disable_delayed_grad_clipping, profiler, tensor_parallelism, tp_ind, tp_group,
                    expert_parallelism, ep_ind, ep_group, dpep_ind, dpep_group, shard_divisible_by,
                    opt_use_chunked_allreduce, opt_use_allreduce_for_grad_acc, opt_use_allreduce_for_param_gather,
                    skip_optimizer_step, disable_optimizer_state_checkpointing, skip_optimizer_step_weight_update,
                    num_shards, shard_id, group, verbose)
        dp, ep = max(1, num_shards), max(1, expert_parallelism)
        rep_names = set(model.get_ep_replicated_param_list())
        mine = {id(p) for p in self.param_list}
        rep = [p for n, p in model.named_parameters() if n in rep_names and id(p) in mine]
        div = [p for n, p in model.named_parameters() if n not in rep_names and id(p) in mine]
        rnd = shard_divisible_by if _chunk_limit is not None else 1
        self._add_family(_FamilySpec("replicated", rep, dpep_group, dp * ep, dpep_ind, float(dp * ep),
                                     chunk_limit=_chunk_limit, chunk_round=rnd))
        self._add_family(_FamilySpec("divided", div, group, dp, shard_id, float(dp),
                                     chunk_limit=_chunk_limit, chunk_round=rnd))
        self._alias_pair()
        self._report()


class SubShardedMixedPrecisionAdamW(ShardedMixedPrecisionAdamW):
    """"shard" with the flat buffer cut into chunks of at most 128Mi elements, each chunk sharded
    over DP on its own (reference :963-1242): bounds the size of every collective."""

    opt_key = "subshard"

    def __init__(self, *args, chunk_size_limit=CHUNK_ELEMS, **kwargs):
        self.chunk_size_limit = chunk_size_limit
        super().__init__(*args, _chunk_limit=chunk_size_limit, **kwargs)


class ParamGroupSubShardedMixedPrecisionAdamW(ParamGroupShardedMixedPrecisionAdamW):
    """"pgshard" with chunked families (reference :1244-1742)."""

    opt_key = "pgsubshard"

    def __init__(self, *args, chunk_size_limit=CHUNK_ELEMS, opt_use_fp32_for_grad_acc=False,
                 opt_alternate_compute_and_comms=True, **kwargs):
        self.chunk_size_limit = chunk_size_limit
        self.opt_use_fp32_for_grad_acc = opt_use_fp32_for_grad_acc
        self.opt_alternate_compute_and_comms = opt_alternate_compute_and_comms
        super().__init__(*args, _chunk_limit=chunk_size_limit, **kwargs)


class TorchAdamW:
    """``--opt_use_pt_optimizer``: ``torch.optim.AdamW`` on the model's own parameters (reference
    dist_train.py:575-589, 889-906).  The reference wraps the model in DistributedDataParallel when there are
    data-parallel replicas; here the gradients are averaged over the data-parallel group right before the
    update, which gives the same numbers without a wrapper module around the model.  Gradient clipping to norm 1
    starts after ``warmup_steps`` optimizer steps unless delayed clipping is disabled, with the local norm as in the
    reference.  Takes the constructor keywords of the flat-buffer classes and ignores those it has no use for."""

    def __init__(self, params, model, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, warmup_steps=0,
                 num_shards=1, group=None, opt_disable_delayed_grad_clipping=False, skip_optimizer_step=False,
                 opt_use_one_step_grad_clipping=False, **_unused):
        self.model = model
        self.inner = torch.optim.AdamW(list(params), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        self.param_groups = self.inner.param_groups
        self.defaults = self.inner.defaults
        self.warmup_steps = warmup_steps
        self.num_shards, self.group = num_shards, group
        self.opt_disable_delayed_grad_clipping = opt_disable_delayed_grad_clipping
        self.skip_optimizer_step = skip_optimizer_step
        self.one_step_clipping = opt_use_one_step_grad_clipping
        self.max_grad_norm = 1.0
        self.step_id = 0

    def _params(self):
        return [p for g in self.param_groups for p in g["params"] if p.grad is not None]

    @torch.no_grad()
    def step(self):
        ps = self._params()
        if self.num_shards > 1 and _group_ok(self.group):
            for p in ps:
                dist.all_reduce(p.grad, group=self.group)
                p.grad.div_(self.num_shards)
        grads = [p.grad for p in ps]
        grad_norm = torch.nn.utils.get_total_norm(grads) if grads else torch.zeros(())
        if grads and (self.opt_disable_delayed_grad_clipping or self.step_id >= self.warmup_steps):
            torch.nn.utils.clip_grads_with_norm_(ps, self.max_grad_norm, grad_norm)
        if not self.skip_optimizer_step:
            self.inner.step()
        self.step_id += 1
        return grad_norm

    def zero_grad(self, set_to_none=True):
        self.inner.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return {"inner": self.inner.state_dict(), "step_id": self.step_id}

    def load_state_dict(self, sd):
        self.inner.load_state_dict(sd["inner"])
        self.step_id = int(sd.get("step_id", 0))
        self.param_groups = self.inner.param_groups


OPTIMIZER_CLASSES = {
    "pt": TorchAdamW,
    "unsharded": MixedPrecisionAdamW,
    "shard": ShardedMixedPrecisionAdamW,
    "pgshard": ParamGroupShardedMixedPrecisionAdamW,
    "subshard": SubShardedMixedPrecisionAdamW,
    "pgsubshard": ParamGroupSubShardedMixedPrecisionAdamW,
}
