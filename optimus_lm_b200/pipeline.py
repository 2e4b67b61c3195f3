"""Pipeline-parallel executor: walks a schedule from ``schedules.py`` and moves activations and
gradients between stages with asynchronous NCCL (or gloo) point-to-point operations.

Differences from the reference trainers (optimus/training.py:18-497, optimus/trainer.py:184-871),
which use blocking ``send``/``recv`` followed by a device synchronise after every micro-step:

* sends are ``isend`` and are only waited for at the end of the step, so a stage starts its next
  micro-batch while the previous output is still in flight; receives are posted when the data is
  needed and only the compute stream waits for them - the host never synchronises;
* every (sender, receiver) pair of neighbouring stages has two process groups of its own, of two ranks each: one
  for the activations going forward, one for the gradients coming back (the wrap-around pair of virtual
  pipelining is one more such pair).  Every channel is then one-directional and in schedule order on both
  ends, which makes the exchange dead-lock free without the reference's recv-before-send choreography; and
  because each group has its own communicator and stream, a transfer waits neither for the other
  direction nor for the collectives of the data / expert / tensor parallel groups.  The operations are
  issued through ``batch_isend_irecv``;
* the global router auxiliary loss travels as ``2E+2`` running sums forward and the global
  selection fractions (``E`` floats) backward instead of the concatenated router logits and their
  gradients (see ``ops/aux_loss.py``);
* activation buffers are allocated per micro-batch in flight from the caching allocator
  (``reuse_buffers_in_1f1b`` is accepted for compatibility; reuse is implicit).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .ops import aux_loss as AL
from .ops import functional as OF
from .profilers import record_pcl_function
from .schedules import Interleaved1f1bBufferManager, PipeOp, make_schedule


class ParallelTrainerOutput:
    def __init__(self, loss=None, logits=None):
        self.loss = loss
        self.logits = logits


class _MicroState:
    __slots__ = ("inp", "out", "loss_scaled", "logits_list", "idx_list", "stats", "prev_stats", "f_global",
                 "aux_partial")

    def __init__(self):
        for s in self.__slots__:
            setattr(self, s, None)


_CHANNEL_GROUPS: Dict[str, object] = {}
_PAIR_GROUPS: Dict[Tuple[int, int, str], object] = {}


def _channel_groups(need_wrap: bool):
    """One world-size process group per traffic direction (the fall-back when the stage neighbours of the other ranks
    cannot be derived from the mapper)."""
    names = ["fwd", "bwd"] + (["wrap_fwd", "wrap_bwd"] if need_wrap else [])
    for n in names:
        if n not in _CHANNEL_GROUPS:
            _CHANNEL_GROUPS[n] = dist.new_group(list(range(dist.get_world_size())))
    return _CHANNEL_GROUPS


def _pair_groups(pmap):
    """Two-rank process groups for every (stage rank -> next stage rank) pair of the job, one for each direction of
    traffic: ``(src, dst, "fwd")`` carries activations from ``src`` to ``dst``, ``(src, dst, "bwd")`` the gradients from
    ``dst`` back to ``src``.  Group creation is collective, so every rank walks all pairs in the same order.  Returns
    ``None`` when the mapper cannot be instantiated for other ranks (legacy mappers)."""
    world = dist.get_world_size()
    if _PAIR_GROUPS:
        return _PAIR_GROUPS
    try:
        nexts = []
        for r in range(world):
            other = type(pmap)(pmap.data_parallelism, pmap.pipeline_parallelism, pmap.expert_parallelism,
                               pmap.tensor_parallelism, rank=r, create_groups=False,
                               use_pp_first=getattr(pmap, "use_pp_first", False))
            nexts.append(other.next_stage_rank)
    except Exception:  # noqa: BLE001 - a mapper with another constructor: keep the world-size channels
        return None
    for r in range(world):
        if nexts[r] == r:
            continue
        for kind in ("fwd", "bwd"):
            _PAIR_GROUPS[(r, nexts[r], kind)] = dist.new_group(sorted((r, nexts[r])))
    return _PAIR_GROUPS


class PipelineExecutor:
    def __init__(self, config, model, pmap, batch_size, micro_batch_size, context_size, opt_grad_acc_steps, dtype,
                 device, pp_scheme="gpipe", reuse_buffers_in_1f1b=True, verbose=False, memory_tracker=None):
        self.config, self.model, self.pmap = config, model, pmap
        self.dtype, self.device = dtype, device
        self.pp_scheme = pp_scheme
        self.batch_size, self.micro_batch_size, self.context_size = batch_size, micro_batch_size, context_size
        self.opt_grad_acc_steps = opt_grad_acc_steps
        assert batch_size % micro_batch_size == 0, "Batch size must be divisible by micro batch size"
        self.num_micro_batches = self.NMB = batch_size // micro_batch_size
        self.PP = pmap.pipeline_parallelism
        self.VPP = getattr(config, "virtual_pipeline_parallelism", 1)
        self.reuse_buffers_in_1f1b = reuse_buffers_in_1f1b
        self.verbose, self.memory_tracker, self.profiler = verbose, memory_tracker, None

        self.vocab_size = config.vocab_size
        self.hidden_size = config.hidden_size
        self.num_experts = getattr(config, "num_experts", 1)
        self.num_experts_per_tok = getattr(config, "num_experts_per_tok", 1)
        self.num_hidden_layers_per_rank = config.num_hidden_layers // self.PP
        self.num_hidden_layers_per_vpp_rank = self.num_hidden_layers_per_rank // self.VPP
        self.router_aux_loss_coef = getattr(config, "router_aux_loss_coef", 0.0)
        self.router_z_loss_coef = getattr(config, "router_z_loss_coef", 0.0)
        self.use_aux_loss = bool(getattr(config, "output_router_logits", False))
        self.use_local_router_aux_loss = self.use_aux_loss and bool(getattr(config, "use_local_router_aux_loss", False))
        self.use_global_router_aux_loss = self.use_aux_loss and not self.use_local_router_aux_loss

        self.schedule: List[PipeOp] = make_schedule(pp_scheme, pmap.pp_ind, self.PP, self.NMB, self.VPP)
        self.groups, self.pairs = {}, None
        if dist.is_initialized() and self.PP > 1:
            self.pairs = _pair_groups(pmap)
            if self.pairs is None:
                self.groups = _channel_groups(self.VPP > 1)
        self.last_virtual = self.PP * self.VPP - 1
        self._pending: List[Tuple[object, torch.Tensor]] = []
        # slot plan of the activations in flight: bounded by the schedule's peak, checked on every step
        self.buffers = Interleaved1f1bBufferManager(pmap, self.VPP, self.PP, self.NMB, reuse_buffers_in_1f1b=True,
                                                    pp_scheme=pp_scheme)
        if verbose and getattr(pmap, "dp_ind", 0) == 0 and getattr(pmap, "ep_ind", 0) == 0:
            print(f"Rank {pmap.rank}: at most {self.buffers.num_act_buffers} micro-batch activations in flight "
                  f"for {pp_scheme} pp_scheme (PP {self.PP}, VPP {self.VPP}, NMB {self.NMB})", flush=True)

    # ------------------------------------------------------------------ topology
    def _virtual(self, vp: int) -> int:
        return vp * self.PP + self.pmap.pp_ind

    def _fwd_src(self, vp):
        """(rank, group) the input of chunk ``vp`` comes from."""
        me, prev = self.pmap.rank, self.pmap.prev_stage_rank
        if self.pairs is not None:
            return prev, self.pairs[(prev, me, "fwd")]
        if self.pmap.pp_ind > 0:
            return prev, self.groups["fwd"]
        return prev, self.groups["wrap_fwd"]  # first stage, vp > 0: from the last stage

    def _fwd_dst(self, vp):
        me, nxt = self.pmap.rank, self.pmap.next_stage_rank
        if self.pairs is not None:
            return nxt, self.pairs[(me, nxt, "fwd")]
        if self.pmap.pp_ind < self.PP - 1:
            return nxt, self.groups["fwd"]
        return nxt, self.groups["wrap_fwd"]

    def _bwd_src(self, vp):
        me, nxt = self.pmap.rank, self.pmap.next_stage_rank
        if self.pairs is not None:
            return nxt, self.pairs[(me, nxt, "bwd")]
        if self.pmap.pp_ind < self.PP - 1:
            return nxt, self.groups["bwd"]
        return nxt, self.groups["wrap_bwd"]

    def _bwd_dst(self, vp):
        me, prev = self.pmap.rank, self.pmap.prev_stage_rank
        if self.pairs is not None:
            return prev, self.pairs[(prev, me, "bwd")]
        if self.pmap.pp_ind > 0:
            return prev, self.groups["bwd"]
        return prev, self.groups["wrap_bwd"]

    def _isend(self, t, dst_group):
        dst, group = dst_group
        t = t.contiguous()
        works = dist.batch_isend_irecv([dist.P2POp(dist.isend, t, dst, group)])
        self._pending.extend((w, t) for w in works)

    def _recv(self, t, src_group):
        src, group = src_group
        for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, t, src, group)]):
            w.wait()
        return t

    # ------------------------------------------------------------------ model call / router info
    def _chunk_layers(self, vp):
        inner = getattr(self.model, "model", self.model)
        LV = self.num_hidden_layers_per_vpp_rank
        return list(inner.layers[vp * LV:(vp + 1) * LV])

    def _call_model(self, x, vp):
        if self.VPP > 1:
            out = self.model(x, vp_ind=vp)
        else:
            out = self.model(x)
        router_logits = None
        if isinstance(out, dict):
            router_logits = out.get("router_logits")
            out = out["output"]
        elif hasattr(out, "logits") and not isinstance(out, torch.Tensor):
            out = out.logits
        return out, router_logits

    def _router_info(self, vp, router_logits):
        layers = self._chunk_layers(vp)
        logits = [r for r in (router_logits or ()) if r is not None]
        if len(logits) != len(layers):
            # raw-tensor stage contract (virtual pipelining): read the logits off the MoE blocks
            logits = [getattr(l.mlp, "last_router_logits", None) for l in layers]
            if any(r is None for r in logits):
                return None
        idx = [getattr(l.mlp, "last_router_indices", None) for l in layers]
        stats = [getattr(l.mlp, "last_router_stats", None) for l in layers]
        return logits, idx, (stats if all(s is not None for s in stats) else None)

    # ------------------------------------------------------------------ aux-loss pieces
    def _aux_scales(self):
        T = self.micro_batch_size * self.context_size
        L_total = self.config.num_hidden_layers
        a_scale = self.router_aux_loss_coef * self.num_experts / (T * L_total)
        z_scale = self.router_z_loss_coef / (T * L_total)
        return T, L_total, a_scale, z_scale

    def _own_running_stats(self, st: _MicroState):
        """[2E+2] running sums after this stage: previous stages' sums + this stage's."""
        E = self.num_experts
        v = torch.zeros(AL.stats_width(E), dtype=torch.float32, device=self.device)
        if st.prev_stats is not None:
            v += st.prev_stats
        if st.stats is not None:
            v[:2 * E + 1] += st.stats.sum(0)
            if self.use_local_router_aux_loss:
                T, L_total, a_scale, z_scale = self._aux_scales()
                f = st.stats[:, :E] / T
                v[2 * E + 1] += a_scale * (f * st.stats[:, E:2 * E]).sum() + z_scale * st.stats[:, 2 * E].sum()
        return v

    def _make_partial(self, st: _MicroState, f_global: Optional[torch.Tensor]):
        """Differentiable aux loss of this stage's layers (``None`` when there is nothing to do)."""
        if st.logits_list is None:
            return None
        E = self.num_experts
        T, L_total, a_scale, z_scale = self._aux_scales()
        L = len(st.logits_list)
        if self.use_local_router_aux_loss:
            f = st.stats[:, :E] / T
        else:
            f = f_global.reshape(1, E).expand(L, E)
        return AL.aux_partial(st.logits_list, st.idx_list, st.stats, f, a_scale=a_scale, z_scale=z_scale)

    # ------------------------------------------------------------------ one op
    def _forward_op(self, op: PipeOp, states, input_list, labels_list, loss_list, logits_list, output_logits):
        s = self._virtual(op.vp)
        st = states[(op.mb, op.vp)] = _MicroState()
        E = self.num_experts
        with record_pcl_function("1pp--1fwd--1recv"):
            if s == 0:
                x = input_list[op.mb]
            else:
                shape = (self.micro_batch_size, self.context_size, self.hidden_size)
                buf = torch.empty(shape, dtype=self.dtype, device=self.device)
                self._recv(buf, self._fwd_src(op.vp))
                if self.use_aux_loss:
                    st.prev_stats = self._recv(torch.empty(AL.stats_width(E), dtype=torch.float32, device=self.device),
                                               self._fwd_src(op.vp))
                st.inp = buf.requires_grad_(True)
                x = st.inp
        with record_pcl_function("1pp--1fwd--2compute"):
            out, router_logits = self._call_model(x, op.vp)
            if self.use_aux_loss:
                info = self._router_info(op.vp, router_logits)
                if info is not None:
                    st.logits_list, st.idx_list, kstats = info
                    st.stats = AL.router_stats(st.logits_list, st.idx_list, kstats, E, self.num_experts_per_tok)
            if s == self.last_virtual:
                if output_logits:
                    logits_list[op.mb] = out.detach().clone()
                if labels_list is not None:
                    loss = OF.shifted_cross_entropy(out, labels_list[op.mb], inplace_backward=not output_logits)
                    report = loss.detach().clone()
                    if self.use_aux_loss and st.stats is not None:
                        running = self._own_running_stats(st)
                        T, L_total, a_scale, z_scale = self._aux_scales()
                        if self.use_local_router_aux_loss:
                            aux_value = running[2 * E + 1]
                        else:
                            st.f_global = running[:E] / (T * L_total)
                            aux_value = a_scale * (st.f_global * running[E:2 * E]).sum() + z_scale * running[2 * E]
                        partial = self._make_partial(st, st.f_global)
                        loss = loss + partial.to(loss.dtype)
                        report = report + aux_value.to(report.dtype)
                    loss_list[op.mb] = report
                    st.loss_scaled = loss / (self.NMB * self.opt_grad_acc_steps)
                st.out = out
            else:
                st.out = out
        with record_pcl_function("1pp--1fwd--3send"):
            if s != self.last_virtual:
                self._isend(out.detach(), self._fwd_dst(op.vp))
                if self.use_aux_loss:
                    self._isend(self._own_running_stats(st), self._fwd_dst(op.vp))

    def _backward_op(self, op: PipeOp, states, output_grad_list):
        s = self._virtual(op.vp)
        st = states.pop((op.mb, op.vp))
        E = self.num_experts
        with record_pcl_function("1pp--2bwd--1recv"):
            grad = None
            if s != self.last_virtual:
                grad = torch.empty_like(st.out)
                self._recv(grad, self._bwd_src(op.vp))
                if self.use_global_router_aux_loss:
                    st.f_global = self._recv(torch.empty(E, dtype=torch.float32, device=self.device),
                                             self._bwd_src(op.vp))
        with record_pcl_function("1pp--2bwd--2compute"):
            if s == self.last_virtual:
                if st.loss_scaled is not None:
                    st.loss_scaled.backward()
                else:
                    g = output_grad_list[op.mb] if output_grad_list is not None else None
                    st.out.backward(g)
            else:
                tensors, grads = [st.out], [grad]
                if self.use_aux_loss and st.logits_list is not None:
                    partial = self._make_partial(st, st.f_global)
                    tensors.append(partial)
                    grads.append(torch.full_like(partial, 1.0 / (self.NMB * self.opt_grad_acc_steps)))
                torch.autograd.backward(tensors, grads)
        with record_pcl_function("1pp--2bwd--3send"):
            if s != 0:
                self._isend(st.inp.grad, self._bwd_dst(op.vp))
                if self.use_global_router_aux_loss:
                    self._isend(st.f_global, self._bwd_dst(op.vp))

    # ------------------------------------------------------------------ public step
    def step(self, input=None, labels=None, only_forward=False, output_grad=None, output_logits=False, debug=False):
        NMB, MBS = self.NMB, self.micro_batch_size
        first_rank = self.pmap.is_first_stage_rank
        last_rank = self.pmap.is_last_stage_rank
        if first_rank:
            assert input is not None, "Input should be provided for the first stage ranks"
        input_list = list(input.split(MBS, dim=0)) if (first_rank and input is not None) else [None] * NMB
        labels_list = list(labels.split(MBS, dim=0)) if (last_rank and labels is not None) else None
        output_grad_list = list(output_grad.split(MBS, dim=0)) if (last_rank and output_grad is not None) else None
        loss_list: List[Optional[torch.Tensor]] = [None] * NMB
        logits_list: List[Optional[torch.Tensor]] = [None] * NMB
        states: Dict[Tuple[int, int], _MicroState] = {}

        self.buffers.reset()
        for op in self.schedule:
            if op.kind == "F":
                if not only_forward:
                    self.buffers.add_forward_to_flight(self.buffers.flat_index(op.mb, op.vp))
                self._forward_op(op, states, input_list, labels_list, loss_list, logits_list, output_logits)
            elif not only_forward:
                self._backward_op(op, states, output_grad_list)
                self.buffers.drain_forward_from_flight(self.buffers.flat_index(op.mb, op.vp))
        for work, _keep in self._pending:
            work.wait()
        self._pending.clear()
        states.clear()

        loss = None
        if last_rank and labels_list is not None:
            loss = torch.stack([l for l in loss_list if l is not None]).mean()
        logits = torch.cat(logits_list, dim=0) if (output_logits and last_rank and logits_list[0] is not None) else None
        return ParallelTrainerOutput(loss=loss, logits=logits)
