"""Pipeline schedules as pure functions: (stage, sizes) -> ordered list of ops.

An op is ``PipeOp(kind, mb, vp)`` with ``kind`` "F" or "B", micro-batch ``mb`` and virtual
chunk ``vp``.  The executor (``pipeline.py``) walks the list; the generators know nothing about
tensors or communication, so they are unit-tested exhaustively on the CPU (every op appears
once, backward after forward, bounded number of micro-batches in flight, producer-before-
consumer across stages).

Covers the reference's three schedules: GPipe (all forwards, then all backwards;
optimus/training.py:223-302, optimus/trainer.py:399-574), non-interleaved 1F1B
(training.py:304-469: ``PP-1-stage`` warm-up forwards, steady one-forward-one-backward,
wind-down) and interleaved 1F1B over virtual chunks with micro-batch groups of size PP
(trainer.py:575-863).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass(frozen=True)
class PipeOp:
    kind: str  # "F" | "B"
    mb: int
    vp: int = 0


def gpipe_schedule(pp_ind: int, PP: int, NMB: int, VPP: int = 1) -> List[PipeOp]:
    """All forwards (chunk by chunk), then all backwards in reverse chunk order."""
    ops = [PipeOp("F", mb, v) for v in range(VPP) for mb in range(NMB)]
    ops += [PipeOp("B", mb, v) for v in reversed(range(VPP)) for mb in range(NMB)]
    return ops


def one_f_one_b_schedule(pp_ind: int, PP: int, NMB: int) -> List[PipeOp]:
    warmup = min(PP - 1 - pp_ind, NMB)
    ops = [PipeOp("F", mb) for mb in range(warmup)]
    nb = 0
    for mb in range(warmup, NMB):
        ops.append(PipeOp("F", mb))
        ops.append(PipeOp("B", nb))
        nb += 1
    ops += [PipeOp("B", mb) for mb in range(nb, NMB)]
    return ops


def _virtual_forward(k: int, PP: int, VPP: int):
    """k-th forward slot -> (micro-batch, chunk): groups of PP micro-batches visit the chunks in turn."""
    group, r = divmod(k, PP * VPP)
    vp, lmb = divmod(r, PP)
    return group * PP + lmb, vp


def _virtual_backward(k: int, PP: int, VPP: int):
    mb, vp = _virtual_forward(k, PP, VPP)
    return mb, VPP - 1 - vp


def interleaved_1f1b_schedule(pp_ind: int, PP: int, NMB: int, VPP: int) -> List[PipeOp]:
    """Interleaved 1F1B.  ``NMB`` must be a multiple of ``PP``."""
    assert NMB % PP == 0, "For 1f1b pp_scheme, num_micro_batches must be divisible by pipeline_parallelism"
    if VPP == 1:
        return one_f_one_b_schedule(pp_ind, PP, NMB)
    total = NMB * VPP
    warmup = min((PP - pp_ind - 1) * 2 + (VPP - 1) * PP, total)
    ops: List[PipeOp] = []
    for k in range(warmup):
        mb, vp = _virtual_forward(k, PP, VPP)
        ops.append(PipeOp("F", mb, vp))
    kb = 0
    for k in range(warmup, total):
        mb, vp = _virtual_forward(k, PP, VPP)
        ops.append(PipeOp("F", mb, vp))
        mb, vp = _virtual_backward(kb, PP, VPP)
        ops.append(PipeOp("B", mb, vp))
        kb += 1
    for k in range(kb, total):
        mb, vp = _virtual_backward(k, PP, VPP)
        ops.append(PipeOp("B", mb, vp))
    return ops


def make_schedule(scheme: str, pp_ind: int, PP: int, NMB: int, VPP: int = 1) -> List[PipeOp]:
    if scheme == "gpipe":
        return gpipe_schedule(pp_ind, PP, NMB, VPP)
    if scheme == "1f1b":
        return interleaved_1f1b_schedule(pp_ind, PP, NMB, VPP) if VPP > 1 else one_f_one_b_schedule(pp_ind, PP, NMB)
    raise ValueError(f"unknown pipeline scheme {scheme}")


def max_in_flight(ops: List[PipeOp]) -> int:
    """Largest number of forwards whose backward has not run yet (activation memory bound)."""
    live = peak = 0
    for op in ops:
        live += 1 if op.kind == "F" else -1
        peak = max(peak, live)
    return peak


def simulate(scheme: str, PP: int, NMB: int, VPP: int = 1) -> int:
    """Dependency simulation of all stages with rendezvous-free (buffered) channels: returns the
    number of rounds needed, raises if the schedules dead-lock.  Virtual stage ``s = vp*PP + p``
    needs the forward of ``s-1`` for the same micro-batch, and its backward needs the backward
    of ``s+1``."""
    scheds = [make_schedule(scheme, p, PP, NMB, VPP) for p in range(PP)]
    pos = [0] * PP
    done = set()
    rounds = 0
    last_virtual = PP * VPP - 1
    while any(pos[p] < len(scheds[p]) for p in range(PP)):
        progressed = False
        newly = []
        for p in range(PP):
            if pos[p] >= len(scheds[p]):
                continue
            op = scheds[p][pos[p]]
            s = op.vp * PP + p
            if op.kind == "F":
                ready = s == 0 or ("F", op.mb, s - 1) in done
            else:
                ready = ("F", op.mb, s) in done and (s == last_virtual or ("B", op.mb, s + 1) in done)
            if ready:
                newly.append((op.kind, op.mb, s))
                pos[p] += 1
                progressed = True
        done.update(newly)
        rounds += 1
        if not progressed:
            raise RuntimeError(f"pipeline schedule dead-locks: scheme={scheme} PP={PP} NMB={NMB} VPP={VPP} pos={pos}")
    return rounds


class Interleaved1f1bBufferManager:
    """Slot plan for the activations a pipeline stage holds between a forward and its backward.

    Same constructor and method names as the reference's bookkeeping class (optimus/trainer.py:89-182), built on
    the schedule generators above instead of on fixed formulas: ``num_act_buffers`` is the largest number of
    forwards in flight that this stage's schedule reaches (with ``reuse_buffers_in_1f1b``; ``VPP * NMB`` without),
    a forward takes the lowest free slot and its backward gives the slot back.  The executor keeps its per-micro-batch
    state in these slots and checks the bound on every step; code that sizes memory ahead of time reads
    ``num_act_buffers`` / ``num_ograd_buffers``.  Indices are flat positions in forward order (micro-batch groups
    of ``PP`` visit the chunks in turn), as in the reference.
    """

    def __init__(self, pmap, VPP, PP, NMB, reuse_buffers_in_1f1b=False, pp_scheme="1f1b"):
        if pp_scheme == "1f1b" and VPP > 1:
            assert NMB % PP == 0, "In Interleaved1f1b schedule, the number of micro batches should be a multiple of pipeline parallelism"
        self.pmap, self.VPP, self.PP, self.NMB = pmap, VPP, PP, NMB
        self.reuse_buffers_in_1f1b = reuse_buffers_in_1f1b
        self.pp_scheme = pp_scheme
        self.NMBG, self.NG = PP, max(NMB // PP, 1)
        self.total = VPP * NMB
        ops = make_schedule(pp_scheme, pmap.pp_ind, PP, NMB, VPP)
        self.schedule_peak = max_in_flight(ops)
        self.num_act_buffers = self.schedule_peak if reuse_buffers_in_1f1b else self.total
        self.num_ograd_buffers = 1 if reuse_buffers_in_1f1b else self.total
        self._slot_of = {}
        self._free = list(range(self.num_act_buffers))  # kept sorted: the lowest free slot goes first
        self.peak_used = 0

    # ---- index arithmetic
    def flat_index(self, mb: int, vp: int) -> int:
        """Position of forward (micro-batch, chunk) in forward order; inverse of ``_virtual_forward`` (GPipe: chunk
        by chunk)."""
        if self.pp_scheme != "1f1b" or self.VPP == 1:
            return vp * self.NMB + mb
        group, lmb = divmod(mb, self.PP)
        return group * self.PP * self.VPP + vp * self.PP + lmb

    def _in_range(self, index) -> bool:
        return index is not None and 0 <= index < self.total

    def get_forward_index_from_backward_index(self, bwd_index):
        """The k-th backward undoes the forward of the same micro-batch on the mirrored chunk."""
        if not self._in_range(bwd_index):
            return None
        if self.pp_scheme != "1f1b" or self.VPP == 1:
            vp, mb = divmod(bwd_index, self.NMB)
            return self.flat_index(mb, self.VPP - 1 - vp)
        mb, vp = _virtual_backward(bwd_index, self.PP, self.VPP)
        return self.flat_index(mb, vp)

    # ---- slots
    def add_forward_to_flight(self, index):
        if not self._in_range(index):
            return None
        assert index not in self._slot_of, f"forward {index} is already in flight"
        assert self._free, (f"more than {self.num_act_buffers} forwards in flight on stage {self.pmap.pp_ind}: "
                            f"{sorted(self._slot_of)} + {index}")
        slot = self._free.pop(0)
        self._slot_of[index] = slot
        self.peak_used = max(self.peak_used, len(self._slot_of))
        return slot

    def get_forward_buffer_id(self, index):
        if not self._in_range(index):
            return None
        assert index in self._slot_of, f"Forward index {index} is not in flight. (Forwards in flight {sorted(self._slot_of)})"
        return self._slot_of[index]

    def get_backward_buffer_id(self, index):
        if not self._in_range(index):
            return None
        return 0 if self.reuse_buffers_in_1f1b else index

    def drain_forward_from_flight(self, index):
        """The backward of ``index`` has consumed its activations: the slot is free again."""
        if not self._in_range(index) or index not in self._slot_of:
            return None
        slot = self._slot_of.pop(index)
        import bisect
        bisect.insort(self._free, slot)
        return slot

    def reset(self):
        self._slot_of.clear()
        self._free = list(range(self.num_act_buffers))
