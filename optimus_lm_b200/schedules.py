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
