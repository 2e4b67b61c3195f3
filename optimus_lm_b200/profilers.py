"""Hierarchical region profiler with device timing.

API of the reference's profiler (optimus/profilers.py:12-503): ``PclProfiler`` owning named
``PclTimer`` objects, the ``record_pcl_function("a--b--c")`` context manager that times the
hierarchy ``a``, ``a--b``, ``a--b--c`` and is a no-op while ``optimus_lm_b200.globals.profiler``
is ``None``, per-module forward/backward hooks, a per-step table, an all-ranks table and a
Chrome trace export.

Device time comes from CUDA events recorded on the current stream (the reference enqueues
SYCL profiling tags through a native shim); the native ``stamp_globaltimer`` kernel supplies
absolute ``%globaltimer`` stamps so that device lanes of different ranks line up in the trace.
On CPU ranks (gloo tests) ``time.perf_counter_ns`` is used instead.
"""
from __future__ import annotations

import json
import time
from collections import OrderedDict, defaultdict
from contextlib import contextmanager

import torch
import torch.distributed as dist

from . import globals as _globals


class _Mark:
    """One point in the stream: a CUDA event (or a host clock reading) plus the CPU time."""

    __slots__ = ("event", "cpu_ns", "dev_ns")

    def __init__(self, use_cuda: bool):
        self.cpu_ns = time.perf_counter_ns()
        self.dev_ns = None
        if use_cuda:
            self.event = torch.cuda.Event(enable_timing=True)
            self.event.record()
        else:
            self.event = None


class NamedEvent:
    def __init__(self, name, mark, key="", name_key=""):
        self.name, self.mark, self.key, self.name_key = name, mark, key, name_key

    def get_cpu_mark_time(self):
        return self.mark.cpu_ns


class PclTimer:
    def __init__(self, name, tag=None, exclude_from_trace=False, add_name_key_to_trace_event=False):
        self.name = name
        self.tag = tag
        self.exclude_from_trace = exclude_from_trace
        self.add_name_key_to_trace_event = add_name_key_to_trace_event
        self.named_events = []  # alternating start / stop

    def start(self, use_cuda, key="", name_key=""):
        self.named_events.append(NamedEvent(self.name, _Mark(use_cuda), key, name_key))

    def stop(self, use_cuda):
        self.named_events.append(NamedEvent(self.name, _Mark(use_cuda)))

    def reset(self):
        self.named_events = []


@contextmanager
def record_pcl_function(full_name, tag=None, exclude_from_trace=False, key="", ignore=False):
    prof = _globals.profiler
    if prof is None or ignore:
        yield
        return
    parts = full_name.split("--")
    names = ["--".join(parts[:i + 1]) for i in range(len(parts))]
    for n in names:
        if n not in prof.timers:
            prof.register_timer(n, tag=tag, exclude_from_trace=exclude_from_trace)
        prof.start(n, key=key)
    try:
        yield
    finally:
        for n in reversed(names):
            prof.stop(n)


# The reference also exposes a cheaper variant that only times the leaf name.
@contextmanager
def record_pcl_fast_function(full_name, tag=None, exclude_from_trace=False, key=""):
    prof = _globals.profiler
    if prof is None:
        yield
        return
    if full_name not in prof.timers:
        prof.register_timer(full_name, tag=tag, exclude_from_trace=exclude_from_trace)
    prof.start(full_name, key=key)
    try:
        yield
    finally:
        prof.stop(full_name)


class PclProfiler:
    def __init__(self, process="GPU", rank=0, world_size=1):
        self.process = process
        self.rank = rank
        self.world_size = world_size
        self.timers = OrderedDict()
        self.use_cuda = torch.cuda.is_available()
        self._base = _Mark(self.use_cuda)

    def register_timer(self, name, tag=None, exclude_from_trace=False, add_name_key_to_trace_event=False):
        self.timers[name] = PclTimer(name, tag, exclude_from_trace, add_name_key_to_trace_event)

    def start(self, name, key="", name_key=""):
        if name not in self.timers:
            self.register_timer(name)
        self.timers[name].start(self.use_cuda, key, name_key)

    def stop(self, name):
        self.timers[name].stop(self.use_cuda)

    def set_base_time(self, event=None):
        self._base = _Mark(self.use_cuda)

    def setup_profiler_for_pytorch_model(self, model, only_leaves=False, module_types=None, prefix="module"):
        """Register forward/backward hooks that time every module of the given classes
        (reference :139-210)."""
        def want(mod):
            if only_leaves and len(list(mod.children())) > 0:
                return False
            return module_types is None or isinstance(mod, tuple(module_types))

        for _, mod in model.named_modules():
            if not want(mod):
                continue
            cname = type(mod).__name__
            fname, bname = f"{prefix}--{cname}--fwd", f"{prefix}--{cname}--bwd"

            mod.register_forward_pre_hook(lambda m, a, n=fname: self.start(n))
            mod.register_forward_hook(lambda m, a, o, n=fname: self.stop(n))
            mod.register_full_backward_pre_hook(lambda m, g, n=bname: self.start(n))
            mod.register_full_backward_hook(lambda m, gi, go, n=bname: self.stop(n))

    # ------------------------------------------------------------------ resolution
    def process_events(self):
        """Resolve device times (ns since the profiler's base mark) of all recorded marks."""
        if self.use_cuda:
            torch.cuda.synchronize()
        for timer in self.timers.values():
            for ne in timer.named_events:
                m = ne.mark
                if m.dev_ns is not None:
                    continue
                if m.event is not None:
                    m.dev_ns = int(self._base.event.elapsed_time(m.event) * 1e6)
                else:
                    m.dev_ns = m.cpu_ns - self._base.cpu_ns

    def reset(self):
        for t in self.timers.values():
            t.reset()
        self._base = _Mark(self.use_cuda)

    def _durations(self, timer, split_by_key=False):
        out = defaultdict(list)
        ev = timer.named_events
        for i in range(len(ev) // 2):
            s, e = ev[2 * i], ev[2 * i + 1]
            out[timer.name + (s.key if split_by_key else "")].append(e.mark.dev_ns - s.mark.dev_ns)
        return out

    def get_cumulative_time(self, name, start_id=0, end_id=-1):
        self.process_events()
        d = self._durations(self.timers[name])[name]
        end_id = len(d) if end_id == -1 else end_id
        return sum(d[start_id:end_id])

    def _table(self, split_by_key=False):
        self.process_events()
        table = OrderedDict()
        for timer in self.timers.values():
            for key, vals in self._durations(timer, split_by_key).items():
                if vals:
                    table[key] = [sum(vals), min(vals), max(vals), sum(vals) / len(vals), len(vals)]
        return table

    @staticmethod
    def _format(table, sort_by_name):
        bar = "-" * 116 + "\n"
        s = bar + f"{'Name':60s}, {'Time(ms) (perc %)':>21s}, {'Minimum':>10s}, {'Maximum':>10s}, {'Average':>10s}, {'#calls'}\n" + bar
        if not table:
            return s + bar
        names = sorted(table) if sort_by_name else sorted(table, key=lambda k: table[k][0], reverse=True)
        top = max(v[0] for v in table.values()) or 1
        for n in names:
            c, mn, mx, av, k = table[n]
            s += f"{n:60s}, {c * 1e-6:10.3f} ({c / top * 100:6.2f} %), {mn * 1e-6:10.3f}, {mx * 1e-6:10.3f}, {av * 1e-6:10.3f}, {k:5d}\n"
        return s + bar

    def get_timing_table_string(self, sort_by_name=False, split_by_key=False):
        return self._format(self._table(split_by_key), sort_by_name)

    def get_all_ranks_timing_table_string(self, group=None, sort_by_name=False):
        """Min / max / mean of each region's cumulative time over the ranks of ``group``."""
        table = self._table()
        if not (dist.is_available() and dist.is_initialized()):
            return self._format(table, sort_by_name)
        gathered = [None] * dist.get_world_size(group)
        dist.all_gather_object(gathered, {k: v[0] for k, v in table.items()}, group=group)
        merged = OrderedDict()
        for k in table:
            vals = [g[k] for g in gathered if k in g]
            merged[k] = [sum(vals) / len(vals), min(vals), max(vals), sum(vals) / len(vals), len(vals)]
        return self._format(merged, sort_by_name)

    def print_timing_table(self, sort_by_name=False):
        print(self.get_timing_table_string(sort_by_name=sort_by_name), flush=True)

    def print_all_ranks_timing_table(self, sort_by_name=False):
        s = self.get_all_ranks_timing_table_string(sort_by_name=sort_by_name)
        if self.rank == 0:
            print(s, flush=True)

    def export_chrome_trace(self, chrome_trace_path):
        """Chrome trace with a device lane and a CPU-submit lane per rank (reference :426-503)."""
        self.process_events()
        events = []
        for timer in self.timers.values():
            if timer.exclude_from_trace:
                continue
            ev = timer.named_events
            for i in range(len(ev) // 2):
                s, e = ev[2 * i], ev[2 * i + 1]
                label = timer.name + (f"[{s.name_key}]" if timer.add_name_key_to_trace_event and s.name_key else "")
                events.append({"name": label, "ph": "X", "pid": f"{self.process} rank {self.rank}", "tid": "device",
                               "ts": s.mark.dev_ns / 1e3, "dur": (e.mark.dev_ns - s.mark.dev_ns) / 1e3})
                events.append({"name": label, "ph": "X", "pid": f"{self.process} rank {self.rank}", "tid": "cpu-submit",
                               "ts": (s.mark.cpu_ns - self._base.cpu_ns) / 1e3,
                               "dur": (e.mark.cpu_ns - s.mark.cpu_ns) / 1e3})
        with open(chrome_trace_path, "w") as fh:
            json.dump({"traceEvents": events, "displayTimeUnit": "ms"}, fh)


def device_timestamp_ns() -> int:
    """Absolute ``%globaltimer`` value at the current point of the current CUDA stream (blocks
    until the stamp kernel has run).  Uses the native extension."""
    from .ops._ext import extension
    slot = torch.zeros(1, dtype=torch.int64, device="cuda")
    extension().stamp_globaltimer(slot)
    return int(slot.item())
