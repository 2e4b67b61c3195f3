"""Kernel-time table of one training step.

``python -m optimus_lm_b200.utils.step_profile [--model NAME] [--layers L] [--batch B] [--context S] [--top N]``
builds the training engine on one GPU, runs three warm-up steps on synthetic tokens, records one more step with
``torch.profiler`` and prints every device kernel's summed time, share and launch count, longest first.  The times are
those of a profiled step (a few per cent slower than an unprofiled one); use them as shares.  The role of the reference's
per-region wall-clock profiler (optimus/profilers.py: Profiler.print_summary) for a step that is one stream of kernels.
"""
from __future__ import annotations

import argparse
import collections


def kernel_table(events, top: int = 45):
    """(total microseconds, rows) with rows = (microseconds, launches, kernel name), longest first."""
    import torch

    tot = collections.defaultdict(lambda: [0.0, 0])
    for ev in events:
        if ev.device_type == torch.autograd.DeviceType.CUDA:
            t = ev.device_time_total if hasattr(ev, "device_time_total") else ev.cuda_time_total
            tot[ev.name[:90]][0] += t
            tot[ev.name[:90]][1] += 1
    total = sum(v[0] for v in tot.values())
    rows = sorted(((t, n, name) for name, (t, n) in tot.items()), reverse=True)[:top]
    return total, rows


def main(argv=None) -> None:
    import torch
    from torch.profiler import ProfilerActivity, profile

    from optimus_lm_b200.engine import EngineArgs, TrainEngine

    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="allenai/OLMoE-1B-7B-0924")
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers (0: as configured)")
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--optimizer", default="pgshard")
    ap.add_argument("--top", type=int, default=45)
    a = ap.parse_args(argv)

    overrides = {"output_router_logits": True}
    if a.layers:
        overrides["num_hidden_layers"] = a.layers
    eng = TrainEngine(EngineArgs(model_choice=a.model, dtype="bf16", batch_size=a.batch, context_size=a.context,
                                 optimizer=a.optimizer, use_fast_moe=True, use_merged_mlp_in_fast_moe=True,
                                 config_overrides=overrides))
    g = torch.Generator().manual_seed(0)
    vocab = eng.config.vocab_size
    toks = [torch.randint(0, vocab, (a.batch, a.context), generator=g).cuda() for _ in range(4)]
    for i in range(3):
        eng.train_step(toks[i])
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        eng.train_step(toks[3])
        torch.cuda.synchronize()
    total, rows = kernel_table(prof.events(), a.top)
    print(f"total kernel time {total / 1e3:.1f} ms")
    for t, n, name in rows:
        print(f"{t / 1e3:9.3f} ms {100 * t / total:5.1f}% {n:5d}x  {name}")


if __name__ == "__main__":
    main()
