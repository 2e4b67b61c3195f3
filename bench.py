#!/usr/bin/env python
"""Headline benchmark: OLMoE-1B-7B training tokens/s on N GPUs of one node.

    python bench.py --gpus 1 --steps 8 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 8 --warmup 3

Config (fixed): OLMoE-1B-7B (16 layers, d_model 2048, 16 heads, 64 experts top-8, expert ffn 1024,
merged-MLP layout, vocab 50304), sequence length 4096, micro-batch 4 sequences per GPU, bf16
compute with fp32 master weights and moments, expert parallel over all N GPUs (EP=N) with the
process-group-sharded AdamW; at N=1 the same model runs with EP=1.  Synthetic uniform-random
tokens, N(0, 0.02) random-init weights.  A step is forward + backward + optimizer step.

Rank 0 prints one JSON line.  ``value`` is total tokens/s over all GPUs, timed on the device
with CUDA events around exactly ``--steps`` steps (max over ranks).  ``e2e`` times the same
steps through ``TrainEngine.train_step`` with the per-step host->device copy of the tokens from
pinned memory and a device->host read of the loss inside the timed region.

``--config`` selects one of the further configurations (OLMoE data parallel, OLMo-1B data parallel with the sharded
AdamW, OLMoE pipeline x expert parallel with 1F1B, reduced DeepSeek-V3 expert parallel); their JSON line carries their
own metric name.

``--impl reference`` runs the reference implementation (installed under baseline/_ref) for the
same metric; see baseline/run_reference.py.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

MODEL_CHOICE = "allenai/OLMoE-1B-7B-0924"
SEQ_LEN = 4096
MICRO_BATCH = 4
VOCAB = 50304
METRIC = "OLMoE-1B-7B EP train tokens/s (device-timed, max over ranks)"


def named_config(name: str, n: int):
    """The other training configurations this repository is measured on, selected with ``--config`` (the default,
    ``olmoe_ep``, is the headline).  Returns (engine keyword arguments, micro-batch, sequence length, vocabulary,
    metric name, parallelism tag)."""
    moe = dict(use_fast_moe=True, use_merged_mlp_in_fast_moe=True)
    if name == "olmoe_ep":
        return (dict(model_choice=MODEL_CHOICE, expert_parallelism=n, data_parallelism=1, optimizer="pgshard", **moe),
                MICRO_BATCH, SEQ_LEN, VOCAB, METRIC, f"ep{n}")
    if name == "olmoe_dp":          # the same model, data parallel only (every GPU holds all 64 experts)
        return (dict(model_choice=MODEL_CHOICE, expert_parallelism=1, data_parallelism=n, optimizer="pgshard", **moe),
                MICRO_BATCH, SEQ_LEN, VOCAB, "OLMoE-1B-7B DP train tokens/s (device-timed, max over ranks)", f"dp{n}")
    if name == "olmo1b_dp":         # OLMo-1B dense, ZeRO-1 sharded AdamW, sequence 2048, micro-batch 8
        return (dict(model_choice="allenai/OLMo-1B-hf", data_parallelism=n, optimizer="shard"),
                8, 2048, 50304, "OLMo-1B DP train tokens/s (device-timed, max over ranks)", f"dp{n}")
    if name == "olmoe_pp_ep":       # 1F1B pipeline over N/2 stages (N at 2 GPUs) x EP pairs, 8 micro-batches of 4 sequences
        ep = 2 if n >= 4 else 1
        pp = n // ep
        assert pp >= 2 and 16 % pp == 0, "olmoe_pp_ep needs 2, 4 or 8 GPUs"
        return (dict(model_choice=MODEL_CHOICE, pipeline_parallelism=pp, expert_parallelism=ep, data_parallelism=1,
                     pp_scheme="1f1b", micro_batch_size=MICRO_BATCH, optimizer="pgshard", **moe),
                8 * MICRO_BATCH, SEQ_LEN, VOCAB, "OLMoE-1B-7B PPxEP 1F1B train tokens/s (device-timed, max over ranks)",
                f"pp{pp}xep{ep}")
    if name == "dsv3_reduced_ep":   # 4 layers (1 dense + 3 MoE) of DeepSeek-V3 at full width: 34 G expert parameters
        assert n == 8, "the reduced DeepSeek-V3 holds 34 G expert parameters: it needs the memory of 8 GPUs"
        return (dict(model_choice="deepseek-ai/DeepSeek-V3--L4-DL1", expert_parallelism=n, data_parallelism=1,
                     optimizer="pgshard", init_std=0.006, **moe),
                1, SEQ_LEN, 129280, "reduced DeepSeek-V3 EP train tokens/s (device-timed, max over ranks)", f"ep{n}")
    raise SystemExit(f"unknown --config {name}")


def metric_name(metric, opts):
    """The configuration's metric name - unless debugging flags changed the shape: a run with another sequence length,
    micro-batch or layer count is not that benchmark and must not carry its name."""
    if opts.config == "olmoe_ep" and (opts.seq_len != SEQ_LEN or opts.micro_batch != MICRO_BATCH) or opts.layers:
        return "DEBUG (not the benchmark configuration): " + metric
    return metric


def result_config(opts, kw, tokens_per_step, par_tag):
    """The ``config`` record of the JSON line: what was measured, in the same keys and words for both arms (what differs
    between the implementations goes under ``impl_notes``)."""
    model = "OLMoE-1B-7B" if kw["model_choice"] == MODEL_CHOICE else kw["model_choice"]
    if opts.layers:
        model += f" (reduced to {opts.layers} layers)"
    return {"model": model, "global_batch": tokens_per_step // opts.seq_len, "seq_len": opts.seq_len,
            "parallelism": par_tag, "optimizer": kw["optimizer"] + " AdamW, bf16 parameters with fp32 master and moments",
            "micro_batch_per_gpu": opts.micro_batch,
            "l2": "activations and weights of every step are far larger than the 126 MB L2; no flush"}


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed
    region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def run_ours(opts):
    import torch
    import torch.distributed as dist

    from optimus_lm_b200.dutils import setup_distributed
    from optimus_lm_b200.engine import EngineArgs, TrainEngine
    from optimus_lm_b200.ops import _ext

    n = opts.gpus
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if n > 1 or world > 1:
        assert world == n, f"launch with torchrun --nproc-per-node {n} (WORLD_SIZE={world})"
        rank, world, local_rank, _ = setup_distributed("nccl", timeout_s=900)
    else:
        rank, local_rank = 0, 0
        torch.cuda.set_device(0)
    dev = torch.device("cuda", torch.cuda.current_device())
    proxy = _ext.enable_launch_counting()

    kw, cfg_mb, cfg_seq, vocab, metric, par_tag = named_config(opts.config, n)
    if opts.config != "olmoe_ep":
        opts.micro_batch, opts.seq_len = cfg_mb, cfg_seq
    metric = metric_name(metric, opts)
    overrides = {"output_router_logits": True} if "OLMoE" in kw["model_choice"] else {}
    if opts.layers:
        overrides["num_hidden_layers"] = opts.layers  # debugging only; reported in the config
    args = EngineArgs(dtype="bf16", batch_size=opts.micro_batch, context_size=opts.seq_len, warmup_steps=2500,
                      use_fused_ep_alltoall=not opts.nccl_only, use_fused_optimizer=not opts.nccl_only,
                      config_overrides=overrides, **kw)
    engine = TrainEngine(args)
    tokens_per_step = engine.tokens_per_step()

    # synthetic data: one pinned host batch per step, uniform-random token ids, per-rank seed
    # (ranks of one pipeline or tensor-parallel group read the same batch: the seed is the data-parallel index)
    g = torch.Generator().manual_seed(1234 + (rank if opts.config == "olmoe_ep" else engine.pmap.dpep_ind))
    total = opts.warmup + 2 * opts.steps
    host_batches = [torch.randint(0, vocab, (opts.micro_batch, opts.seq_len), generator=g, dtype=torch.int64).pin_memory()
                    for _ in range(total)]
    dev_batches = [b.to(dev) for b in host_batches[:opts.warmup + opts.steps]]

    def barrier():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    from optimus_lm_b200.engine import get_learning_rate

    def step(batch):
        # the training recipe's schedule: linear warm-up from min_lr over 2500 optimizer steps
        engine.set_lr(get_learning_rate(engine.step_id, 1 << 20, args))
        return engine.train_step(batch)

    for i in range(opts.warmup):
        out = step(dev_batches[i])
    barrier()
    status = engine.check_device_status()

    # ---- device-timed region: exactly K steps, inputs already resident
    sampler = ClockSampler(int(os.environ.get("CUDA_VISIBLE_DEVICES", "0,1,2,3,4,5,6,7").split(",")[local_rank])
                           if os.environ.get("CUDA_VISIBLE_DEVICES") else local_rank)
    if rank == 0:
        sampler.start()
    launches0 = proxy.launches
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(opts.steps):
        out = step(dev_batches[opts.warmup + i])
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    launches = proxy.launches - launches0
    last_loss = out.loss.item() if out.loss is not None else None     # pipeline: only the last stage sees the loss

    # ---- end-to-end region: H2D of the tokens and D2H of the loss every step
    barrier()
    t0 = time.perf_counter()
    for i in range(opts.steps):
        out = step(host_batches[opts.warmup + opts.steps + i])
        e2e_loss = out.loss.item() if out.loss is not None else float(out.grad_norm)   # a device->host read either way
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    status = status or engine.check_device_status()

    t = torch.tensor([dev_ms, e2e_s, float(status)], dtype=torch.float64, device=dev)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_s, status = t[0].item(), t[1].item(), int(t[2].item())
    if status != 0:
        # a kernel reported a timeout or a buffer overflow (e.g. more routed rows than the expert-parallel
        # receive buffers hold): the step did not do all of its work, so there is no number to report
        if rank == 0:
            print(json.dumps({"metric": metric, "error": f"device status word = {status} on some rank; run invalid",
                              "n_gpus": n, "impl": "optimus_lm_b200"}), flush=True)
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
        sys.exit(3)
    if rank == 0:
        value = tokens_per_step * opts.steps / (dev_ms / 1e3)
        e2e_value = tokens_per_step * opts.steps / e2e_s
        h2d = opts.micro_batch * opts.seq_len * 8
        res = {
            "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": n, "steps": opts.steps,
            "warmup": opts.warmup, "ms_per_step": dev_ms / opts.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": result_config(opts, kw, tokens_per_step, par_tag),
            "impl_notes": {"ep_transport": "nccl all-gather/reduce-scatter" if opts.nccl_only
                           else "dispatch / combine inside the grouped GEMM launches over NVLink peer memory",
                           "optimizer_collectives": "nccl" if opts.nccl_only else "fused reduce-scatter + AdamW + all-gather kernel"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_s * 1e3 / opts.steps},
            "gpu_launches": launches, "gpu_launches_by_kernel": dict(sorted(proxy.by_name.items())),
            "loss_last_step": last_loss, "loss_e2e_last_step": e2e_loss, "device_status": status,
            "impl": "optimus_lm_b200",
        }
        print(json.dumps(res), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    ap.add_argument("--seq-len", dest="seq_len", type=int, default=SEQ_LEN)
    ap.add_argument("--micro-batch", dest="micro_batch", type=int, default=MICRO_BATCH)
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers (the result is then not the headline config)")
    ap.add_argument("--config", type=str, default="olmoe_ep",
                    choices=["olmoe_ep", "olmoe_dp", "olmo1b_dp", "olmoe_pp_ep", "dsv3_reduced_ep"],
                    help="olmoe_ep is the headline; the others are the further measured configurations")
    ap.add_argument("--nccl-only", dest="nccl_only", action="store_true",
                    help="use the NCCL all-gather/reduce-scatter EP transport and NCCL optimizer collectives")
    opts = ap.parse_args()
    if opts.impl == "reference":
        from baseline.run_reference import run_reference
        run_reference(opts)
        return
    run_ours(opts)


if __name__ == "__main__":
    main()
