"""Reference arm of the benchmark.

Runs the IntelLabs/Optimus-LM code installed (unmodified) under ``baseline/_ref`` for the same
metric and config as ``bench.py``: OLMoE-1B-7B, sequence 4096, micro-batch 4 per GPU, bf16,
EP = number of GPUs, its process-group-sharded AdamW, synthetic uniform-random tokens and
N(0, 0.02) random-init weights.

What is the reference's and what is the harness's:

* the model (``OlmoeParallelForCausalLM`` with its stock, non-FastMoE expert loop; the FastMoE
  path needs the XPU-only ``pcl_xpu_customops`` extension or XPU Triton kernels), the config
  (``OlmoeParallelConfig`` + ``get_modified_config``), the rank mapper, the autograd collectives
  and the optimizer (``ParamGroupShardedMixedPrecisionAdamW``) are the reference's classes, called
  the way ``dist_train.py`` calls them (dist_train.py:278-285, 365-393, 534-574, 748-923);
* ``dist_train.py`` itself cannot run here: it initialises distributed only through an XPU-only
  function, needs dataset files and (for its caching step) the HuggingFace hub.  The harness
  therefore re-creates its step loop - forward, backward, local gradient norm, loss all-reduce,
  device synchronisations, optimizer step, zero_grad - and aliases ``torch.xpu`` to ``torch.cuda``
  at run time (the reference calls ``torch.xpu.synchronize()`` inside its collectives).  No file
  of the reference is changed.
"""
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
METRIC = "OLMoE-1B-7B EP train tokens/s (device-timed, max over ranks)"
VOCAB = 50304


def _unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run_reference(opts):
    if not os.path.isdir(os.path.join(REF, "optimus")):
        _unavailable("baseline/_ref is missing (the offline install of the reference was not done on this machine)")
        return
    try:
        _run(opts)
    except Exception as exc:  # noqa: BLE001 - the arm must always print one line and exit 0
        import traceback
        traceback.print_exc()
        if int(os.environ.get("RANK", "0")) == 0:
            _unavailable(f"reference run failed: {type(exc).__name__}: {str(exc)[:300]}")


def _run(opts):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REF)
    # the reference addresses its device through torch.xpu
    for name in ("synchronize", "set_device", "current_device", "memory_allocated", "memory_reserved",
                 "max_memory_allocated", "empty_cache", "Event", "device_count"):
        if hasattr(torch.cuda, name):
            setattr(torch.xpu, name, getattr(torch.cuda, name))

    from bench import ClockSampler  # same sampler as the other arm

    n = opts.gpus
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank, local_rank = 0, 0
    if n > 1 or world > 1:
        assert world == n
        rank, local_rank = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    else:
        torch.cuda.set_device(0)
    dev = torch.device("cuda", torch.cuda.current_device())

    from optimus.config_utils import get_modified_config
    from optimus.mapper import ParallelDpPpEpTpMapper
    from optimus.models.olmoe.configuration_olmoe import OlmoeParallelConfig
    from optimus.models.olmoe.modeling_olmoe import OlmoeParallelForCausalLM
    from optimus.optimizers import ParamGroupShardedMixedPrecisionAdamW
    from optimus.utils import get_total_norm, no_init_weights

    torch.manual_seed(0)
    pmap = ParallelDpPpEpTpMapper(data_parallelism=1, pipeline_parallelism=1, expert_parallelism=n,
                                  tensor_parallelism=1, rank=rank, create_groups=(n > 1))
    config = OlmoeParallelConfig(pipeline_parallelism=1, expert_parallelism=n, tensor_parallelism=1,
                                 virtual_pipeline_parallelism=1)
    config = get_modified_config("allenai/OLMoE-1B-7B-0924", config)
    if opts.layers:
        config.num_hidden_layers = opts.layers
    config.check_compatibility()
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with no_init_weights(), torch.device(dev):
            model = OlmoeParallelForCausalLM(config, pmap=pmap, memory_tracker=None)
    finally:
        torch.set_default_dtype(prev)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                p.normal_(0.0, 0.02)
    model = model.to(torch.bfloat16).to(dev)

    optimizer = ParamGroupShardedMixedPrecisionAdamW(
        model.parameters(), model, lr=4e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, warmup_steps=2500,
        dtype=torch.bfloat16, device=dev, num_shards=pmap.data_parallelism, shard_id=pmap.dp_ind, group=pmap.dp_group,
        opt_disable_delayed_grad_clipping=False, profiler=None, tensor_parallelism=1, tp_ind=0, tp_group=pmap.tp_group,
        expert_parallelism=n, ep_ind=pmap.ep_ind, ep_group=pmap.ep_group, dpep_ind=pmap.dpep_ind,
        dpep_group=pmap.dpep_group, opt_use_chunked_allreduce=False, opt_use_allreduce_for_grad_acc=False,
        opt_use_allreduce_for_param_gather=False, skip_optimizer_step=False)
    optimizer.pmap, optimizer.config, optimizer.dump_weight_gradients = pmap, config, False

    def sync_all():
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()

    def step(tokens):
        """One iteration of the reference's training loop (dist_train.py:748-923)."""
        input_ids = tokens.to(dev).long()
        outputs = model(input_ids, labels=input_ids)
        loss = outputs.loss
        loss.backward()
        local_grad_norm = get_total_norm([p.grad for p in model.parameters() if p.grad is not None])
        global_loss = loss.detach().clone()
        if dist.is_initialized():
            dist.all_reduce(global_loss)
            global_loss /= (pmap.data_parallelism * n)
        torch.cuda.synchronize()
        grad_norm = optimizer.step()
        optimizer.zero_grad()
        torch.cuda.synchronize()
        return global_loss, grad_norm, local_grad_norm

    g = torch.Generator().manual_seed(1234 + rank)
    total = opts.warmup + 2 * opts.steps
    host = [torch.randint(0, VOCAB, (opts.micro_batch, opts.seq_len), generator=g, dtype=torch.int64).pin_memory()
            for _ in range(total)]
    devb = [b.to(dev) for b in host[:opts.warmup + opts.steps]]

    for i in range(opts.warmup):
        step(devb[i])
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    sync_all()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(opts.steps):
        out = step(devb[opts.warmup + i])
    ev1.record()
    sync_all()
    dev_ms = ev0.elapsed_time(ev1)
    last_loss = out[0].item()

    sync_all()
    t0 = time.perf_counter()
    for i in range(opts.steps):
        out = step(host[opts.warmup + opts.steps + i])
        e2e_loss = out[0].item()
    sync_all()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([dev_ms, e2e_s], dtype=torch.float64, device=dev)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_s = t[0].item(), t[1].item()
    tokens_per_step = opts.micro_batch * opts.seq_len * n
    if rank == 0:
        res = {
            "impl": "reference", "metric": METRIC, "value": tokens_per_step * opts.steps / (dev_ms / 1e3),
            "unit": "tokens/s", "n_gpus": n, "steps": opts.steps, "warmup": opts.warmup,
            "ms_per_step": dev_ms / opts.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"model": "OLMoE-1B-7B" + (f" (reduced to {opts.layers} layers)" if opts.layers else ""),
                       "global_batch": opts.micro_batch * n, "seq_len": opts.seq_len,
                       "parallelism": f"ep{n}" if n > 1 else "ep1", "optimizer": "pgshard (reference)",
                       "moe_path": "reference stock expert loop (use_fast_moe=False)",
                       "l2": "activations and weights of every step are far larger than the 126 MB L2; no flush"},
            "clocks": clocks,
            "e2e": {"value": tokens_per_step * opts.steps / e2e_s, "unit": "tokens/s",
                    "h2d_bytes_per_step": opts.micro_batch * opts.seq_len * 8, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_s * 1e3 / opts.steps},
            "gpu_launches": 0, "loss_last_step": last_loss, "loss_e2e_last_step": e2e_loss,
        }
        print(json.dumps(res), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
