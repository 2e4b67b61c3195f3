"""Reference arm of the benchmark.

Runs the IntelLabs/Optimus-LM code installed (unmodified) under ``baseline/_ref`` for the same
metric and config as ``bench.py``: by default OLMoE-1B-7B, sequence 4096, micro-batch 4 per GPU, bf16,
EP = number of GPUs, its process-group-sharded AdamW, synthetic uniform-random tokens and
N(0, 0.02) random-init weights; ``--config`` selects the further configurations (OLMoE data parallel, OLMo-1B
with ``ShardedMixedPrecisionAdamW``, OLMoE pipeline x expert parallel through the reference's
``ParallelTrainer``, reduced DeepSeek-V3 expert parallel).

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


def _build(opts, kw, n, rank, dev):
    """Model, optimizer and (for pipeline runs) trainer of the reference for one named configuration, built the way
    ``dist_train.py`` builds them (dist_train.py:278-285, 365-450, 534-574, 716-730)."""
    import torch

    from optimus.config_utils import get_modified_config
    from optimus.mapper import ParallelDpPpEpTpMapper
    from optimus.utils import no_init_weights
    import optimus.optimizers as ropt

    pp = kw.get("pipeline_parallelism", 1)
    ep = kw.get("expert_parallelism", 1)
    dp = kw.get("data_parallelism") or max(1, n // (pp * ep))
    model_choice = kw["model_choice"]
    pmap = ParallelDpPpEpTpMapper(data_parallelism=dp, pipeline_parallelism=pp, expert_parallelism=ep,
                                  tensor_parallelism=1, rank=rank, create_groups=(n > 1))
    family = model_choice.split("--")[0]
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        if family == "allenai/OLMoE-1B-7B-0924":
            from optimus.models.olmoe.configuration_olmoe import OlmoeParallelConfig
            from optimus.models.olmoe.modeling_olmoe import OlmoeParallelForCausalLM
            config = OlmoeParallelConfig(pipeline_parallelism=pp, expert_parallelism=ep, tensor_parallelism=1,
                                         virtual_pipeline_parallelism=1)
            config = get_modified_config(model_choice, config)
            if opts.layers:
                config.num_hidden_layers = opts.layers
            config.check_compatibility()
            with no_init_weights(), torch.device(dev):
                model = OlmoeParallelForCausalLM(config, pmap=pmap, memory_tracker=None)
        elif family == "allenai/OLMo-1B-hf":
            from optimus.models.olmo.configuration_olmo import OlmoParallelConfig
            from optimus.models.olmo.modeling_olmo import OlmoParallelForCausalLM
            # the class defaults are OLMo-1B's sizes (the reference copies them from the hub's config, which needs a network)
            config = OlmoParallelConfig(tensor_parallelism=1, pipeline_parallelism=pp, virtual_pipeline_parallelism=1)
            config = get_modified_config(model_choice, config)
            if opts.layers:
                config.num_hidden_layers = opts.layers
            with no_init_weights(), torch.device(dev):
                model = OlmoParallelForCausalLM(config, pmap=pmap)
        elif family == "deepseek-ai/DeepSeek-V3":
            from optimus.models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3ParallelConfig
            from optimus.models.deepseek_v3.modeling_deepseek_v3 import DeepseekV3ParallelForCausalLM
            config = DeepseekV3ParallelConfig(expert_parallelism=ep, pipeline_parallelism=pp, tensor_parallelism=1,
                                              virtual_pipeline_parallelism=1)
            config = get_modified_config(model_choice, config)
            with no_init_weights(), torch.device(dev):
                model = DeepseekV3ParallelForCausalLM(config, pmap=pmap, memory_tracker=None)
        else:
            raise ValueError(f"no reference builder for {model_choice}")
    finally:
        torch.set_default_dtype(prev)
    std = kw.get("init_std") or 0.02
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 1:
                p.fill_(1.0)
            else:
                p.normal_(0.0, std)
    model = model.to(torch.bfloat16).to(dev)

    cls = {"pgshard": ropt.ParamGroupShardedMixedPrecisionAdamW, "shard": ropt.ShardedMixedPrecisionAdamW}[kw["optimizer"]]
    optimizer = cls(
        model.parameters(), model, lr=4e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, warmup_steps=2500,
        dtype=torch.bfloat16, device=dev, num_shards=pmap.data_parallelism, shard_id=pmap.dp_ind, group=pmap.dp_group,
        opt_disable_delayed_grad_clipping=False, profiler=None, tensor_parallelism=1, tp_ind=0, tp_group=pmap.tp_group,
        expert_parallelism=ep, ep_ind=pmap.ep_ind, ep_group=pmap.ep_group, dpep_ind=pmap.dpep_ind,
        dpep_group=pmap.dpep_group, opt_use_chunked_allreduce=False, opt_use_allreduce_for_grad_acc=False,
        opt_use_allreduce_for_param_gather=False, skip_optimizer_step=False)
    optimizer.pmap, optimizer.config, optimizer.dump_weight_gradients = pmap, config, False

    trainer = None
    if pp > 1:
        from optimus.training import ParallelTrainer
        trainer = ParallelTrainer(config, model, pmap, opts.micro_batch, kw.get("micro_batch_size") or opts.micro_batch,
                                  opts.seq_len, 1, torch.bfloat16, dev, kw.get("pp_scheme", "1f1b"), True,
                                  memory_tracker=None)
    return pmap, config, model, optimizer, trainer


def _run(opts):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REF)
    # the reference addresses its device through torch.xpu
    for name in ("synchronize", "set_device", "current_device", "memory_allocated", "memory_reserved",
                 "max_memory_allocated", "empty_cache", "Event", "device_count"):
        if hasattr(torch.cuda, name):
            setattr(torch.xpu, name, getattr(torch.cuda, name))

    from bench import ClockSampler, metric_name, named_config, result_config  # shared with the other arm

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

    from optimus.utils import get_total_norm

    kw, cfg_mb, cfg_seq, vocab, metric, par_tag = named_config(opts.config, n)
    if opts.config != "olmoe_ep":
        opts.micro_batch, opts.seq_len = cfg_mb, cfg_seq
    metric = metric_name(metric, opts)
    torch.manual_seed(0)
    pmap, config, model, optimizer, trainer = _build(opts, kw, n, rank, dev)
    dpep = pmap.data_parallelism * pmap.expert_parallelism

    def sync_all():
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()

    def step(tokens):
        """One iteration of the reference's training loop (dist_train.py:748-923)."""
        input_ids = tokens.to(dev).long()
        if trainer is None:
            outputs = model(input_ids, labels=input_ids)
            loss = outputs.loss
            loss.backward()
        else:
            loss = trainer.step(input_ids, input_ids).loss
        local_grad_norm = get_total_norm([p.grad for p in model.parameters() if p.grad is not None])
        global_loss = torch.zeros(1, dtype=torch.float32, device=dev)
        if pmap.is_last_stage_rank and loss is not None:
            global_loss += loss.detach().float()
        if dist.is_initialized():
            dist.all_reduce(global_loss)
            global_loss /= dpep
        torch.cuda.synchronize()
        grad_norm = optimizer.step()
        optimizer.zero_grad()
        torch.cuda.synchronize()
        return global_loss, grad_norm, local_grad_norm

    # ranks of one pipeline read the same batch: the seed is the data-parallel index (as in the other arm)
    g = torch.Generator().manual_seed(1234 + (rank if opts.config == "olmoe_ep" else pmap.dpep_ind))
    settle = 5   # untimed steps before the warm-up proper: the reference's allocation pattern needs them to settle
    total = settle + opts.warmup + 2 * opts.steps
    host = [torch.randint(0, vocab, (opts.micro_batch, opts.seq_len), generator=g, dtype=torch.int64).pin_memory()
            for _ in range(total)]
    devb = [b.to(dev) for b in host[:settle + opts.warmup + opts.steps]]

    for i in range(settle + opts.warmup):
        step(devb[i])
    sync_all()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    sync_all()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for i in range(opts.steps):
        out = step(devb[settle + opts.warmup + i])
    ev1.record()
    sync_all()
    dev_ms = ev0.elapsed_time(ev1)
    last_loss = out[0].item()

    sync_all()
    t0 = time.perf_counter()
    for i in range(opts.steps):
        out = step(host[settle + opts.warmup + opts.steps + i])
        e2e_loss = out[0].item()
    sync_all()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([dev_ms, e2e_s], dtype=torch.float64, device=dev)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_s = t[0].item(), t[1].item()
    tokens_per_step = opts.micro_batch * opts.seq_len * dpep
    if rank == 0:
        res = {
            "impl": "reference", "metric": metric, "value": tokens_per_step * opts.steps / (dev_ms / 1e3),
            "unit": "tokens/s", "n_gpus": n, "steps": opts.steps, "warmup": opts.warmup, "warmup_extra": settle,
            "ms_per_step": dev_ms / opts.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": result_config(opts, kw, tokens_per_step, par_tag),
            "impl_notes": {"optimizer": f"{kw['optimizer']} (reference class)",
                           "moe_path": "reference stock expert loop (use_fast_moe=False: its FastMoE path needs XPU-only code)",
                           "trainer": "optimus.training.ParallelTrainer" if trainer is not None else "model(input_ids, labels)"},
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
