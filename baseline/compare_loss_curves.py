"""Loss-curve parity against the reference implementation, on one GPU or expert parallel over N GPUs.

Runs N training steps of the same model (OLMoE-1B-7B, all 16 layers by default), the same initial weights (every tensor
drawn from its serial name, ``model_io.seeded_serial_tensor``, whatever the expert-parallel layout), the same token
batches and the same optimizer settings through

* this framework (``TrainEngine``: tcgen05 kernels, fused expert-parallel MoE, pgshard AdamW), and
* the reference's classes installed under ``baseline/_ref`` (stock expert loop, its all-gather / reduce-scatter expert
  parallelism, its ``ParamGroupShardedMixedPrecisionAdamW``), driven as in ``baseline/run_reference.py``,

one after the other, and prints the per-step losses (mean over ranks) and their differences.  The data is learnable:
every rank cycles through a fixed set of ``--cycle`` batches at a constant learning rate, so the loss has to fall
and a wrong gradient shows up as a curve that separates from the reference's.

    python baseline/compare_loss_curves.py --steps 32
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29571 \
        baseline/compare_loss_curves.py --steps 32
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
REF = os.path.join(ROOT, "baseline", "_ref")
MODEL = "allenai/OLMoE-1B-7B-0924"
VOCAB = 50304


def batches(opts, rank):
    """``--cycle`` fixed batches per rank, repeated: data a model can learn."""
    import torch
    g = torch.Generator().manual_seed(4321 + rank)
    fixed = [torch.randint(0, VOCAB, (opts.micro_batch, opts.seq_len), generator=g, dtype=torch.int64)
             for _ in range(opts.cycle)]
    return [fixed[s % opts.cycle] for s in range(opts.steps)]


def _dist():
    import torch.distributed as dist
    return dist if dist.is_available() and dist.is_initialized() else None


def _global_mean(loss, dev):
    import torch
    t = torch.tensor([float(loss)], dtype=torch.float64, device=dev)
    d = _dist()
    if d is not None:
        d.all_reduce(t)
        t /= d.get_world_size()
    return float(t.item())


def run_ours(opts, rank, world):
    import torch
    from optimus_lm_b200.engine import EngineArgs, TrainEngine
    args = EngineArgs(model_choice=MODEL, dtype="bf16", batch_size=opts.micro_batch, context_size=opts.seq_len,
                      optimizer="pgshard", warmup_steps=2500, use_fast_moe=True, use_merged_mlp_in_fast_moe=True,
                      expert_parallelism=world, data_parallelism=1, seed=0,
                      config_overrides={"num_hidden_layers": opts.layers, "output_router_logits": True})
    eng = TrainEngine(args)
    losses = []
    for b in batches(opts, rank):
        eng.set_lr(opts.lr)
        losses.append(_global_mean(eng.train_step(b.cuda()).loss, eng.device))
    assert eng.check_device_status() == 0
    del eng
    torch.cuda.empty_cache()
    return losses


def run_reference(opts, rank, world):
    import re
    import torch
    sys.path.insert(0, REF)
    for name in ("synchronize", "set_device", "current_device", "memory_allocated", "memory_reserved",
                 "max_memory_allocated", "empty_cache", "Event", "device_count"):
        if hasattr(torch.cuda, name):
            setattr(torch.xpu, name, getattr(torch.cuda, name))
    from optimus.config_utils import get_modified_config
    from optimus.mapper import ParallelDpPpEpTpMapper
    from optimus.models.olmoe.configuration_olmoe import OlmoeParallelConfig
    from optimus.models.olmoe.modeling_olmoe import OlmoeParallelForCausalLM
    from optimus.optimizers import ParamGroupShardedMixedPrecisionAdamW
    from optimus.utils import no_init_weights
    from optimus_lm_b200 import model_io

    dev = torch.device("cuda", torch.cuda.current_device())
    pmap = ParallelDpPpEpTpMapper(data_parallelism=1, pipeline_parallelism=1, expert_parallelism=world,
                                  tensor_parallelism=1, rank=rank, create_groups=(world > 1))
    config = OlmoeParallelConfig(pipeline_parallelism=1, expert_parallelism=world, tensor_parallelism=1,
                                 virtual_pipeline_parallelism=1)
    config = get_modified_config(MODEL, config)
    config.num_hidden_layers = opts.layers
    config.output_router_logits = True
    config.check_compatibility()
    prev = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with no_init_weights(), torch.device(dev):
            model = OlmoeParallelForCausalLM(config, pmap=pmap, memory_tracker=None)
    finally:
        torch.set_default_dtype(prev)
    e_start = pmap.ep_ind * (config.num_experts // world)
    with torch.no_grad():   # same values as the other arm: a tensor's initial value depends on its serial name only
        for name, p in model.named_parameters():
            serial = re.sub(r"\.experts\.(\d+)\.", lambda m: f".experts.{int(m.group(1)) + e_start}.", name)
            p.copy_(model_io.seeded_serial_tensor(serial, tuple(p.shape), config.initializer_range, 0, device=dev))
        pad = getattr(model.model.embed_tokens, "padding_idx", None)
        if pad is not None:
            model.model.embed_tokens.weight[pad].zero_()
    model = model.to(torch.bfloat16).to(dev)
    opt = ParamGroupShardedMixedPrecisionAdamW(
        model.parameters(), model, lr=opts.lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, warmup_steps=2500,
        dtype=torch.bfloat16, device=dev, num_shards=1, shard_id=0, group=pmap.dp_group,
        opt_disable_delayed_grad_clipping=False, profiler=None, tensor_parallelism=1, tp_ind=0, tp_group=pmap.tp_group,
        expert_parallelism=world, ep_ind=pmap.ep_ind, ep_group=pmap.ep_group, dpep_ind=pmap.dpep_ind,
        dpep_group=pmap.dpep_group, opt_use_chunked_allreduce=False, opt_use_allreduce_for_grad_acc=False,
        opt_use_allreduce_for_param_gather=False, skip_optimizer_step=False)
    opt.pmap, opt.config, opt.dump_weight_gradients = pmap, config, False
    losses = []
    for b in batches(opts, rank):
        for grp in opt.param_groups:
            grp["lr"] = opts.lr
        ids = b.to(dev)
        out = model(ids, labels=ids)
        out.loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(_global_mean(out.loss, dev))
    del model, opt
    torch.cuda.empty_cache()
    return losses


def main():
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--layers", type=int, default=16)
    p.add_argument("--steps", type=int, default=32)
    p.add_argument("--micro-batch", type=int, default=4)
    p.add_argument("--seq-len", type=int, default=4096)
    p.add_argument("--cycle", type=int, default=8, help="number of distinct batches per rank")
    p.add_argument("--lr", type=float, default=1e-3)
    opts = p.parse_args()
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = 0
    if world > 1:
        from optimus_lm_b200.dutils import setup_distributed
        rank, world, _, _ = setup_distributed("nccl", timeout_s=900)
    else:
        torch.cuda.set_device(0)
    if not os.path.isdir(os.path.join(REF, "optimus")):
        ours = run_ours(opts, rank, world)
        if rank == 0:
            print(json.dumps({"ours": ours, "reference": None, "unavailable": "baseline/_ref is missing"}))
        return
    ref = run_reference(opts, rank, world)
    ours = run_ours(opts, rank, world)
    if rank == 0:
        diffs = [abs(a - b) for a, b in zip(ours, ref)]
        for s, (a, b) in enumerate(zip(ours, ref)):
            print(f"step {s:3d}  ours {a:9.5f}  reference {b:9.5f}  diff {a - b:+.5f}")
        print(json.dumps({"layers": opts.layers, "steps": opts.steps, "n_gpus": world, "lr": opts.lr, "cycle": opts.cycle,
                          "max_abs_diff": max(diffs), "mean_abs_diff": sum(diffs) / len(diffs),
                          "first_loss": [ours[0], ref[0]], "last_loss": [ours[-1], ref[-1]],
                          "loss_drop": [ours[0] - ours[-1], ref[0] - ref[-1]]}))
    d = _dist()
    if d is not None:
        d.barrier()
        d.destroy_process_group()


if __name__ == "__main__":
    main()
