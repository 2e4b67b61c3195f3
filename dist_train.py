#!/usr/bin/env python
"""Training driver.

Command line of the reference's ``dist_train.py`` (every flag of dist_train.py:86-191 with the
same name and default; ``--dist_backend`` additionally accepts ``nccl`` and ``gloo``), the same
stdout step line (parsed by ``compare_losses.py``), the same checkpoint layout and resume rules.
Launch with ``torchrun`` (or ``mpiexec``; the PALS/PMI environment names are understood):

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 dist_train.py \
        --model_choice allenai/OLMoE-1B-7B-0924 --expert_parallelism 8 --opt_use_pgsharded_optimizer \
        --use_fast_moe --use_merged_mlp_in_fast_moe --use_om_cached_model --batch_size 4 --context_size 4096

Differences by design: the step loop never synchronises the host with the device except to
print a logged step; weights come from OM-cached shards, an init directory, or - with no files at
all - from the layout-independent seeded initialiser (``--synthetic_init``); ``--synthetic_data``
replaces the dataset directory by uniform-random tokens.
"""
import argparse
import math
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from optimus_lm_b200 import checkpoint as ckpt  # noqa: E402
from optimus_lm_b200 import config_utils  # noqa: E402
from optimus_lm_b200 import globals as olb_globals  # noqa: E402
from optimus_lm_b200.datasets import (PclDataPrallelDataset, PclShardedDataParallelDataset,  # noqa: E402
                                      SyntheticTokenDataset)
from optimus_lm_b200.dutils import setup_distributed  # noqa: E402
from optimus_lm_b200.engine import EngineArgs, TrainEngine, build_model, get_learning_rate, init_weights  # noqa: E402
from optimus_lm_b200.mapper import ParallelDpPpEpTpMapper  # noqa: E402
from optimus_lm_b200.memory_profiler import MemoryTracker  # noqa: E402
from optimus_lm_b200.ops import functional as OF  # noqa: E402
from optimus_lm_b200.profilers import PclProfiler, record_pcl_function  # noqa: E402


def build_parser():
    p = argparse.ArgumentParser()
    # Model
    p.add_argument("--model_choice", type=str, default="allenai/OLMo-1B-hf", help="Hugging face model name")
    p.add_argument("--dtype", type=str, default="bf16", help="Data type to use for training")
    p.add_argument("--use_activation_checkpointing", action="store_true")
    p.add_argument("--activation_checkpointing_level", type=int, default=0,
                   help="Activation checkpointing level in a decoder block (0->None, 1->MoE 2->Attention, 4->Norms)")
    p.add_argument("--use_fast_moe", action="store_true", help="Use custom ops in the model")
    p.add_argument("--use_merged_mlp_in_fast_moe", action="store_true", help="Use merged mlp in fast moe")
    p.add_argument("--use_triton_path_for_gemm_in_fast_moe", action="store_true",
                   help="Accepted for compatibility; GEMMs always run on the tcgen05 kernels")
    p.add_argument("--use_triton_path_for_nongemm_in_fast_moe", action="store_true",
                   help="Accepted for compatibility; non-GEMM MoE ops always run on the CUDA kernels")
    # MoE specific
    p.add_argument("--force_uniform_routing", action="store_true", help="Force uniform routing for MoE layers")
    p.add_argument("--use_local_router_aux_loss", action="store_true", help="Use layer level router aux loss")
    # Initialization
    p.add_argument("--use_om_cached_model", action="store_true", help="Use cached model generated from optimus scripts")
    p.add_argument("--init_model_dir", type=str, default=None)
    p.add_argument("--use_broadcast_for_model_init", action="store_true")
    p.add_argument("--use_allreduce_in_broadcast_model_init", action="store_true")
    # Parallelism
    p.add_argument("--dist_backend", type=str, default="xccl", help="nccl / gloo (xccl, ccl, mpi select the native one)")
    p.add_argument("--use_hf_model", action="store_true", help="Use Hugging Face model")
    p.add_argument("--data_parallelism", type=int, default=None)
    p.add_argument("--pipeline_parallelism", type=int, default=1)
    p.add_argument("--virtual_pipeline_parallelism", type=int, default=1)
    p.add_argument("--expert_parallelism", type=int, default=1)
    p.add_argument("--tensor_parallelism", type=int, default=1)
    p.add_argument("--use_sequence_parallelism_in_tp", action="store_true", help="Parsed and unused, as in the reference")
    p.add_argument("--pp_scheme", type=str, default="1f1b", choices=["gpipe", "1f1b"])
    p.add_argument("--use_pp_first", action="store_true")
    p.add_argument("--reuse_buffers_in_1f1b", action="store_true")
    # Data
    p.add_argument("--dataset_dir", type=str, default="datasets/HuggingFaceFW_fineweb-edu/preprocessed/olmo/")
    p.add_argument("--num_data_files", type=int, default=-1)
    p.add_argument("--use_sharded_dataset", action="store_true")
    # Input
    p.add_argument("--batch_size", type=int, default=1)
    p.add_argument("--micro_batch_size", type=int, default=None)
    p.add_argument("--context_size", type=int, default=4096)
    # Optimizer
    p.add_argument("--warmup_steps", type=int, default=2500)
    p.add_argument("--lr", type=float, default=4e-4)
    p.add_argument("--min_lr", type=float, default=4e-5)
    p.add_argument("--weight_decay", type=float, default=0.1)
    p.add_argument("--beta1", type=float, default=0.9)
    p.add_argument("--beta2", type=float, default=0.95)
    p.add_argument("--eps", type=float, default=1e-8)
    p.add_argument("--lr_schedule", type=str, default="cosine", choices=["cosine", "linear", "constant"])
    p.add_argument("--lr_train_steps", type=int, default=None)
    p.add_argument("--opt_use_pt_optimizer", action="store_true", help="torch.optim.AdamW on DDP")
    p.add_argument("--opt_use_sharded_optimizer", action="store_true")
    p.add_argument("--opt_use_pgsharded_optimizer", action="store_true")
    p.add_argument("--opt_use_subsharded_optimizer", action="store_true")
    p.add_argument("--opt_use_pgsubsharded_optimizer", action="store_true")
    p.add_argument("--opt_use_fp32_for_grad_acc", action="store_true")
    p.add_argument("--opt_use_allreduce_for_grad_acc", action="store_true")
    p.add_argument("--opt_use_allreduce_for_param_gather", action="store_true")
    p.add_argument("--opt_use_chunked_allreduce", action="store_true")
    p.add_argument("--opt_disable_delayed_grad_clipping", action="store_true")
    p.add_argument("--opt_use_one_step_grad_clipping", action="store_true")
    p.add_argument("--opt_grad_acc_steps", type=int, default=1)
    # Profiling
    p.add_argument("--logging_steps", type=int, default=1)
    p.add_argument("--profile", action="store_true")
    p.add_argument("--profile_modules", action="store_true")
    p.add_argument("--verbose", action="store_true")
    # Checkpointing
    p.add_argument("--exp_dir", type=str, default="experiment")
    p.add_argument("--enable_checkpointing", action="store_true")
    p.add_argument("--disable_optimizer_state_checkpointing", action="store_true")
    p.add_argument("--disable_cold_checkpointing", action="store_true")
    p.add_argument("--dp_staggered_checkpointing", action="store_true")
    p.add_argument("--checkpoint_steps", type=int, default=1000)
    # Caching
    p.add_argument("--cached_models_dir", type=str, default="cached_models")
    p.add_argument("--om_cached_models_dir", type=str, default="parallel_models")
    p.add_argument("--disable_model_caching", action="store_true")
    # Debug
    p.add_argument("--log_memory_usage", action="store_true")
    p.add_argument("--exit_steps", type=int, default=-1)
    p.add_argument("--enable_bad_grad_check", action="store_true")
    p.add_argument("--skip_optimizer_step", action="store_true")
    p.add_argument("--skip_optimizer_step_weight_update", action="store_true")
    p.add_argument("--skip_backward_pass", action="store_true")
    p.add_argument("--dump_weight_gradients", action="store_true")
    p.add_argument("--log_all_ranks", action="store_true")
    p.add_argument("--enable_pp_debug", action="store_true")
    p.add_argument("--use_latest_trainer", action="store_true", help="Trainer with virtual pipeline support")
    # Additions of this implementation
    p.add_argument("--synthetic_data", action="store_true", help="Uniform-random tokens instead of --dataset_dir")
    p.add_argument("--synthetic_init", action="store_true", help="Seeded random initialisation instead of weight files")
    p.add_argument("--train_steps", type=int, default=None, help="Override the number of steps (default: one epoch)")
    p.add_argument("--disable_fused_ep_alltoall", action="store_true", help="Use the NCCL all-gather/reduce-scatter EP transport")
    p.add_argument("--disable_fused_optimizer", action="store_true", help="Use NCCL collectives in the optimizer step")
    p.add_argument("--router_z_loss_coef", type=float, default=0.0)
    p.add_argument("--moe_capacity_factor", type=float, default=None,
                   help="0 (default): expert-parallel activation buffers sized from each layer's routed counts, nothing "
                        "is ever dropped; > 0: fixed buffers of that multiple of the balanced share (no host read per "
                        "layer), a rank that receives more stops the run with ST_OVERFLOW")
    p.add_argument("--enable_tb_logging", action="store_true",
                   help="Write loss / grad norm / lr / throughput scalars to <exp_dir>/scalars.jsonl and, when "
                        "tensorboard is installed, to <exp_dir>/tb")
    p.add_argument("--dist_timeout_s", type=float, default=1800.0)
    p.add_argument("--chrome_trace", type=str, default=None, help="Write a Chrome trace of the profiled regions here")
    return p


def optimizer_key(args) -> str:
    flags = {"shard": args.opt_use_sharded_optimizer, "pgshard": args.opt_use_pgsharded_optimizer,
             "subshard": args.opt_use_subsharded_optimizer, "pgsubshard": args.opt_use_pgsubsharded_optimizer}
    chosen = [k for k, v in flags.items() if v]
    assert len(chosen) <= 1, "choose at most one optimizer"
    if args.opt_use_pt_optimizer:
        assert not chosen, "--opt_use_pt_optimizer excludes the flat-buffer optimizers"
        return "pt"
    return chosen[0] if chosen else "unsharded"


def load_initial_weights(args, model, pmap, rank):
    """OM-cached shard / init directory / seeded random init (reference dist_train.py:316-497)."""
    merged = args.use_fast_moe and args.use_merged_mlp_in_fast_moe
    key = config_utils.cached_model_key(args.model_choice, args.pipeline_parallelism, args.expert_parallelism,
                                        args.tensor_parallelism, args.virtual_pipeline_parallelism, merged)
    path = None
    if args.init_model_dir is not None:
        name = f"model_checkpoint_shard-{pmap.mp_ind}.pth" if pmap.is_model_parallel else "model_checkpoint.pth"
        path = os.path.join(args.init_model_dir, name)
        assert os.path.exists(path), f"Initialization model not found at {path}"
    elif args.use_om_cached_model:
        path = os.path.join(args.om_cached_models_dir, key, f"model_{pmap.mp_ind}.pth")
        assert os.path.exists(path), f"OM cached model not found at {path}"
    elif not args.synthetic_init:
        cand = os.path.join(args.cached_models_dir, key, f"model_{pmap.mp_ind}.pth")
        if os.path.exists(cand):
            path = cand
    if path is None:
        if rank == 0:
            print("No weight files given: seeded random initialisation", flush=True)
        init_weights(model, getattr(model.config, "initializer_range", 0.02), seed=0)
        return
    reader = (not args.use_broadcast_for_model_init) or pmap.dp_ind == 0
    if reader:
        if rank == 0:
            print(f"Loading the model from {path}", flush=True)
        sd = torch.load(path, map_location="cpu", weights_only=True)
        sd = sd.get("state_dict", sd) if isinstance(sd, dict) and "state_dict" in sd else sd
        model.load_state_dict(sd)
    elif args.use_allreduce_in_broadcast_model_init:
        with torch.no_grad():
            for p in model.parameters():
                p.zero_()
    if args.use_broadcast_for_model_init and dist.is_initialized() and pmap.data_parallelism > 1:
        model.to(torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu")
        for p in model.parameters():
            if args.use_allreduce_in_broadcast_model_init:
                dist.all_reduce(p.data, group=pmap.dp_group)
            else:
                dist.broadcast(p.data, src=pmap.mp_rank, group=pmap.dp_group)


def local_grad_norm(engine) -> torch.Tensor:
    acc = torch.zeros(1, dtype=torch.float32, device=engine.device)
    if hasattr(engine.optimizer, "_finish_direct_grads"):
        engine.optimizer._finish_direct_grads()  # buffers no GEMM has written in this step yet count as zero
    for fam in engine.optimizer.families:
        OF.sum_of_squares(fam.flat_grad, 1.0, out=acc, accumulate=True)
    return acc.sqrt().reshape(())


class ScalarLog:
    """Per-step scalars of the logging rank: one JSON object per line in ``scalars.jsonl`` and, when the
    ``tensorboard`` package is importable, the same values under ``<exp_dir>/tb``."""

    def __init__(self, exp_dir):
        os.makedirs(exp_dir, exist_ok=True)
        self.fh = open(os.path.join(exp_dir, "scalars.jsonl"), "a")
        try:
            from torch.utils.tensorboard import SummaryWriter
            self.tb = SummaryWriter(os.path.join(exp_dir, "tb"))
        except Exception:
            self.tb = None

    def write(self, step, scalars):
        import json
        self.fh.write(json.dumps({"step": int(step), **{k: float(v) for k, v in scalars.items()}}) + "\n")
        self.fh.flush()
        if self.tb is not None:
            for k, v in scalars.items():
                self.tb.add_scalar(k, float(v), int(step))


DEVICE_STATUS_NAMES = {1: "ST_TIMEOUT_FULL (GEMM consumer waited for an operand stage)",
                       2: "ST_TIMEOUT_EMPTY (GEMM producer waited for a free stage)",
                       3: "ST_TIMEOUT_ACC_FULL (epilogue waited for an accumulator)",
                       4: "ST_TIMEOUT_ACC_EMPTY (tensor-core warp waited for a drained accumulator)",
                       5: "ST_TIMEOUT_PEER (a wait on another GPU's flag ran out: a peer is late or gone)",
                       6: "ST_OVERFLOW (an expert-parallel receive buffer limited by moe_capacity_factor was too small; "
                          "moe_capacity_factor 0 sizes the buffers from the routed counts and cannot overflow)",
                       7: "ST_BAD_ARG"}
EXIT_DEVICE_STATUS = 3


def device_status_failed(engine, rank, pmap, device) -> bool:
    """Read (and clear) this rank's device status word and agree on it over all ranks.  True when any rank's kernels
    reported a timeout or an overflow since the last check: the steps since then did not do all of their work, so the
    caller stops without writing a checkpoint."""
    mine = engine.check_device_status()
    worst = torch.tensor([float(mine)], device=device)
    if dist.is_initialized():
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    if worst.item() == 0:
        return False
    if mine:
        print(f"Device status word {mine} = {DEVICE_STATUS_NAMES.get(mine, 'unknown code')} on rank {rank:4d} "
              f"(dp_ind {pmap.dp_ind}, pp_ind {pmap.pp_ind}, ep_ind {pmap.ep_ind}, tp_ind {pmap.tp_ind}); "
              "stopping, no checkpoint is written", flush=True)
    elif rank == 0:
        print(f"Device status word {int(worst.item())} reported by another rank; stopping", flush=True)
    return True


def report_soft_failures(flags, pmap, rank, world_size):
    """Append the nodes of the flagged ranks to launch_info/<job>/failed_soft_nodes.txt."""
    if rank != 0:
        return
    job_id = os.getenv("PBS_JOBID", os.getenv("SLURM_JOB_ID", "0")).split(".")[0]
    d = os.path.join(os.getenv("OPTIMUS_LAUNCH_INFO_DIR", "launch_info"), job_id)
    os.makedirs(d, exist_ok=True)
    nodes = []
    for r in range(world_size):
        if flags[r] > 0:
            node = pmap.rank_to_node_list[r] if r < len(pmap.rank_to_node_list) else f"rank{r}"
            if node not in nodes:
                nodes.append(node)
    with open(os.path.join(d, "failed_soft_nodes.txt"), "a") as fh:
        for n in nodes:
            fh.write(f"{n}\n")


def main(argv=None):
    torch.manual_seed(0)
    import numpy as np
    np.random.seed(42)
    args = build_parser().parse_args(argv)
    assert args.dtype in ["bf16", "fp32"], "Invalid data type"
    if args.micro_batch_size is None:
        args.micro_batch_size = args.batch_size
    if args.pipeline_parallelism > 1 or args.expert_parallelism > 1 or args.tensor_parallelism > 1:
        assert not args.use_hf_model, "Huggingface model does not support parallelism"

    launched = int(os.environ.get("WORLD_SIZE", os.environ.get("PMI_SIZE", "1"))) > 1
    rank, world_size, local_rank = 0, 1, 0
    if launched:
        rank, world_size, local_rank, _ = setup_distributed(args.dist_backend, timeout_s=args.dist_timeout_s)
    elif torch.cuda.is_available():
        torch.cuda.set_device(0)
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    if rank == 0:
        print(f"PMI_SIZE = {world_size}", flush=True)
        print(args, flush=True)

    mp = args.pipeline_parallelism * args.expert_parallelism * args.tensor_parallelism
    dp = args.data_parallelism if args.data_parallelism is not None else world_size // mp
    assert dp * mp == world_size, f"DP {dp} x PP*EP*TP {mp} must equal the world size {world_size}"
    pmap = ParallelDpPpEpTpMapper(dp, args.pipeline_parallelism, args.expert_parallelism, args.tensor_parallelism,
                                  rank=rank, create_groups=launched, use_pp_first=args.use_pp_first)
    if args.verbose:
        print(pmap, flush=True)
    memory_tracker = MemoryTracker(pmap) if args.log_memory_usage else None
    profiler = None
    if args.profile:
        profiler = PclProfiler(process="GPU" if device.type == "cuda" else "CPU", rank=rank, world_size=world_size)
        olb_globals.profiler = profiler

    # ------------------------------------------------------------------ model + optimizer
    dtype = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    overrides = {"router_z_loss_coef": args.router_z_loss_coef} if args.router_z_loss_coef else {}
    if args.moe_capacity_factor is not None:
        overrides["moe_capacity_factor"] = args.moe_capacity_factor
    if args.use_hf_model:
        from optimus_lm_b200.engine import build_hf_model
        config, model = build_hf_model(args.model_choice, dtype=dtype, device=device, config_overrides=overrides)
    else:
        config, model = build_model(
        args.model_choice, pmap, dtype=dtype, device=device, memory_tracker=memory_tracker, config_overrides=overrides,
        pipeline_parallelism=args.pipeline_parallelism, expert_parallelism=args.expert_parallelism,
        tensor_parallelism=args.tensor_parallelism, virtual_pipeline_parallelism=args.virtual_pipeline_parallelism,
        use_local_router_aux_loss=args.use_local_router_aux_loss,
        use_activation_checkpointing=args.use_activation_checkpointing,
        activation_checkpointing_level=args.activation_checkpointing_level, use_fast_moe=args.use_fast_moe,
        use_merged_mlp_in_fast_moe=args.use_merged_mlp_in_fast_moe, force_uniform_routing=args.force_uniform_routing,
        use_fused_ep_alltoall=not args.disable_fused_ep_alltoall)
    if rank == 0:
        print(config, flush=True)
    if not args.use_hf_model:
        load_initial_weights(args, model, pmap, rank)
    if profiler is not None and args.profile_modules:
        profiler.setup_profiler_for_pytorch_model(model)

    eargs = EngineArgs(
        model_choice=args.model_choice, dtype=args.dtype, data_parallelism=dp,
        pipeline_parallelism=args.pipeline_parallelism, virtual_pipeline_parallelism=args.virtual_pipeline_parallelism,
        expert_parallelism=args.expert_parallelism, tensor_parallelism=args.tensor_parallelism,
        use_pp_first=args.use_pp_first, pp_scheme=args.pp_scheme, reuse_buffers_in_1f1b=args.reuse_buffers_in_1f1b,
        use_latest_trainer=args.use_latest_trainer, batch_size=args.batch_size, micro_batch_size=args.micro_batch_size,
        context_size=args.context_size, optimizer=optimizer_key(args), lr=args.lr, min_lr=args.min_lr,
        weight_decay=args.weight_decay, beta1=args.beta1, beta2=args.beta2, eps=args.eps, warmup_steps=args.warmup_steps,
        opt_grad_acc_steps=args.opt_grad_acc_steps,
        opt_disable_delayed_grad_clipping=args.opt_disable_delayed_grad_clipping,
        opt_use_allreduce_for_grad_acc=args.opt_use_allreduce_for_grad_acc,
        opt_use_allreduce_for_param_gather=args.opt_use_allreduce_for_param_gather,
        opt_use_chunked_allreduce=args.opt_use_chunked_allreduce, use_fused_optimizer=not args.disable_fused_optimizer,
        skip_optimizer_step=args.skip_optimizer_step,
        skip_optimizer_step_weight_update=args.skip_optimizer_step_weight_update,
        skip_backward_pass=args.skip_backward_pass,
        disable_optimizer_state_checkpointing=args.disable_optimizer_state_checkpointing)
    engine = TrainEngine(eargs, pmap=pmap, model=model, config=config, device=device)
    optimizer = engine.optimizer
    optimizer.dump_weight_gradients = args.dump_weight_gradients
    sharded_opt = optimizer_key(args) not in ("unsharded", "pt")

    # ------------------------------------------------------------------ resume
    train_step_id = 0
    if args.enable_checkpointing:
        train_step_id, name = ckpt.load_checkpoint(
            args.exp_dir, model, optimizer, pmap, optimizer_sharded=sharded_opt, rank=rank,
            use_broadcast=args.use_broadcast_for_model_init,
            use_allreduce_in_broadcast=args.use_allreduce_in_broadcast_model_init, verbose=(rank == 0))
        engine.step_id = train_step_id

    # ------------------------------------------------------------------ data
    dp_size, dp_index = pmap.data_parallelism * pmap.expert_parallelism, pmap.dp_ind * pmap.expert_parallelism + pmap.ep_ind
    if args.synthetic_data:
        dataset = SyntheticTokenDataset(config.vocab_size, args.context_size, dp_size=dp_size, dp_ind=dp_index)
    elif args.use_sharded_dataset:
        dataset = PclShardedDataParallelDataset(args.dataset_dir, args.num_data_files, args.context_size,
                                                dp_size=dp_size, dp_ind=dp_index)
    else:
        dataset = PclDataPrallelDataset(args.dataset_dir, args.num_data_files, args.context_size, dp_size=dp_size,
                                        dp_ind=dp_index)
    dataset.set_base_dp_idx(train_step_id * args.batch_size)
    loader = torch.utils.data.DataLoader(dataset, batch_size=args.batch_size, num_workers=2, prefetch_factor=4,
                                         pin_memory=(device.type == "cuda"))
    it = iter(loader)
    train_steps = args.train_steps if args.train_steps is not None else len(dataset) // args.batch_size
    if rank == 0:
        print(f"Number of training steps : {train_steps}", flush=True)

    # ------------------------------------------------------------------ loop
    is_logger = (pmap.is_last_stage_rank and pmap.dp_ind == 0 and pmap.tp_ind == 0 and pmap.ep_ind == 0)
    scalar_log = ScalarLog(args.exp_dir) if (args.enable_tb_logging and is_logger and args.exp_dir) else None
    flops_per_seq = model.get_flops(args.context_size) if hasattr(model, "get_flops") else 0
    last_log_time = time.time()
    exit_code = 0
    while train_step_id < train_steps:
        if train_step_id == args.exit_steps:
            break
        st = time.time()
        lr = get_learning_rate(train_step_id, train_steps, args)
        engine.set_lr(lr)
        with record_pcl_function("0train-step-block--1data"):
            dl_st = time.time()
            input_ids = next(it)
            dl_et = time.time()
        with record_pcl_function("0train-step-block--2step"):
            out = engine.train_step(input_ids)

        logging_step = (train_step_id % args.logging_steps == 0)
        failure = False
        if logging_step or args.enable_bad_grad_check:
            loss = out.loss
            lgn = out.grad_norm if out.grad_norm is not None else local_grad_norm(engine)
            global_loss = torch.zeros(1, dtype=torch.float32, device=device)
            if pmap.is_last_stage_rank and loss is not None:
                global_loss += loss.detach().float()
            if dist.is_initialized():
                dist.all_reduce(global_loss)
                global_loss /= (pmap.data_parallelism * pmap.expert_parallelism * pmap.tensor_parallelism)
            # soft node failure: a rank whose loss or gradient norm is not finite
            flags = torch.zeros(world_size, dtype=torch.float32, device=device)
            bad = (~torch.isfinite(lgn.float())).float()
            if loss is not None:
                bad = torch.maximum(bad, (~torch.isfinite(loss.detach().float())).float())
            flags[rank] = bad.reshape(())
            if dist.is_initialized():
                dist.all_reduce(flags)
            if flags.sum().item() > 0:
                if rank == 0:
                    print("Softnode failure detected", flush=True)
                if flags[rank] > 0:
                    print(f"Node : {pmap.node}, Rank : {rank:4d}, dp_ind : {pmap.dp_ind:3d}, pp_ind : {pmap.pp_ind:3d}, "
                          f"ep_ind : {pmap.ep_ind:3d}, tp_ind : {pmap.tp_ind:2d}", flush=True)
                report_soft_failures(flags.cpu(), pmap, rank, world_size)
                failure = True
            # A kernel that gave up (bounded wait ran out, capacity-limited buffer too small) says nothing about the
            # health of this node: it gets its own message and exit code and never enters the soft-failure node list.
            if device_status_failed(engine, rank, pmap, device):
                failure = True
                exit_code = EXIT_DEVICE_STATUS
            if args.enable_bad_grad_check and not torch.isfinite(lgn).item():
                debug_dir = os.path.join(args.exp_dir, os.getenv("PBS_JOBID", "0"))
                os.makedirs(debug_dir, exist_ok=True)
                path = os.path.join(debug_dir, f"bad_grad_debug_rank{rank}-d{pmap.dp_ind}-e{pmap.ep_ind}-t{pmap.tp_ind}.txt")
                with open(path, "w") as fh:
                    fh.write("Parameter, Gradient Norm\n")
                    for n, p in model.named_parameters():
                        if p.grad is not None:
                            fh.write(f"{n:45s}, {p.grad.float().norm().item():.6f}\n")
        if failure:
            exit_code = exit_code or 2
            break

        if logging_step:
            if device.type == "cuda":
                torch.cuda.synchronize()
            now = time.time()
            iter_time = (now - last_log_time) / max(1, args.logging_steps) if train_step_id > 0 else (now - st)
            last_log_time = now
            gn = out.grad_norm if out.grad_norm is not None else lgn
            s = f"Step {train_step_id:4d} / {train_steps}"
            s += f", Loss : {global_loss.item():9.6f}"
            s += f", Grad norm : {float(gn):.6f}"
            s += f", LR : {lr:.8f}"
            s += f", Time : {iter_time:.4f} sec"
            s += f", DL time : {dl_et - dl_st:.4f} sec"
            s += f", Tokens Processed : {(train_step_id + 1) * (pmap.data_parallelism * args.expert_parallelism * args.batch_size) * args.context_size}"
            s += f", Tokens/sec : {((args.batch_size * args.context_size) / iter_time) / (pmap.pipeline_parallelism * pmap.tensor_parallelism):.0f}"
            s += f", Timestamp : {time.time()}"
            s += f", Tflops : {(args.batch_size * flops_per_seq * 1e-12) / iter_time:.2f}"
            s += f", ETA : {((train_steps - (train_step_id + 1)) * iter_time) / 3600:.2f} hr"
            s += f", Local Loss : {(out.loss.item() if out.loss is not None else 0):9.6f}"
            s += f", Local Grad norm : {float(lgn):9.6f}"
            s += f", Rank : {rank} ({pmap.dp_ind},{pmap.pp_ind},{pmap.ep_ind},{pmap.tp_ind})"
            if is_logger and scalar_log is not None:
                scalar_log.write(train_step_id, {"loss": global_loss.item(), "grad_norm": float(gn), "lr": lr,
                                                 "iter_time_s": iter_time,
                                                 "tokens_per_sec_per_gpu": (args.batch_size * args.context_size) / iter_time})
            if is_logger or args.log_all_ranks:
                print(s, flush=True)
                if profiler is not None:
                    profiler.print_timing_table(sort_by_name=True)

        # ------------------------------------------------------------------ checkpoints
        hot_due = args.enable_checkpointing and ((train_step_id + 1) % (args.checkpoint_steps * args.opt_grad_acc_steps) == 0)
        last_due = args.enable_checkpointing and train_step_id == train_steps - 1
        if (hot_due or last_due) and not (logging_step or args.enable_bad_grad_check):
            # the status word is sticky: read it before anything is written (on logging steps it was read above)
            if device_status_failed(engine, rank, pmap, device):
                exit_code = EXIT_DEVICE_STATUS
                break
        if hot_due:
            ckpt.save_checkpoint(args.exp_dir, model, optimizer, pmap, train_step_id, optimizer_sharded=sharded_opt,
                                 dp_staggered=args.dp_staggered_checkpointing, rank=rank)
            if not args.disable_cold_checkpointing:
                ckpt.save_checkpoint(args.exp_dir, model, optimizer, pmap, train_step_id, model_only=True,
                                     name=ckpt.cold_checkpoint_name(train_step_id, pmap, args.batch_size, args.context_size),
                                     optimizer_sharded=sharded_opt, dp_staggered=args.dp_staggered_checkpointing, rank=rank)
        if last_due:
            ckpt.save_checkpoint(args.exp_dir, model, optimizer, pmap, train_step_id, name="main",
                                 optimizer_sharded=sharded_opt, dp_staggered=args.dp_staggered_checkpointing, rank=rank)
        train_step_id += 1
        if profiler is not None:
            if args.chrome_trace and train_step_id == min(train_steps, 3):
                profiler.export_chrome_trace(args.chrome_trace.replace(".json", f"_rank{rank}.json"))
            profiler.reset()

    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return exit_code


if __name__ == "__main__":
    sys.exit(main())
