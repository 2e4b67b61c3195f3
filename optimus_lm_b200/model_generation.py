"""Random-init model generators: serial per-tensor store -> sharded ``model_<mp_ind>.pth`` files.

Two stages, as in the reference (generate_serial_model.py, generate_parallel_model.py and their
DeepSeek-V3 twins):

1. ``generate_serial_model`` writes every tensor of the unsharded model as ``<name>.pt`` under
   ``serial_models/<model_choice with / -> __>/``.  Work is split over ``world_size`` workers by
   tensor index; workers need no communication because a tensor's values depend on its name only.
2. ``generate_parallel_model`` builds the shard of one (pp, ep, tp) position, fills it from the store
   and saves ``parallel_models/<key>/model_<mp_ind>.pth`` - the file ``dist_train.py
   --use_om_cached_model`` loads.

Unlike the reference these cover all four model families, tensor parallelism and the EP-sharded
dense MLP of DeepSeek-V3, and the result equals what ``--synthetic_init`` builds in memory.
"""
from __future__ import annotations

import os
import time
from typing import List, Optional

import torch

from . import config_utils, model_io
from .engine import build_model
from .mapper import ParallelDpPpEpTpMapper


def _log(rank, msg):
    print(f"Rank {rank} : {msg}", flush=True)


def serial_model_dir(serial_models_dir: str, model_choice: str) -> str:
    return os.path.join(serial_models_dir, model_io.serial_dir_name(model_choice))


def parallel_model_dir(parallel_models_dir: str, model_choice: str, pp: int, ep: int, tp: int, vpp: int,
                       merged_mlp: bool = False) -> str:
    return os.path.join(parallel_models_dir, config_utils.cached_model_key(model_choice, pp, ep, tp, vpp, merged_mlp))


def serial_tensor_list(model_choice: str):
    """(config, [(name, shape)]) of the unsharded model, from a ``meta``-device instance."""
    pmap = ParallelDpPpEpTpMapper(data_parallelism=1, pipeline_parallelism=1, expert_parallelism=1,
                                  tensor_parallelism=1, rank=0, create_groups=False)
    cfg, model = build_model(model_choice, pmap, device="meta", pipeline_parallelism=1, expert_parallelism=1,
                             tensor_parallelism=1, virtual_pipeline_parallelism=1)
    shapes = model_io.serial_parameter_shapes([model_io.shard_plan(model)])
    for mod in model.modules():  # the embedding's padding row is stored as zeros
        if getattr(mod, "padding_idx", None) is not None and hasattr(mod, "weight"):
            cfg._serial_padding_idx = int(mod.padding_idx)
    return cfg, list(shapes.items())


def generate_serial_model(model_choice: str, serial_models_dir: str = "./serial_models", *, rank: int = 0,
                          world_size: int = 1, seed: int = 0, dtype: torch.dtype = torch.float32,
                          overwrite: bool = False, verbose: bool = True) -> List[str]:
    """Write this worker's share of the serial tensors; returns the names it processed."""
    out_dir = serial_model_dir(serial_models_dir, model_choice)
    os.makedirs(out_dir, exist_ok=True)
    t0 = time.time()
    cfg, tensors = serial_tensor_list(model_choice)
    if verbose and rank == 0:
        total = sum(int(torch.Size(s).numel()) for _, s in tensors)
        print(f"Number of parameter names : {len(tensors)}", flush=True)
        print(f"Number of parameters : {total}", flush=True)
    std = cfg.initializer_range
    done = []
    for i, (name, shape) in enumerate(tensors):
        if i % world_size != rank:
            continue
        if overwrite or not os.path.exists(model_io.tensor_path(out_dir, name)):
            t = model_io.seeded_serial_tensor(name, shape, std, seed).to(dtype)
            pad = getattr(cfg, "_serial_padding_idx", None)
            if name.endswith("embed_tokens.weight") and pad is not None and pad < t.shape[0]:
                t[pad].zero_()
            model_io.save_serial_tensor(out_dir, name, t, overwrite=overwrite)
        done.append(name)
        if verbose:
            _log(rank, f"processed {name}")
    if verbose:
        _log(rank, f"serial model creation took {(time.time() - t0) / 60:.2f} minutes ({len(done)} tensors)")
    return done


def generate_parallel_model(model_choice: str, *, pipeline_parallelism: int = 1, expert_parallelism: int = 1,
                            tensor_parallelism: int = 1, virtual_pipeline_parallelism: int = 1,
                            use_merged_mlp_in_fast_moe: bool = False, rank: int = 0,
                            serial_models_dir: str = "./serial_models",
                            parallel_models_dir: str = "./parallel_models", dtype: torch.dtype = torch.bfloat16,
                            verbose: bool = True) -> str:
    """Build, fill and save the shard of model-parallel position ``rank`` (= ``mp_ind``)."""
    pp, ep, tp, vpp = pipeline_parallelism, expert_parallelism, tensor_parallelism, virtual_pipeline_parallelism
    assert 0 <= rank < pp * ep * tp, f"rank {rank} outside the model-parallel grid pp*ep*tp = {pp * ep * tp}"
    pmap = ParallelDpPpEpTpMapper(data_parallelism=1, pipeline_parallelism=pp, expert_parallelism=ep,
                                  tensor_parallelism=tp, rank=rank, create_groups=False)
    kwargs = dict(pipeline_parallelism=pp, expert_parallelism=ep, tensor_parallelism=tp,
                  virtual_pipeline_parallelism=vpp)
    if config_utils.model_family(model_choice) in ("olmoe", "deepseek_v3"):
        kwargs.update(use_fast_moe=True, use_merged_mlp_in_fast_moe=use_merged_mlp_in_fast_moe)
    cfg, model = build_model(model_choice, pmap, dtype=dtype, device="cpu", **kwargs)
    src = serial_model_dir(serial_models_dir, model_choice)
    model_io.fill_shard(model, model_io.file_fetcher(src))
    if verbose:
        _log(rank, "Model parameters initialized from serial model")
    out_dir = parallel_model_dir(parallel_models_dir, model_choice, pp, ep, tp, vpp, use_merged_mlp_in_fast_moe)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, f"model_{pmap.mp_ind}.pth")
    tmp = f"{path}.tmp{os.getpid()}"
    torch.save(model.state_dict(), tmp)
    os.replace(tmp, path)
    if verbose:
        _log(rank, f"Saved the model at {path}")
    return path


def worker_identity():
    """(rank, world_size) of this process from the launcher's environment (torchrun, MPI/PMI), 0/1 when
    run directly.  The generators need no process group, only a way to split the work."""
    for r, w in (("RANK", "WORLD_SIZE"), ("PMI_RANK", "PMI_SIZE"), ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE")):
        if r in os.environ and w in os.environ:
            return int(os.environ[r]), int(os.environ[w])
    return 0, 1


def serial_main(default_model_choice: str, argv: Optional[List[str]] = None):
    import argparse

    p = argparse.ArgumentParser(description="Generate a serial (unsharded) random-init model")
    p.add_argument("--model_choice", type=str, default=default_model_choice)
    p.add_argument("--serial_models_dir", type=str, default="./serial_models")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--dtype", type=str, default="float32", choices=["float32", "bfloat16"])
    p.add_argument("--overwrite", action="store_true")
    args = p.parse_args(argv)
    rank, world = worker_identity()
    generate_serial_model(args.model_choice, args.serial_models_dir, rank=rank, world_size=world, seed=args.seed,
                          dtype=getattr(torch, args.dtype), overwrite=args.overwrite)


def parallel_main(default_model_choice: str, argv: Optional[List[str]] = None):
    import argparse

    p = argparse.ArgumentParser(description="Generate the sharded model files of a parallel layout")
    p.add_argument("--model_choice", type=str, default=default_model_choice)
    p.add_argument("--expert_parallelism", type=int, default=1)
    p.add_argument("--pipeline_parallelism", type=int, default=1)
    p.add_argument("--tensor_parallelism", type=int, default=1)
    p.add_argument("--virtual_pipeline_parallelism", type=int, default=1)
    p.add_argument("--use_merged_mlp_in_fast_moe", action="store_true")
    p.add_argument("--serial_models_dir", type=str, default="./serial_models")
    p.add_argument("--parallel_models_dir", type=str, default="./parallel_models")
    args = p.parse_args(argv)
    rank, world = worker_identity()
    grid = args.pipeline_parallelism * args.expert_parallelism * args.tensor_parallelism
    # one worker per shard when launched with pp*ep*tp processes (the reference's mode), otherwise
    # the shards are dealt round-robin to however many workers there are
    for mp in range(rank, grid, world):
        generate_parallel_model(args.model_choice, pipeline_parallelism=args.pipeline_parallelism,
                                expert_parallelism=args.expert_parallelism,
                                tensor_parallelism=args.tensor_parallelism,
                                virtual_pipeline_parallelism=args.virtual_pipeline_parallelism,
                                use_merged_mlp_in_fast_moe=args.use_merged_mlp_in_fast_moe, rank=mp,
                                serial_models_dir=args.serial_models_dir,
                                parallel_models_dir=args.parallel_models_dir)
