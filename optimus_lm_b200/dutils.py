"""Distributed bring-up: one process per GPU over NCCL (or CPU ranks over gloo).

Counterpart of the reference's optimus/dutils.py:5-117 (``print_rank_0``,
``setup_xpu_distributed``, ``setup_distributed``).  The launcher environment is read from
torchrun (RANK / WORLD_SIZE / LOCAL_RANK / LOCAL_WORLD_SIZE) first and then from the MPI /
PALS / PMI names the reference accepts, so the same job scripts work under ``torchrun`` and
``mpiexec``.
"""
from __future__ import annotations

import datetime
import os
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist

_RANK_KEYS = ("RANK", "PMI_RANK", "OMPI_COMM_WORLD_RANK", "MV2_COMM_WORLD_RANK", "PALS_RANKID")
_WORLD_KEYS = ("WORLD_SIZE", "PMI_SIZE", "OMPI_COMM_WORLD_SIZE", "MV2_COMM_WORLD_SIZE")
_LOCAL_RANK_KEYS = ("LOCAL_RANK", "MPI_LOCALRANKID", "OMPI_COMM_WORLD_LOCAL_RANK",
                    "MV2_COMM_WORLD_LOCAL_RANK", "PALS_LOCAL_RANKID", "TPI_LOCALRANKID")
_LOCAL_WORLD_KEYS = ("LOCAL_WORLD_SIZE", "MPI_LOCALNRANKS", "OMPI_COMM_WORLD_LOCAL_SIZE",
                     "MV2_COMM_WORLD_LOCAL_SIZE", "PALS_LOCAL_SIZE", "TPI_LOCALNRANKS")

SUPPORTED_BACKENDS = ("nccl", "gloo")
# Names the reference's job scripts pass (--dist_backend xccl is its default); they select
# the native backend of the device in use here.
_BACKEND_ALIASES = {"xccl": None, "ccl": None, "mpi": None}


def print_rank_0(string, flush=True, skip=False):
    if skip:
        return
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(string, flush=flush)


def _env_int(keys: Sequence[str], default: int) -> int:
    for k in keys:
        if k in os.environ:
            return int(os.environ[k])
    return default


def resolve_backend(dist_backend: str) -> str:
    """Map a requested backend name to one that exists on this machine."""
    if dist_backend in _BACKEND_ALIASES:
        return "nccl" if torch.cuda.is_available() else "gloo"
    if dist_backend not in SUPPORTED_BACKENDS:
        raise ValueError(f"Unsupported distributed backend {dist_backend}; use one of {SUPPORTED_BACKENDS}")
    return dist_backend


def setup_distributed(dist_backend: str = "nccl", local_rank_to_device_map=None, num_ranks_per_gpu: int = 1,
                      timeout_s: Optional[float] = None) -> Tuple[int, int, int, int]:
    """Initialise ``torch.distributed`` and bind this process to its GPU.

    Returns ``(rank, world_size, local_rank, local_world_size)``.  ``timeout_s`` gives the
    process group a finite collective timeout so that a rank that never joins ends the
    others' next collective with an error instead of a hang.
    """
    assert not (local_rank_to_device_map is not None and num_ranks_per_gpu > 1)
    backend = resolve_backend(dist_backend)
    rank = _env_int(_RANK_KEYS, 0)
    world = _env_int(_WORLD_KEYS, 1)
    local_rank = _env_int(_LOCAL_RANK_KEYS, 0)
    local_world = _env_int(_LOCAL_WORLD_KEYS, max(1, world))
    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(rank), str(world)
    os.environ["LOCAL_RANK"] = os.environ["MPI_LOCALRANKID"] = str(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")

    device_index = None
    if backend == "nccl":
        if local_rank_to_device_map is not None:
            device_index = local_rank_to_device_map[local_rank]
        elif os.environ.get("CUDA_VISIBLE_DEVICES", "").startswith("MIG"):
            device_index = 0
        else:
            device_index = local_rank // num_ranks_per_gpu
        torch.cuda.set_device(device_index)

    kwargs = {}
    if timeout_s is not None:
        kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
    if backend == "nccl":
        kwargs["device_id"] = torch.device("cuda", device_index)
    if not dist.is_initialized():
        dist.init_process_group(backend, rank=rank, world_size=world, **kwargs)
    return dist.get_rank(), dist.get_world_size(), local_rank, local_world


def setup_xpu_distributed(dist_backend: str = "xccl"):
    """Entry point name kept for scripts written against the reference
    (optimus/dutils.py:15-49); it brings up NCCL on a GPU box and gloo elsewhere."""
    return setup_distributed(dist_backend)


def get_default_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")
