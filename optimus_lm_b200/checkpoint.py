"""Checkpoint / resume in the reference's on-disk format (dist_train.py:593-690, 963-1087).

``<exp_dir>/checkpoints/<name>/``
    ``model_checkpoint.pth`` or ``model_checkpoint_shard-{mp_ind}.pth``
        ``{"train_step_id": step + 1, "state_dict": model.state_dict()}``, written by ``dp_ind == 0``
        (or by ``dp_ind == mp_ind % DP`` with staggered checkpointing)
    ``optimizer_checkpoint.pth`` (rank 0, unsharded) or ``optimizer_checkpoint_shard-{rank}.pth``
        ``{"state_dict": optimizer.state_dict()}``
    ``completed``   text file with the step number, written last by rank 0; removed first when a
                    directory is overwritten

Names: the *hot* double buffer ``checkpoint1`` / ``checkpoint2`` (write to the older or invalid
one, read the newer valid one), *cold* model-only ``step{N}-tokens{X}B`` and ``main`` at the end.

Written files go through a temporary name + ``os.replace`` so that a crash during ``torch.save``
never leaves a truncated file under the final name.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

HOT = ("checkpoint1", "checkpoint2")
MARKER = "completed"


def _ckpt_dir(exp_dir, name):
    return os.path.join(exp_dir, "checkpoints", name)


def read_marker(exp_dir, name) -> Optional[int]:
    """Step number of a completed checkpoint, or None if it is missing / unreadable."""
    path = os.path.join(_ckpt_dir(exp_dir, name), MARKER)
    try:
        with open(path) as fh:
            return int(fh.readline().strip())
    except (OSError, ValueError):
        return None


def choose_checkpoint_for_reading(exp_dir, verbose=False) -> Optional[str]:
    steps = {n: read_marker(exp_dir, n) for n in HOT}
    valid = {n: s for n, s in steps.items() if s is not None}
    if not valid:
        if verbose:
            print("Both checkpoints are invalid. Starting training from scratch", flush=True)
        return None
    name = max(valid, key=lambda n: valid[n])
    if verbose:
        print(f"Valid checkpoints {valid}. Choosing latest checkpoint i.e, {name} for reading", flush=True)
    return name


def choose_checkpoint_for_writing(exp_dir, verbose=False) -> str:
    """The invalid one if any, else the older one (never the newest valid checkpoint)."""
    s1, s2 = read_marker(exp_dir, HOT[0]), read_marker(exp_dir, HOT[1])
    if s1 is not None and s2 is not None:
        name = HOT[1] if s1 > s2 else HOT[0]
    elif s1 is not None:
        name = HOT[1]
    else:
        name = HOT[0]
    if verbose:
        print(f"Checkpoint steps: checkpoint1={s1} checkpoint2={s2}. Writing to {name}", flush=True)
    return name


def model_file(ckpt_dir, pmap):
    if pmap.is_model_parallel:
        return os.path.join(ckpt_dir, f"model_checkpoint_shard-{pmap.mp_ind}.pth")
    return os.path.join(ckpt_dir, "model_checkpoint.pth")


def optimizer_file(ckpt_dir, rank, sharded: bool):
    if sharded:
        return os.path.join(ckpt_dir, f"optimizer_checkpoint_shard-{rank}.pth")
    return os.path.join(ckpt_dir, "optimizer_checkpoint.pth")


def _atomic_save(obj, path):
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def _barrier():
    if dist.is_available() and dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        dist.barrier()


def cold_checkpoint_name(train_step_id, pmap, batch_size, context_size) -> str:
    tokens_b = (train_step_id + 1) * (pmap.data_parallelism * pmap.expert_parallelism) * (batch_size * context_size) * 1e-9
    return f"step{train_step_id + 1}-tokens{round(tokens_b):.0f}B"


def save_checkpoint(exp_dir, model, optimizer, pmap, train_step_id, *, name=None, model_only=False,
                    optimizer_sharded=True, dp_staggered=False, rank=None, verbose=True) -> str:
    """Collective over all ranks.  ``train_step_id`` is the step that just finished."""
    fused = getattr(optimizer, "_fused", None)
    if fused is not None and hasattr(fused, "materialize"):
        fused.materialize()      # weights whose all-gather is pending until their next forward GEMM
    rank = (dist.get_rank() if dist.is_initialized() else 0) if rank is None else rank
    name = choose_checkpoint_for_writing(exp_dir, verbose and rank == 0) if name is None else name
    d = _ckpt_dir(exp_dir, name)
    marker = os.path.join(d, MARKER)
    if rank == 0:
        if verbose:
            print(f"Saving checkpoint to {d}", flush=True)
        os.makedirs(d, exist_ok=True)
    _barrier()
    if rank == 0 and os.path.exists(marker):
        os.remove(marker)
    _barrier()
    writer = (pmap.dp_ind == pmap.mp_ind % pmap.data_parallelism) if dp_staggered else (pmap.dp_ind == 0)
    if writer:
        state = {k: v.detach().cpu() for k, v in model.state_dict().items()}
        _atomic_save({"train_step_id": train_step_id + 1, "state_dict": state}, model_file(d, pmap))
    _barrier()
    if not model_only and (optimizer_sharded or rank == 0):
        sd = optimizer.state_dict()
        sd = {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in sd.items()}
        _atomic_save({"state_dict": sd}, optimizer_file(d, rank, optimizer_sharded))
    _barrier()
    if rank == 0:
        with open(marker + ".tmp", "w") as fh:
            fh.write(f"{train_step_id + 1}")
        os.replace(marker + ".tmp", marker)
        if verbose:
            print(f"Saved checkpoint to {name} successfully", flush=True)
    _barrier()
    return name


def load_checkpoint(exp_dir, model, optimizer, pmap, *, name=None, optimizer_sharded=True, rank=None,
                    use_broadcast=False, use_allreduce_in_broadcast=False, verbose=True) -> Tuple[int, Optional[str]]:
    """Load the newest valid hot checkpoint (or ``name``).  Returns ``(train_step_id, name)``;
    ``(0, None)`` when there is nothing to resume from.

    ``use_broadcast``: only ``dp_ind == 0`` reads the model file; the parameters then travel over
    the data-parallel group (broadcast, or all-reduce of zero-filled copies)."""
    rank = (dist.get_rank() if dist.is_initialized() else 0) if rank is None else rank
    name = choose_checkpoint_for_reading(exp_dir, verbose and rank == 0) if name is None else name
    if name is None:
        return 0, None
    d = _ckpt_dir(exp_dir, name)
    device = next(model.parameters()).device
    if not use_broadcast or not dist.is_initialized():
        ck = torch.load(model_file(d, pmap), map_location="cpu", weights_only=True)
        model.load_state_dict(ck["state_dict"])
        step = int(ck["train_step_id"])
    else:
        step_t = torch.zeros(1, dtype=torch.long, device=device)
        if pmap.dp_ind == 0:
            ck = torch.load(model_file(d, pmap), map_location="cpu", weights_only=True)
            model.load_state_dict(ck["state_dict"])
            step_t[0] = int(ck["train_step_id"])
        # everything the state dict holds travels: parameters and persistent buffers (DeepSeek-V3's routing bias is a
        # buffer that training may modify; replicas that kept their own copy would route differently after a resume)
        tensors = [t for t in model.state_dict().values() if torch.is_tensor(t)]
        if pmap.dp_ind != 0 and use_allreduce_in_broadcast:
            with torch.no_grad():
                for t in tensors:
                    t.zero_()
        if pmap.data_parallelism > 1:
            src = pmap.mp_rank  # global rank of the dp_ind == 0 member of this DP group
            for t in tensors:
                if use_allreduce_in_broadcast:
                    dist.all_reduce(t, group=pmap.dp_group)
                else:
                    dist.broadcast(t, src=src, group=pmap.dp_group)
            if use_allreduce_in_broadcast:
                dist.all_reduce(step_t, group=pmap.dp_group)
            else:
                dist.broadcast(step_t, src=src, group=pmap.dp_group)
        step = int(step_t.item())
    opt_path = optimizer_file(d, rank, optimizer_sharded)
    if optimizer is not None and os.path.exists(opt_path):
        ock = torch.load(opt_path, map_location="cpu", weights_only=True)
        optimizer.load_state_dict(ock["state_dict"])
    return step, name
