"""General helpers with the reference's names (optimus/utils.py:12-497): device helpers,
``get_load_balanced_expert_mask``, ``no_init_weights``, ``print_error_info``,
``get_total_norm``, ``dump_weight_gradients`` and friends."""
from __future__ import annotations

import math
import os
from collections import OrderedDict
from contextlib import contextmanager
from typing import Iterable, Union

import torch
from torch import nn


# --------------------------------------------------------------------------- device helpers
def get_device() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_dist_backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


def set_device(device):
    if torch.device(device).type == "cuda":
        torch.cuda.set_device(device)


def device_synchronize():
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def get_shape_string(tensor) -> str:
    return "x".join(str(d) for d in tensor.shape)


def get_pg_world_size(group) -> int:
    import torch.distributed as dist
    return dist.get_world_size(group) if dist.is_initialized() else 1


def get_comms_profile_info_string(tensor, group) -> str:
    """``(<shape>,<dtype>,<group size>)`` suffix used in profiler region names."""
    return f"({get_shape_string(tensor)},{str(tensor.dtype).replace('torch.', '')},{get_pg_world_size(group)})"


def get_torch_dtype(dtype_str: str) -> torch.dtype:
    table = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}
    assert dtype_str in table, "Invalid dtype"
    return table[dtype_str]


def print_debug(string, enabled=True):
    if enabled:
        print(string, flush=True)


def print_pytorch_memory_summary(info="", enabled=True):
    if enabled and torch.cuda.is_available():
        print(f"{info}\n{torch.cuda.memory_summary()}", flush=True)


# --------------------------------------------------------------------------- routing helper
def get_load_balanced_expert_mask(sequence_length, num_experts, num_experts_per_tok, ep_ind=0):
    """``[S, E]`` bool mask that forces perfectly uniform routing: position ``s`` may only
    pick the ``C`` consecutive experts starting at ``(ep_ind*S + s) % E`` (with wrap-around).
    Reference optimus/utils.py:132-155; built vectorised here."""
    S, E, C = sequence_length, num_experts, num_experts_per_tok
    start = (ep_ind * S + torch.arange(S)) % E
    cols = (start[:, None] + torch.arange(C)[None, :]) % E
    mask = torch.zeros((S, E), dtype=torch.bool)
    mask.scatter_(1, cols, True)
    return mask


# --------------------------------------------------------------------------- construction
@contextmanager
def no_init_weights():
    """Skip ``reset_parameters`` of every module constructed inside the context (the weights
    are about to be loaded from a file)."""
    patched = []
    originals = {}
    for cls in (nn.Linear, nn.Embedding, nn.LayerNorm):
        originals[cls] = cls.reset_parameters
        cls.reset_parameters = lambda self, *a, **k: None
        patched.append(cls)
    try:
        yield
    finally:
        for cls in patched:
            cls.reset_parameters = originals[cls]


def get_layer_info_of_pipeline_stage(pp_ind, num_layers, pipeline_parallelism):
    per = math.ceil(num_layers / pipeline_parallelism)
    start = pp_ind * per
    end = min((pp_ind + 1) * per, num_layers) - 1
    return start, end - start + 1


def get_partition_lists(data, num_partitions):
    """Greedy split of ``data`` (sizes) into ``num_partitions`` index lists of roughly equal sum."""
    ideal = sum(data) // num_partitions
    parts = [[] for _ in range(num_partitions)]
    cur, pid = 0, 0
    for i, v in enumerate(data):
        cur += v
        parts[min(pid, num_partitions - 1)].append(i)
        if cur >= ideal:
            pid += 1
            cur = 0
    return parts


def get_model_and_optimizer_memory_usage(model, optimizer):
    """(model GB counting weights + gradients, optimizer-state GB, total GB)."""
    gb = 1024 ** 3
    model_b = sum(2 * t.numel() * t.element_size() for t in model.state_dict().values())
    opt_b = 0
    if optimizer is not None:
        for t in optimizer.state_dict().values():
            if isinstance(t, torch.Tensor):
                opt_b += t.numel() * t.element_size()
    return model_b / gb, opt_b / gb, (model_b + opt_b) / gb


# --------------------------------------------------------------------------- comparisons
def _first(t):
    return t if isinstance(t, torch.Tensor) else t[0]


def error_info(tensor, tensor_ref) -> dict:
    a = _first(tensor).detach().flatten().to(torch.float32)
    b = _first(tensor_ref).detach().flatten().to(torch.float32)
    err = (a - b).abs()
    return {"obs_norm": a.norm().item(), "ref_norm": b.norm().item(), "err_norm": err.norm().item(),
            "min_err": err.min().item(), "max_err": err.max().item(), "avg_err": err.mean().item(),
            "diff_count": int((err > 0).sum().item()), "numel": a.numel()}


def print_error_info(tensor, tensor_ref, name=None, print_sample=True, sort=False):
    """Human-readable error report in the reference's format (optimus/utils.py:326-368)."""
    info = error_info(tensor, tensor_ref)
    a = _first(tensor).detach().flatten()
    b = _first(tensor_ref).detach().flatten()
    s = "*" * 40 + "\n"
    if name is not None:
        s += f"Error information for ({name})\n"
    s += f"Obs tensor norm : {info['obs_norm']:10g}\nRef tensor norm : {info['ref_norm']:10g}\n"
    s += f"Err tensor norm : {info['err_norm']:10g}\nMin error value : {info['min_err']:10g}\n"
    s += f"Max error value : {info['max_err']:10g}\nAvg error value : {info['avg_err']:10g}\n"
    s += f"Diff count      : {info['diff_count']} / {info['numel']} ({info['diff_count'] / info['numel'] * 100:.2f} %)\n"
    if print_sample:
        err = (a.float() - b.float()).abs()
        idx = torch.argsort(err, descending=True) if sort else torch.arange(a.numel(), device=a.device)
        n = min(a.numel(), 8)
        s += f"First {n} values\n"
        for i in range(n):
            s += f"{idx[i]}, {a[idx[i]].item():10g}, {b[idx[i]].item():10g}\n"
    s += "*" * 40 + "\n"
    print(s, flush=True)
    return info


def compare_tensors(tensor, tensor_ref, tensor_name="Tensor", print_sample_size=10):
    info = error_info(tensor, tensor_ref)
    print(f"{tensor_name}: max abs err {info['max_err']:g}, rel err "
          f"{info['err_norm'] / max(info['ref_norm'], 1e-30):g}", flush=True)
    return info


# --------------------------------------------------------------------------- norms / dumps
@torch.no_grad()
def get_total_norm(tensors: Union[torch.Tensor, Iterable[torch.Tensor]], norm_type: float = 2.0,
                   error_if_nonfinite: bool = False, foreach=None) -> torch.Tensor:
    """Norm of the concatenation of ``tensors`` (2-norm on GPU uses the deterministic
    sum-of-squares kernel)."""
    tensors = [tensors] if isinstance(tensors, torch.Tensor) else [t for t in tensors]
    if not tensors:
        return torch.tensor(0.0)
    norm_type = float(norm_type)
    dev = tensors[0].device
    if norm_type == 2.0 and dev.type == "cuda":
        from ..ops import functional as OF
        acc = torch.zeros(1, dtype=torch.float32, device=dev)
        for t in tensors:
            OF.sum_of_squares(t.contiguous(), 1.0, out=acc, accumulate=True)
        total = acc.sqrt().reshape(())
    else:
        norms = [torch.linalg.vector_norm(t.to(torch.float32), norm_type) for t in tensors]
        total = torch.linalg.vector_norm(torch.stack([n.to(dev) for n in norms]), norm_type)
    if error_if_nonfinite and not torch.isfinite(total):
        raise RuntimeError(f"The total norm of order {norm_type} is non-finite")
    return total


def dump_weight_gradients(model, config, pmap, opt_key=None, prefix=None, out_dir="weight_grads"):
    """Save ``{global parameter name: grad}`` for offline diffs between parallel layouts."""
    grads = OrderedDict()
    e_loc = getattr(config, "num_experts", 0) // max(1, pmap.expert_parallelism) if hasattr(config, "num_experts") else 0
    for name, p in model.named_parameters():
        key = name
        toks = name.split(".")
        if "experts" in toks and len(toks) > 5 and toks[5].isdigit():
            toks[5] = str(pmap.ep_ind * e_loc + int(toks[5]))
            key = ".".join(toks)
        if p.grad is not None:
            grads[key] = p.grad.detach().cpu()
    fname = f"grads_dp{pmap.data_parallelism}-ep{pmap.expert_parallelism}-tp{pmap.tensor_parallelism}_rank{pmap.rank}"
    if opt_key is not None:
        fname = f"{opt_key}_{fname}"
    if prefix is not None:
        fname = f"{prefix}_{fname}"
    os.makedirs(out_dir, exist_ok=True)
    torch.save(grads, os.path.join(out_dir, f"{fname}.pt"))


def save_tensor(tensor, name, out_dir="tensors"):
    os.makedirs(out_dir, exist_ok=True)
    torch.save(tensor.detach().cpu(), os.path.join(out_dir, f"{name}.pt"))
