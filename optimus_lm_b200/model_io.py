"""Serial <-> sharded weight layouts.

A *serial* model is the unsharded network: one tensor per parameter, named with global layer and
expert indices (``model.layers.17.mlp.experts.42.up_proj.weight``), stored as one ``<name>.pt`` file
per tensor so that models far larger than one host's memory can be produced and consumed piecewise
(the reference's generators do the same, generate_serial_model.py:98-106).  A *shard* is the
``state_dict`` of the model one (pp_ind, ep_ind, tp_ind) position owns.

``shard_plan(model)`` describes every local parameter as a list of pieces of serial tensors.  The
plan is derived from the constructed module tree (it works on the ``meta`` device), so the same
description drives

* the serial -> shard generators (reference generate_parallel_model.py:117-160 renames layers for
  PP/VPP and experts for EP and splits merged expert tensors; here TP slices and the EP-sharded
  dense MLP of DeepSeek-V3 are covered too),
* the shard -> serial / Hugging Face converters (reference
  evals/convert_olmoe_ppep_om_checkpoint_to_hf.py:17-42), and
* the seeded random initialiser, which draws a tensor from its *serial* name.
"""
from __future__ import annotations

import os
import re
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.nn as nn


@dataclass
class Piece:
    """One slice of a serial tensor inside a local parameter.

    ``index``: position along dim 0 of a merged ``[E_local, ...]`` parameter (``None`` when the local
    parameter is not merged).  ``dim``/``start``/``stop``: the slice of the serial tensor
    (``dim is None`` = the whole tensor).  ``serial_shape``: shape of the serial tensor.
    ``pad_rows``: rows of zero padding appended to the serial tensor before slicing (vocabulary
    padded to a multiple of the TP degree)."""
    serial_name: str
    serial_shape: Tuple[int, ...]
    index: Optional[int] = None
    dim: Optional[int] = None
    start: int = 0
    stop: int = 0
    pad_rows: int = 0


def _inner(model):
    return getattr(model, "model", model)


def global_layer_of(model, local_layer: int) -> int:
    inner = _inner(model)
    if hasattr(inner, "global_layer_index"):
        return int(inner.global_layer_index(local_layer))
    if hasattr(inner, "layer_ids"):
        return int(inner.layer_ids[local_layer])
    return int(getattr(inner, "layer_start_idx", 0)) + local_layer


_LAYER_RE = re.compile(r"^(.*layers\.)(\d+)(\..*)$")
_EXPERT_RE = re.compile(r"^(.*\.experts\.)(\d+)(\..*)$")
_COL_RE = re.compile(r"\.(q|k|v|gate|up)_proj\.weight$")   # output features sharded over TP
_ROW_RE = re.compile(r"\.(o|down)_proj\.weight$")          # input features sharded over TP


def shard_plan(model: nn.Module) -> Dict[str, List[Piece]]:
    """Map every local parameter name to the serial pieces it is made of."""
    pmap = getattr(model, "pmap", None)
    tp = pmap.tensor_parallelism if pmap is not None else 1
    tp_ind = pmap.tp_ind if pmap is not None else 0
    modules = dict(model.named_modules())
    plan: Dict[str, List[Piece]] = {}
    for name, p in model.named_parameters():
        shape = tuple(p.shape)
        key = name
        m = _LAYER_RE.match(key)
        if m:
            key = f"{m.group(1)}{global_layer_of(model, int(m.group(2)))}{m.group(3)}"
        owner = modules.get(name.rsplit(".", 1)[0])                              # e.g. the nn.Linear
        mlp = modules.get(name.rsplit(".", 2)[0]) if name.count(".") >= 2 else None  # its parent block
        m = _EXPERT_RE.match(key)
        if m:
            block = modules.get(name.split(".experts.")[0])
            e0 = int(getattr(block, "expert_start_idx", 0))
            plan[name] = [Piece(f"{m.group(1)}{e0 + int(m.group(2))}{m.group(3)}", shape)]
        elif name.endswith("_merged_weight"):
            block = modules.get(name.split(".experts.")[0])
            e0 = int(getattr(block, "expert_start_idx", 0))
            proj = name.rsplit(".", 1)[1].replace("_merged_weight", "")
            base = key.rsplit(".", 1)[0]
            plan[name] = [Piece(f"{base}.{e0 + le}.{proj}.weight", shape[1:], index=le) for le in range(shape[0])]
        elif tp > 1 and type(owner).__name__ == "ParallelEmbedding":
            plan[name] = [Piece(key, (owner.vocab_size, shape[1]), dim=0, start=owner.start_embedding_id,
                                stop=owner.end_embedding_id, pad_rows=owner.vocab_size_padded - owner.vocab_size)]
        elif tp > 1 and type(owner).__name__ == "ParallelLMHead":
            plan[name] = [Piece(key, (shape[0], shape[1] * tp), dim=1, start=tp_ind * shape[1],
                                stop=(tp_ind + 1) * shape[1])]
        elif tp > 1 and p.dim() == 2 and _COL_RE.search(name):
            plan[name] = [Piece(key, (shape[0] * tp, shape[1]), dim=0, start=tp_ind * shape[0],
                                stop=(tp_ind + 1) * shape[0])]
        elif tp > 1 and p.dim() == 2 and _ROW_RE.search(name):
            plan[name] = [Piece(key, (shape[0], shape[1] * tp), dim=1, start=tp_ind * shape[1],
                                stop=(tp_ind + 1) * shape[1])]
        elif mlp is not None and getattr(mlp, "intermediate_size_per_rank", None) is not None \
                and getattr(mlp, "intermediate_size", None) != mlp.intermediate_size_per_rank and tp == 1 \
                and getattr(mlp, "pmap", None) is not None and p.dim() == 2:
            # DeepSeek-V3 dense MLP: intermediate dimension sharded over the EP group
            ep, ei = mlp.pmap.expert_parallelism, mlp.pmap.ep_ind
            if name.endswith("down_proj.weight"):
                plan[name] = [Piece(key, (shape[0], shape[1] * ep), dim=1, start=ei * shape[1], stop=(ei + 1) * shape[1])]
            else:
                plan[name] = [Piece(key, (shape[0] * ep, shape[1]), dim=0, start=ei * shape[0], stop=(ei + 1) * shape[0])]
        else:
            plan[name] = [Piece(key, shape)]
    return plan


def serial_parameter_shapes(plan_list: Iterable[Dict[str, List[Piece]]]) -> Dict[str, Tuple[int, ...]]:
    """Union of the serial tensors (name -> shape) that a set of shard plans refers to."""
    out: Dict[str, Tuple[int, ...]] = {}
    for plan in plan_list:
        for pieces in plan.values():
            for pc in pieces:
                out[pc.serial_name] = tuple(pc.serial_shape)
    return out


def _slice_of(full: torch.Tensor, pc: Piece) -> torch.Tensor:
    if pc.dim is None:
        return full
    if pc.pad_rows:
        pad = torch.zeros((pc.pad_rows,) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
        full = torch.cat([full, pad], dim=0)
    return full.narrow(pc.dim, pc.start, pc.stop - pc.start)


@torch.no_grad()
def fill_shard(model: nn.Module, fetch: Callable[[str, Tuple[int, ...]], torch.Tensor], plan=None) -> None:
    """Set every local parameter from serial tensors returned by ``fetch(serial_name, serial_shape)``."""
    plan = shard_plan(model) if plan is None else plan
    params = dict(model.named_parameters())
    for name, pieces in plan.items():
        p = params[name]
        for pc in pieces:
            full = fetch(pc.serial_name, tuple(pc.serial_shape))
            assert tuple(full.shape) == tuple(pc.serial_shape), \
                f"{pc.serial_name}: stored shape {tuple(full.shape)} != expected {tuple(pc.serial_shape)}"
            src = _slice_of(full, pc)
            dst = p if pc.index is None else p[pc.index]
            dst.copy_(src)


@torch.no_grad()
def scatter_shard(plan: Dict[str, List[Piece]], state_dict: Dict[str, torch.Tensor],
                  serial: Dict[str, torch.Tensor]) -> None:
    """Write the parameters of one shard ``state_dict`` into the serial tensors of ``serial``
    (allocated on first touch).  Replicated parameters are simply overwritten with equal values."""
    for name, pieces in plan.items():
        if name not in state_dict:
            continue
        t = state_dict[name]
        for pc in pieces:
            src = t if pc.index is None else t[pc.index]
            if pc.serial_name not in serial:
                serial[pc.serial_name] = torch.zeros(pc.serial_shape, dtype=src.dtype)
            full = serial[pc.serial_name]
            if pc.dim is None:
                full.copy_(src)
                continue
            start, stop = pc.start, pc.stop
            limit = full.shape[pc.dim]
            if start >= limit:
                continue  # this slice is vocabulary padding only
            n = min(stop, limit) - start
            full.narrow(pc.dim, start, n).copy_(src.narrow(pc.dim, 0, n))


# ---------------------------------------------------------------- seeded serial tensors


def is_norm_weight(serial_name: str, serial_shape) -> bool:
    return len(serial_shape) == 1 and "norm" in serial_name


def seeded_serial_tensor(serial_name: str, serial_shape, std: float, seed: int = 0, device="cpu") -> torch.Tensor:
    """The initial value of a serial tensor as a function of its name alone: ones for norm weights,
    N(0, std) (fp32) for everything else, from a generator seeded with (seed, crc32(name)).  The
    reference's generator draws Linear / Embedding weights ~ N(0, initializer_range) and sets norm
    weights to one (generate_serial_model.py:118-158); tying the stream to the name lets any rank of
    any layout draw exactly its own slices."""
    import zlib

    shape = tuple(int(s) for s in serial_shape)
    if is_norm_weight(serial_name, shape):
        return torch.ones(shape, dtype=torch.float32, device=device)
    if serial_name.endswith(".bias"):
        return torch.zeros(shape, dtype=torch.float32, device=device)
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + zlib.crc32(serial_name.encode())) % (2 ** 63))
    n = 1
    for d in shape:
        n *= d
    if n <= (1 << 28):
        return torch.randn(shape, device=device, dtype=torch.float32, generator=g) * std
    out = torch.empty(n, dtype=torch.float32, device=device)  # big tensors: bounded temporaries
    step = 1 << 26
    for s in range(0, n, step):
        e = min(s + step, n)
        out[s:e] = torch.randn(e - s, device=device, dtype=torch.float32, generator=g) * std
    return out.view(shape)


# ---------------------------------------------------------------- per-tensor file store


def serial_dir_name(model_choice: str) -> str:
    return model_choice.replace("/", "__")


def tensor_path(serial_dir: str, name: str) -> str:
    return os.path.join(serial_dir, f"{name}.pt")


def save_serial_tensor(serial_dir: str, name: str, tensor: torch.Tensor, overwrite: bool = False) -> bool:
    """Atomic write of one serial tensor; an existing file is kept unless ``overwrite``."""
    path = tensor_path(serial_dir, name)
    if os.path.exists(path) and not overwrite:
        return False
    tmp = f"{path}.tmp{os.getpid()}"
    torch.save(tensor.contiguous(), tmp)
    os.replace(tmp, path)
    return True


def load_serial_tensor(serial_dir: str, name: str) -> torch.Tensor:
    return torch.load(tensor_path(serial_dir, name), map_location="cpu", weights_only=True)


def file_fetcher(serial_dir: str) -> Callable[[str, Tuple[int, ...]], torch.Tensor]:
    def fetch(name, shape):
        return load_serial_tensor(serial_dir, name)
    return fetch


def dict_fetcher(tensors: Dict[str, torch.Tensor]) -> Callable[[str, Tuple[int, ...]], torch.Tensor]:
    def fetch(name, shape):
        return tensors[name]
    return fetch
