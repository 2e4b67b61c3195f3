"""Checkpoint conversion between the framework's sharded files and Hugging Face checkpoints.

* ``om_checkpoint_to_serial``: merge the ``model_checkpoint[_shard-<mp>].pth`` files of a PP x EP x TP
  (x VPP, merged or per-expert) run into one serial name -> tensor dict.  The reference does this
  by renaming layers and experts and splitting merged tensors
  (evals/convert_olmoe_ppep_om_checkpoint_to_hf.py:17-42, evals/convert_olmoe_om_checkpoint_to_hf.py:36-92);
  here the shard plan of a ``meta``-device model gives the mapping, so every layout is covered.
* ``om_checkpoint_to_hf``: the serial dict written as ``model[-xxxxx-of-yyyyy].safetensors`` +
  ``config.json`` in the on-disk key format of ``transformers`` (one tensor per expert
  projection); tokenizer files are copied when a source directory is given.  No model is
  instantiated, so a 100B-parameter checkpoint converts with one shard in memory at a time.
* ``hf_checkpoint_to_omcached``: an HF checkpoint directory cut into ``model_<mp_ind>.pth`` files
  for a parallel layout (reference scripts/convert_hfcp_to_omcached.py does this for Llama with
  PP only).
* ``om_checkpoint_to_omcached``: training checkpoint shards re-saved as cached model shards
  (reference scripts/convert_omcp_to_omcached.py).
"""
from __future__ import annotations

import json
import os
import re
import shutil
from typing import Dict, Iterable, Optional

import torch

from . import config_utils, model_io
from .engine import build_model
from .mapper import ParallelDpPpEpTpMapper


def _layout_kwargs(model_choice, pp, ep, tp, vpp, merged):
    kw = dict(pipeline_parallelism=pp, expert_parallelism=ep, tensor_parallelism=tp, virtual_pipeline_parallelism=vpp)
    if config_utils.model_family(model_choice) in ("olmoe", "deepseek_v3"):
        kw.update(use_fast_moe=True, use_merged_mlp_in_fast_moe=merged)
    return kw


def meta_shard(model_choice: str, mp_ind: int, pp=1, ep=1, tp=1, vpp=1, merged=False, device="meta",
               dtype=torch.bfloat16):
    """(config, model, pmap) of model-parallel position ``mp_ind`` without allocating weights."""
    pmap = ParallelDpPpEpTpMapper(data_parallelism=1, pipeline_parallelism=pp, expert_parallelism=ep,
                                  tensor_parallelism=tp, rank=mp_ind, create_groups=False)
    cfg, model = build_model(model_choice, pmap, device=device, dtype=dtype,
                             **_layout_kwargs(model_choice, pp, ep, tp, vpp, merged))
    return cfg, model, pmap


def _is_merged(state_dict) -> bool:
    return any(k.endswith("_merged_weight") for k in state_dict)


def checkpoint_shard_path(ckpt_dir: str, mp_ind: int, grid: int) -> str:
    if grid == 1:
        single = os.path.join(ckpt_dir, "model_checkpoint.pth")
        if os.path.exists(single):
            return single
    return os.path.join(ckpt_dir, f"model_checkpoint_shard-{mp_ind}.pth")


def _load_state(path):
    obj = torch.load(path, map_location="cpu", weights_only=True)
    return obj["state_dict"] if isinstance(obj, dict) and "state_dict" in obj else obj


def om_checkpoint_to_serial(model_choice: str, ckpt_dir: str, *, pp=1, ep=1, tp=1, vpp=1, cached=False,
                            verbose=False) -> Dict[str, torch.Tensor]:
    """Merge all model shards under ``ckpt_dir`` (training checkpoint files, or ``model_<mp>.pth``
    cached files with ``cached=True``) into serial tensors.  Buffers that are part of the state
    dict (DeepSeek-V3's ``e_score_correction_bias``) are carried over by their global layer name."""
    grid = pp * ep * tp
    serial: Dict[str, torch.Tensor] = {}
    for mp in range(grid):
        path = os.path.join(ckpt_dir, f"model_{mp}.pth") if cached else checkpoint_shard_path(ckpt_dir, mp, grid)
        sd = _load_state(path)
        if verbose:
            print(f"Processing model shard {mp} ({path})", flush=True)
        _, model, _ = meta_shard(model_choice, mp, pp, ep, tp, vpp, merged=_is_merged(sd))
        plan = model_io.shard_plan(model)
        missing = [k for k in plan if k not in sd]
        assert not missing, f"{path} lacks parameters {missing[:4]}..."
        model_io.scatter_shard(plan, sd, serial)
        for k, v in sd.items():  # persistent buffers
            if k in plan:
                continue
            m = re.match(r"^(.*layers\.)(\d+)(\..*)$", k)
            if m:
                k = f"{m.group(1)}{model_io.global_layer_of(model, int(m.group(2)))}{m.group(3)}"
            serial[k] = v.clone()
    return serial


# ---------------------------------------------------------------- Hugging Face side


def hf_config_dict(model_choice: str, cfg=None, torch_dtype="bfloat16") -> dict:
    """``config.json`` content for the HF architecture of ``model_choice``: the HF config class is
    constructed from the attributes our config shares with it."""
    import inspect

    import transformers

    fam = config_utils.model_family(model_choice)
    cfg = config_utils.build_config(model_choice) if cfg is None else cfg
    cls_name, arch = {"olmoe": ("OlmoeConfig", "OlmoeForCausalLM"), "olmo": ("OlmoConfig", "OlmoForCausalLM"),
                      "llama": ("LlamaConfig", "LlamaForCausalLM"),
                      "deepseek_v3": ("DeepseekV3Config", "DeepseekV3ForCausalLM")}[fam]
    hf_cls = getattr(transformers, cls_name)
    names = set(inspect.signature(hf_cls.__init__).parameters) | set(getattr(hf_cls, "__annotations__", {}))
    kwargs = {}
    if hasattr(cfg, "rope_theta"):
        # newer transformers carry theta and the scaling rule in one ``rope_parameters`` dict
        scaling = dict(getattr(cfg, "rope_scaling", None) or {})
        legacy_type = scaling.pop("type", None)
        scaling.setdefault("rope_type", legacy_type or "default")
        if "rope_parameters" in names:
            kwargs["rope_parameters"] = {**scaling, "rope_theta": float(cfg.rope_theta)}
        else:
            kwargs["rope_theta"] = float(cfg.rope_theta)
            if scaling:
                kwargs["rope_scaling"] = scaling
    names -= {"self", "kwargs", "rope_scaling", "rope_parameters", "rope_theta", "layer_types"}
    for n in names:
        if hasattr(cfg, n):
            v = getattr(cfg, n)
            if isinstance(v, (int, float, bool, str)) or v is None:
                kwargs[n] = v
    if fam == "olmoe" and getattr(cfg, "padding_idx", None) is not None:
        kwargs["pad_token_id"] = cfg.padding_idx
    if fam == "deepseek_v3":
        kwargs["n_routed_experts"] = getattr(cfg, "n_routed_experts", getattr(cfg, "num_experts", None))
    hf = hf_cls(**{k: v for k, v in kwargs.items() if v is not None or k == "pad_token_id"})
    d = hf.to_dict()
    d["architectures"] = [arch]
    d["use_cache"] = True
    d["torch_dtype"] = torch_dtype
    return d


def write_hf_checkpoint(serial: Dict[str, torch.Tensor], config: dict, hf_dir: str, *,
                        max_shard_bytes: int = 5 << 30, tokenizer_dir: Optional[str] = None,
                        tie_word_embeddings: bool = False) -> None:
    from safetensors.torch import save_file

    os.makedirs(hf_dir, exist_ok=True)
    names = sorted(serial)
    if tie_word_embeddings:
        names = [n for n in names if n != "lm_head.weight"]
    shards, cur, cur_bytes = [], [], 0
    for n in names:
        b = serial[n].numel() * serial[n].element_size()
        if cur and cur_bytes + b > max_shard_bytes:
            shards.append(cur)
            cur, cur_bytes = [], 0
        cur.append(n)
        cur_bytes += b
    if cur:
        shards.append(cur)
    if len(shards) == 1:
        save_file({n: serial[n].contiguous() for n in shards[0]}, os.path.join(hf_dir, "model.safetensors"),
                  metadata={"format": "pt"})
    else:
        weight_map, total = {}, 0
        for i, group in enumerate(shards):
            fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            save_file({n: serial[n].contiguous() for n in group}, os.path.join(hf_dir, fname), metadata={"format": "pt"})
            for n in group:
                weight_map[n] = fname
                total += serial[n].numel() * serial[n].element_size()
        with open(os.path.join(hf_dir, "model.safetensors.index.json"), "w") as fh:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, fh, indent=2)
    with open(os.path.join(hf_dir, "config.json"), "w") as fh:
        json.dump(config, fh, indent=2, default=str)
    if tokenizer_dir is not None and os.path.isdir(tokenizer_dir):
        for f in os.listdir(tokenizer_dir):
            if f.startswith(("tokenizer", "special_tokens", "vocab", "merges", "added_tokens")):
                shutil.copy(os.path.join(tokenizer_dir, f), os.path.join(hf_dir, f))


def om_checkpoint_to_hf(model_choice: str, om_checkpoint_dir: str, hf_checkpoint_dir: str, *, pp=1, ep=1, tp=1,
                        vpp=1, cached=False, tokenizer_dir: Optional[str] = None, verbose=True) -> None:
    serial = om_checkpoint_to_serial(model_choice, om_checkpoint_dir, pp=pp, ep=ep, tp=tp, vpp=vpp, cached=cached,
                                     verbose=verbose)
    cfg = config_utils.build_config(model_choice)
    dtype = str(next(iter(serial.values())).dtype).replace("torch.", "")
    if verbose:
        print(f"Saving HF checkpoint to {hf_checkpoint_dir}", flush=True)
    write_hf_checkpoint(serial, hf_config_dict(model_choice, cfg, dtype), hf_checkpoint_dir,
                        tokenizer_dir=tokenizer_dir, tie_word_embeddings=bool(getattr(cfg, "tie_word_embeddings", False)))
    if verbose:
        print("Saving checkpoint done", flush=True)


class HFCheckpointReader:
    """Tensor-at-a-time reader of an HF checkpoint directory (safetensors, single or indexed;
    ``pytorch_model.bin`` as a fallback)."""

    def __init__(self, hf_dir: str):
        self.dir = hf_dir
        self.where: Dict[str, str] = {}
        self._bin = None
        idx = os.path.join(hf_dir, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as fh:
                self.where = dict(json.load(fh)["weight_map"])
        elif os.path.exists(os.path.join(hf_dir, "model.safetensors")):
            from safetensors import safe_open
            with safe_open(os.path.join(hf_dir, "model.safetensors"), "pt") as f:
                self.where = {k: "model.safetensors" for k in f.keys()}
        else:
            self._bin = torch.load(os.path.join(hf_dir, "pytorch_model.bin"), map_location="cpu", weights_only=True)
            self.where = {k: "pytorch_model.bin" for k in self._bin}

    def names(self) -> Iterable[str]:
        return self.where.keys()

    def get(self, name: str) -> torch.Tensor:
        if self._bin is not None:
            return self._bin[name]
        from safetensors import safe_open
        with safe_open(os.path.join(self.dir, self.where[name]), "pt") as f:
            return f.get_tensor(name)


def hf_checkpoint_to_omcached(model_choice: str, hf_dir: str, parallel_models_dir: str, *, pp=1, ep=1, tp=1, vpp=1,
                              merged=False, ranks: Optional[Iterable[int]] = None, dtype=torch.bfloat16,
                              verbose=True):
    """Cut an HF checkpoint into ``model_<mp_ind>.pth`` files of a parallel layout; returns the paths."""
    reader = HFCheckpointReader(hf_dir)
    tied = "lm_head.weight" not in reader.where

    def fetch(name, shape):
        if name == "lm_head.weight" and tied:
            name = "model.embed_tokens.weight"
        return reader.get(name)

    out_dir = os.path.join(parallel_models_dir, config_utils.cached_model_key(model_choice, pp, ep, tp, vpp, merged))
    os.makedirs(out_dir, exist_ok=True)
    paths = []
    for mp in (range(pp * ep * tp) if ranks is None else ranks):
        _, model, pmap = meta_shard(model_choice, mp, pp, ep, tp, vpp, merged, device="cpu", dtype=dtype)
        model_io.fill_shard(model, fetch)
        sd = model.state_dict()
        for k in list(sd):  # buffers stored in the HF checkpoint (router bias of DeepSeek-V3)
            if k.endswith("e_score_correction_bias"):
                m = re.match(r"^(.*layers\.)(\d+)(\..*)$", k)
                g = f"{m.group(1)}{model_io.global_layer_of(model, int(m.group(2)))}{m.group(3)}"
                if g in reader.where:
                    sd[k] = reader.get(g).to(sd[k].dtype)
        path = os.path.join(out_dir, f"model_{pmap.mp_ind}.pth")
        torch.save(sd, path + ".tmp")
        os.replace(path + ".tmp", path)
        paths.append(path)
        if verbose:
            print(f"Saved the model at {path}", flush=True)
    return paths


def om_checkpoint_to_omcached(om_checkpoint_dir: str, om_cached_dir: str, verbose=True):
    """``model_checkpoint_shard-<i>.pth`` (``{"state_dict": ...}``) -> ``model_<i>.pth`` (bare state dict)."""
    files = [f for f in os.listdir(om_checkpoint_dir) if f.startswith("model_checkpoint")]
    os.makedirs(om_cached_dir, exist_ok=True)
    out = []
    for f in sorted(files):
        m = re.match(r"model_checkpoint_shard-(\d+)\.pth$", f)
        idx = int(m.group(1)) if m else 0
        if verbose:
            print(f"Converting {f}", flush=True)
        sd = _load_state(os.path.join(om_checkpoint_dir, f))
        path = os.path.join(om_cached_dir, f"model_{idx}.pth")
        torch.save(sd, path + ".tmp")
        os.replace(path + ".tmp", path)
        out.append(path)
    return out


def add_layout_arguments(parser, pp=1, ep=1, tp=1, vpp=1):
    parser.add_argument("--pipeline_parallelism", type=int, default=pp)
    parser.add_argument("--expert_parallelism", type=int, default=ep)
    parser.add_argument("--tensor_parallelism", type=int, default=tp)
    parser.add_argument("--virtual_pipeline_parallelism", type=int, default=vpp)
    return parser


def om_to_hf_main(default_model_choice: str, family: str, argv=None, pp=1, ep=1):
    """Shared command line of the ``evals/convert_*_om_checkpoint_to_hf.py`` scripts."""
    import argparse

    p = argparse.ArgumentParser(description="Convert a training checkpoint of this framework to Hugging Face format")
    p.add_argument("--model_choice", type=str, default=default_model_choice)
    p.add_argument("--om_checkpoint_dir", type=str, required=True)
    p.add_argument("--hf_checkpoint_dir", type=str, default="checkpoint_hf")
    p.add_argument("--tokenizer_dir", type=str, default=None, help="directory whose tokenizer files are copied")
    p.add_argument("--cached", action="store_true", help="input is a cached model directory (model_<i>.pth)")
    p.add_argument("--use_init_empty_weights", action="store_true",
                   help="accepted for compatibility; no model is instantiated here")
    add_layout_arguments(p, pp=pp, ep=ep)
    args = p.parse_args(argv)
    print(args)
    assert config_utils.model_family(args.model_choice) == family, \
        f"--model_choice {args.model_choice} is not of the {family} family"
    om_checkpoint_to_hf(args.model_choice, args.om_checkpoint_dir, args.hf_checkpoint_dir,
                        pp=args.pipeline_parallelism, ep=args.expert_parallelism, tp=args.tensor_parallelism,
                        vpp=args.virtual_pipeline_parallelism, cached=args.cached, tokenizer_dir=args.tokenizer_dir)
