"""Training engine: the public entry point that builds a model + optimizer for a parallel
layout and runs training steps.

``TrainEngine`` packages what the reference's ``dist_train.py`` does inline (pmap -> config ->
model -> optimizer -> trainer -> step loop, dist_train.py:278-589, 739-923) so that the driver,
the benchmark and the tests share one code path:

    engine = TrainEngine(EngineArgs(model_choice="allenai/OLMoE-1B-7B-0924", expert_parallelism=8, ...))
    out = engine.train_step(input_ids)        # pinned host (or device) int tensor [B, S]
    out.loss, out.grad_norm

One step = host->device copy of the tokens (non-blocking, from pinned memory), forward,
backward (through the pipeline schedule when PP > 1), optimizer step every
``opt_grad_acc_steps`` steps, ``zero_grad``.  Nothing in the step synchronises the host with
the device; the loss and the gradient norm are returned as device tensors.
"""
from __future__ import annotations

import dataclasses
import math
import os
from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.distributed as dist
from torch import nn

from . import config_utils
from .mapper import ParallelDpPpEpTpMapper
from .optimizers import OPTIMIZER_CLASSES
from .utils import no_init_weights


@dataclass
class EngineArgs:
    model_choice: str = "allenai/OLMoE-1B-7B-0924"
    dtype: str = "bf16"
    data_parallelism: Optional[int] = None
    pipeline_parallelism: int = 1
    virtual_pipeline_parallelism: int = 1
    expert_parallelism: int = 1
    tensor_parallelism: int = 1
    use_pp_first: bool = False
    pp_scheme: str = "1f1b"
    reuse_buffers_in_1f1b: bool = False
    use_latest_trainer: bool = False
    batch_size: int = 1
    micro_batch_size: Optional[int] = None
    context_size: int = 4096
    optimizer: str = "unsharded"          # unsharded | shard | pgshard | subshard | pgsubshard
    lr: float = 4e-4
    min_lr: float = 4e-5
    weight_decay: float = 0.1
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    warmup_steps: int = 2500
    opt_grad_acc_steps: int = 1
    opt_disable_delayed_grad_clipping: bool = False
    opt_use_allreduce_for_grad_acc: bool = False
    opt_use_allreduce_for_param_gather: bool = False
    opt_use_chunked_allreduce: bool = False
    use_fused_optimizer: bool = True
    use_activation_checkpointing: bool = False
    activation_checkpointing_level: int = 0
    use_fast_moe: bool = True
    use_merged_mlp_in_fast_moe: bool = True
    force_uniform_routing: bool = False
    use_local_router_aux_loss: bool = False
    use_fused_ep_alltoall: bool = True
    skip_optimizer_step: bool = False
    skip_optimizer_step_weight_update: bool = False
    skip_backward_pass: bool = False
    disable_optimizer_state_checkpointing: bool = False
    init_std: Optional[float] = None      # None -> config.initializer_range
    seed: int = 0
    config_overrides: dict = field(default_factory=dict)


@dataclass
class StepOutput:
    loss: Optional[torch.Tensor]
    grad_norm: Optional[torch.Tensor]
    did_optimizer_step: bool


def build_model(model_choice: str, pmap, *, dtype=torch.bfloat16, device="cpu", memory_tracker=None,
                config_overrides=None, **parallel_kwargs):
    """Construct (config, model) for ``model_choice`` on ``device`` with uninitialised weights."""
    cfg = config_utils.build_config(model_choice, **parallel_kwargs)
    for k, v in (config_overrides or {}).items():
        setattr(cfg, k, v)
    cfg.check_compatibility()
    fam = config_utils.model_family(model_choice)
    if fam == "olmoe":
        from .models.olmoe.modeling_olmoe import OlmoeParallelForCausalLM as M
    elif fam == "olmo":
        from .models.olmo.modeling_olmo import OlmoParallelForCausalLM as M
    elif fam == "llama":
        from .models.llama.modeling_llama import LlamaParallelForCausalLM as M
    else:
        from .models.deepseek_v3.modeling_deepseek_v3 import DeepseekV3ParallelForCausalLM as M
    prev = torch.get_default_dtype()
    try:
        torch.set_default_dtype(dtype)
        with no_init_weights(), torch.device(device):
            try:
                model = M(cfg, pmap=pmap, memory_tracker=memory_tracker)
            except TypeError:
                model = M(cfg, pmap=pmap)
    finally:
        torch.set_default_dtype(prev)
    return cfg, model


@torch.no_grad()
def init_weights(model: nn.Module, std: float, seed: int = 0):
    """Random initialisation in the style of the reference generators
    (generate_serial_model.py:118-158): Linear / Embedding / merged expert weights ~ N(0, std),
    padding row of the embedding zeroed, norm weights = 1.  The generator is seeded per
    parameter name, so a parameter gets the same values whatever rank builds it."""
    import re
    import zlib

    inner = getattr(model, "model", model)
    pmap = getattr(model, "pmap", None)
    tp = pmap.tensor_parallelism if pmap is not None else 1
    tp_ind = pmap.tp_ind if pmap is not None else 0

    def global_layer(l: int) -> int:
        if hasattr(inner, "global_layer_index"):
            return inner.global_layer_index(l)
        if hasattr(inner, "layer_ids"):
            return inner.layer_ids[l]
        return getattr(inner, "layer_start_idx", 0) + l

    def fill(t, key, shape=None):
        """N(0, std) values determined by ``key`` alone (independent of the rank that draws them)."""
        g = torch.Generator(device=t.device)
        g.manual_seed((seed * 1000003 + zlib.crc32(key.encode())) % (2 ** 63))
        shape = tuple(t.shape) if shape is None else shape
        n = 1
        for d in shape:
            n *= d
        if shape == tuple(t.shape) and n > (1 << 28):
            flat = t.view(-1)  # big tensors: fp32 pieces bound the temporary
            step = 1 << 26
            for s in range(0, n, step):
                e = min(s + step, n)
                flat[s:e].copy_(torch.randn(e - s, device=t.device, dtype=torch.float32, generator=g) * std)
            return None
        full = torch.randn(shape, device=t.device, dtype=torch.float32, generator=g) * std
        if shape == tuple(t.shape):
            t.copy_(full)
            return None
        return full

    modules = dict(model.named_modules())
    for name, p in model.named_parameters():
        if p.dim() == 1 and ("norm" in name or "layernorm" in name):
            p.fill_(1.0)
            continue
        # the seed key uses global layer / expert indices so that every parallel layout draws the
        # same model
        key = name
        m = re.match(r"^(.*layers\.)(\d+)(\..*)$", key)
        if m:
            key = f"{m.group(1)}{global_layer(int(m.group(2)))}{m.group(3)}"
        owner = modules.get(name.rsplit(".", 1)[0])
        m = re.match(r"^(.*\.experts\.)(\d+)(\..*)$", key)
        if m:
            block = modules.get(name.split(".experts.")[0])
            e0 = getattr(block, "expert_start_idx", 0)
            key = f"{m.group(1)}{e0 + int(m.group(2))}{m.group(3)}"
            fill(p, key)
        elif name.endswith("_merged_weight"):
            block = modules.get(name.split(".experts.")[0])
            e0 = getattr(block, "expert_start_idx", 0)
            proj = name.rsplit(".", 1)[1].replace("_merged_weight", "")
            base = key.rsplit(".", 1)[0]
            for le in range(p.shape[0]):
                fill(p[le], f"{base}.{e0 + le}.{proj}.weight")
        elif tp > 1 and owner is not None and hasattr(owner, "intermediate_size_per_rank") is False and \
                type(owner).__name__ in ("ParallelEmbedding", "ParallelLMHead"):
            if type(owner).__name__ == "ParallelEmbedding":
                full = fill(p, key, (owner.vocab_size_padded, p.shape[1]))
                full[owner.vocab_size:].zero_()
                p.copy_(full[owner.start_embedding_id:owner.end_embedding_id])
            else:
                full = fill(p, key, (p.shape[0], p.shape[1] * tp))
                p.copy_(full[:, tp_ind * p.shape[1]:(tp_ind + 1) * p.shape[1]])
        elif tp > 1 and p.dim() == 2 and re.search(r"\.(q|k|v|gate|up)_proj\.weight$", name):
            full = fill(p, key, (p.shape[0] * tp, p.shape[1]))
            p.copy_(full[tp_ind * p.shape[0]:(tp_ind + 1) * p.shape[0]])
        elif tp > 1 and p.dim() == 2 and re.search(r"\.(o|down)_proj\.weight$", name):
            full = fill(p, key, (p.shape[0], p.shape[1] * tp))
            p.copy_(full[:, tp_ind * p.shape[1]:(tp_ind + 1) * p.shape[1]])
        elif owner is not None and getattr(owner, "pmap", None) is not None and hasattr(owner, "intermediate_size_per_rank") \
                and owner.intermediate_size_per_rank != owner.intermediate_size and tp == 1:
            # DeepSeek-V3 dense MLP: intermediate dimension sharded over the EP group
            ep, ei = owner.pmap.expert_parallelism, owner.pmap.ep_ind
            if name.endswith("down_proj.weight"):
                full = fill(p, key, (p.shape[0], p.shape[1] * ep))
                p.copy_(full[:, ei * p.shape[1]:(ei + 1) * p.shape[1]])
            else:
                full = fill(p, key, (p.shape[0] * ep, p.shape[1]))
                p.copy_(full[ei * p.shape[0]:(ei + 1) * p.shape[0]])
        else:
            fill(p, key)
    for mod in model.modules():
        if isinstance(mod, nn.Embedding) and mod.padding_idx is not None:
            mod.weight[mod.padding_idx].zero_()
    for name, b in model.named_buffers():
        if name.endswith("e_score_correction_bias"):
            b.zero_()


def get_learning_rate(step_id, train_steps, args):
    """Linear warm-up from ``min_lr`` then constant / cosine / linear decay, as a function of the
    optimizer step ``step_id // opt_grad_acc_steps`` (reference dist_train.py:53-78)."""
    gas = args.opt_grad_acc_steps
    opt_step = step_id // gas
    total = (train_steps if getattr(args, "lr_train_steps", None) is None else args.lr_train_steps) // gas
    if opt_step < args.warmup_steps:
        return args.min_lr + (args.lr - args.min_lr) * opt_step / float(max(1, args.warmup_steps))
    schedule = getattr(args, "lr_schedule", "cosine")
    if schedule == "constant":
        return args.lr
    ratio = (opt_step - args.warmup_steps) / (total - args.warmup_steps)
    if schedule == "cosine":
        coeff = 0.5 * (1.0 + math.cos(math.pi * ratio))
    elif schedule == "linear":
        coeff = 1.0 - ratio
    else:
        raise ValueError(f"Invalid learning rate schedule: {schedule}. Choose 'constant', 'cosine' or 'linear'.")
    return args.min_lr + coeff * (args.lr - args.min_lr)


class TrainEngine:
    def __init__(self, args: EngineArgs, pmap: Optional[ParallelDpPpEpTpMapper] = None, model=None, config=None,
                 device=None):
        self.args = args
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        if args.micro_batch_size is None:
            args.micro_batch_size = args.batch_size
        if pmap is None:
            mp = args.pipeline_parallelism * args.expert_parallelism * args.tensor_parallelism
            dp = args.data_parallelism if args.data_parallelism is not None else max(1, world // mp)
            assert dp * mp == world, f"DP {dp} x PP x EP x TP {mp} != world size {world}"
            pmap = ParallelDpPpEpTpMapper(dp, args.pipeline_parallelism, args.expert_parallelism,
                                          args.tensor_parallelism, rank=rank, create_groups=dist.is_initialized(),
                                          use_pp_first=args.use_pp_first)
        self.pmap = pmap
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.dtype = torch.bfloat16 if args.dtype in ("bf16", "bfloat16") else torch.float32

        if model is None:
            config, model = build_model(
                args.model_choice, pmap, dtype=self.dtype, device=self.device,
                config_overrides=args.config_overrides,
                pipeline_parallelism=args.pipeline_parallelism, expert_parallelism=args.expert_parallelism,
                tensor_parallelism=args.tensor_parallelism,
                virtual_pipeline_parallelism=args.virtual_pipeline_parallelism,
                use_local_router_aux_loss=args.use_local_router_aux_loss,
                use_activation_checkpointing=args.use_activation_checkpointing,
                activation_checkpointing_level=args.activation_checkpointing_level,
                use_fast_moe=args.use_fast_moe, use_merged_mlp_in_fast_moe=args.use_merged_mlp_in_fast_moe,
                force_uniform_routing=args.force_uniform_routing, use_fused_ep_alltoall=args.use_fused_ep_alltoall)
            std = args.init_std if args.init_std is not None else getattr(config, "initializer_range", 0.02)
            init_weights(model, std, args.seed)
        self.config, self.model = config, model
        self.model.to(self.device)
        self.optimizer = self._build_optimizer()
        self.trainer = self._build_trainer()
        self.step_id = 0
        self._staging = None

    # ------------------------------------------------------------------ construction
    def _build_optimizer(self):
        a, p = self.args, self.pmap
        cls = OPTIMIZER_CLASSES[a.optimizer]
        kwargs = dict(lr=a.lr, betas=(a.beta1, a.beta2), eps=a.eps, weight_decay=a.weight_decay,
                      warmup_steps=a.warmup_steps, dtype=self.dtype, device=self.device,
                      num_shards=p.data_parallelism, shard_id=p.dp_ind, group=p.dp_group,
                      opt_disable_delayed_grad_clipping=a.opt_disable_delayed_grad_clipping,
                      tensor_parallelism=p.tensor_parallelism, tp_ind=p.tp_ind, tp_group=p.tp_group,
                      expert_parallelism=p.expert_parallelism, ep_ind=p.ep_ind, ep_group=p.ep_group,
                      dpep_ind=p.dpep_ind, dpep_group=p.dpep_group, skip_optimizer_step=a.skip_optimizer_step,
                      opt_use_chunked_allreduce=a.opt_use_chunked_allreduce)
        if a.optimizer != "unsharded":
            kwargs.update(opt_use_allreduce_for_grad_acc=a.opt_use_allreduce_for_grad_acc,
                          opt_use_allreduce_for_param_gather=a.opt_use_allreduce_for_param_gather,
                          disable_optimizer_state_checkpointing=a.disable_optimizer_state_checkpointing,
                          skip_optimizer_step_weight_update=a.skip_optimizer_step_weight_update)
        opt = cls(self.model.parameters(), self.model, **kwargs)
        opt.pmap, opt.config = p, self.config
        if a.use_fused_optimizer and self.device.type == "cuda" and dist.is_initialized() and a.optimizer != "unsharded":
            try:
                from .parallel.fused_optimizer import FusedShardedStep
                opt._fused = FusedShardedStep.try_create(opt)
            except ImportError:
                opt._fused = None
        return opt

    def _build_trainer(self):
        a, p = self.args, self.pmap
        if p.pipeline_parallelism == 1:
            return None
        if a.use_latest_trainer or a.virtual_pipeline_parallelism > 1:
            from .trainer import ParallelTrainer
        else:
            from .training import ParallelTrainer
        return ParallelTrainer(self.config, self.model, p, a.batch_size, a.micro_batch_size, a.context_size,
                               a.opt_grad_acc_steps, self.dtype, self.device, pp_scheme=a.pp_scheme,
                               reuse_buffers_in_1f1b=a.reuse_buffers_in_1f1b)

    # ------------------------------------------------------------------ stepping
    def set_lr(self, lr: float):
        self.optimizer.param_groups[0]["lr"] = lr

    def stage_inputs(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Copy a host batch to the device (asynchronously when it is pinned)."""
        if input_ids.device == self.device:
            return input_ids.long() if input_ids.dtype != torch.long else input_ids
        return input_ids.to(self.device, non_blocking=True).long()

    def forward_backward(self, input_ids: torch.Tensor):
        a = self.args
        gas = a.opt_grad_acc_steps
        if self.trainer is not None:
            out = self.trainer.step(input_ids, input_ids, only_forward=a.skip_backward_pass)
            return out.loss
        out = self.model(input_ids, labels=input_ids)
        loss = out.loss
        if not a.skip_backward_pass:
            (loss / gas if gas > 1 else loss).backward()
        return loss.detach()

    def train_step(self, input_ids: torch.Tensor) -> StepOutput:
        ids = self.stage_inputs(input_ids)
        loss = self.forward_backward(ids)
        grad_norm = None
        did = False
        if (self.step_id + 1) % self.args.opt_grad_acc_steps == 0 and not self.args.skip_backward_pass:
            grad_norm = self.optimizer.step()
            self.optimizer.zero_grad()
            did = True
        self.step_id += 1
        return StepOutput(loss, grad_norm, did)

    # ------------------------------------------------------------------ info
    def tokens_per_step(self) -> int:
        """Tokens consumed per step by the whole job (every DP x EP rank reads its own batch)."""
        p = self.pmap
        return self.args.batch_size * self.args.context_size * p.data_parallelism * p.expert_parallelism

    def check_device_status(self) -> int:
        if self.device.type != "cuda":
            return 0
        from .ops import functional as OF
        return OF.check_status(self.device)
