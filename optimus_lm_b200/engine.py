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
    optimizer: str = "unsharded"          # unsharded | shard | pgshard | subshard | pgsubshard | pt (torch.optim.AdamW)
    use_hf_model: bool = False            # the transformers implementation of the architecture (no model parallelism)
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
    use_direct_grads: bool = True         # weight-gradient GEMMs store into the flat gradient buffer themselves
    use_early_updates: bool = False       # AdamW of a finished layer runs under the backward of the layers before it
                                          # (measured neutral on a power-capped B200: 205.1 vs 205.0 ms/step)
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


def build_hf_model(model_choice: str, *, dtype=torch.bfloat16, device="cpu", config_overrides=None):
    """``--use_hf_model``: the ``transformers`` implementation of ``model_choice`` with the sizes of the model tag
    (reference dist_train.py:304-318).  The reference fetches the base configuration from the hub; here it is built from
    this package's own configuration of the architecture, so no network is needed.  Random initialisation as
    ``from_config`` does it; no pipeline, expert or tensor parallelism."""
    import transformers

    from .convert import hf_config_dict
    cfg = config_utils.build_config(model_choice)
    for k, v in (config_overrides or {}).items():
        setattr(cfg, k, v)
    d = hf_config_dict(model_choice, cfg, torch_dtype="bfloat16" if dtype == torch.bfloat16 else "float32")
    d = {k: v for k, v in d.items() if k not in ("architectures", "torch_dtype", "dtype", "transformers_version")}
    hf_cfg = transformers.AutoConfig.for_model(**d)
    hf_cfg.use_cache = False
    if getattr(cfg, "output_router_logits", False):
        hf_cfg.output_router_logits = True
    model = transformers.AutoModelForCausalLM.from_config(hf_cfg)
    return cfg, model.to(dtype).to(device)


@torch.no_grad()
def init_weights(model: nn.Module, std: float, seed: int = 0):
    """Random initialisation in the style of the reference generators
    (generate_serial_model.py:118-158): Linear / Embedding / merged expert weights ~ N(0, std),
    padding row of the embedding zeroed, norm weights = 1.  The generator is seeded per
    parameter name, so a parameter gets the same values whatever rank builds it."""
    from . import model_io

    device = next(model.parameters()).device

    def draw(serial_name, serial_shape):
        return model_io.seeded_serial_tensor(serial_name, serial_shape, std, seed, device=device)

    # every local parameter is cut out of its serial tensor, which is drawn from the serial name:
    # all parallel layouts (PP/VPP/EP/TP, merged or per-expert) therefore hold the same model
    model_io.fill_shard(model, draw)
    for mod in model.modules():
        if isinstance(mod, nn.Embedding) and mod.padding_idx is not None:
            mod.weight[mod.padding_idx].zero_()
        elif getattr(mod, "local_padding_idx", None) is not None:
            mod.weight[mod.local_padding_idx].zero_()
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

        if model is None and args.use_hf_model:
            assert args.pipeline_parallelism == args.expert_parallelism == args.tensor_parallelism == 1, \
                "Huggingface model does not support parallelism"
            config, model = build_hf_model(args.model_choice, dtype=self.dtype, device=self.device,
                                           config_overrides=args.config_overrides)
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
        self._setup_early_updates()

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
        if a.optimizer not in ("unsharded", "pt"):
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
        if a.use_direct_grads and self.device.type == "cuda" and self.dtype == torch.bfloat16 \
                and hasattr(opt, "enable_direct_grads"):
            opt.enable_direct_grads()
        return opt

    def _setup_early_updates(self):
        """Hook every decoder layer's input: when its gradient arrives, the layer's backward is complete and the
        optimizer may update that layer's parameters on a side stream (``optimizers.enable_early_updates``)."""
        a, opt = self.args, self.optimizer
        self._early = False
        layers = getattr(getattr(self.model, "model", None), "layers", None)
        if not (a.use_early_updates and os.environ.get("OLB_EARLY_UPDATES", "1") != "0" and self.device.type == "cuda" and self.trainer is None and layers is not None
                and hasattr(opt, "enable_early_updates") and not a.skip_backward_pass):
            return
        if opt.enable_early_updates([list(layer.parameters()) for layer in layers]) == 0:
            return
        self._early = True

        def pre_hook(idx):
            def hook(module, inputs):
                h = inputs[0] if inputs else None
                if opt._early_armed and torch.is_tensor(h) and h.requires_grad and torch.is_grad_enabled():
                    h.register_hook(lambda g, i=idx: opt.early_update_layer(i))
            return hook

        for i, layer in enumerate(layers):
            layer.register_forward_pre_hook(pre_hook(i))

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
        if self._early:
            self.optimizer.arm_early_updates((self.step_id + 1) % self.args.opt_grad_acc_steps == 0)
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
