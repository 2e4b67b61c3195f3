"""``ParallelTrainer`` with virtual pipeline stages: GPipe over chunks and interleaved 1F1B
(``--use_latest_trainer``).  Same constructor and ``step`` signature as the reference's
optimus/trainer.py:184-871.  ``python -m optimus_lm_b200.trainer`` runs the reference's self-test
(:897-998): a toy 16-layer Linear+ReLU model, PP = world size, VPP = 2, 1F1B, compared against a
serial forward/backward.
"""
from __future__ import annotations

import torch
from torch import nn

from .pipeline import ParallelTrainerOutput, PipelineExecutor  # noqa: F401
from .schedules import Interleaved1f1bBufferManager, _virtual_forward  # noqa: F401


def get_coord_info_from_flat_index(i, NG, VPP, NMBG, backward=False):
    """Flat slot index -> (micro-batch group, virtual stage, local micro-batch); the backward
    order visits the virtual stages from last to first (reference trainer.py:20-30)."""
    mb, vp = _virtual_forward(i, NMBG, VPP)
    mg, lmb = divmod(mb, NMBG)
    return mg, (VPP - 1 - vp if backward else vp), lmb


class ParallelTrainer(PipelineExecutor):
    pass


# ----------------------------------------------------------------------------- self-test model
class Config:
    def __init__(self, num_hidden_layers=16, hidden_size=64, pipeline_parallelism=1, virtual_pipeline_parallelism=1):
        self.num_hidden_layers = num_hidden_layers
        self.hidden_size = hidden_size
        self.vocab_size = hidden_size
        self.pipeline_parallelism = pipeline_parallelism
        self.virtual_pipeline_parallelism = virtual_pipeline_parallelism
        self.num_experts, self.num_experts_per_tok = 1, 1
        self.router_aux_loss_coef, self.output_router_logits, self.use_local_router_aux_loss = 0.0, False, False


class Model(nn.Module):
    """Toy stack of Linear+ReLU layers partitioned like the real models (round-robin chunks)."""

    def __init__(self, config, pmap):
        super().__init__()
        self.config, self.pmap = config, pmap
        PP, VPP = config.pipeline_parallelism, config.virtual_pipeline_parallelism
        per_rank = config.num_hidden_layers // PP
        self.LV = per_rank // VPP
        self.layer_ids = [(v * PP + pmap.pp_ind) * self.LV + l for v in range(VPP) for l in range(self.LV)]
        self.layers = nn.ModuleList([nn.Linear(config.hidden_size, config.hidden_size) for _ in self.layer_ids])
        for gid, layer in zip(self.layer_ids, self.layers):
            g = torch.Generator().manual_seed(1000 + gid)
            with torch.no_grad():
                layer.weight.copy_(torch.randn(layer.weight.shape, generator=g) / config.hidden_size ** 0.5)
                layer.bias.copy_(torch.randn(layer.bias.shape, generator=g) * 0.1)

    def forward(self, x, vp_ind=0):
        for l in range(vp_ind * self.LV, (vp_ind + 1) * self.LV):
            x = torch.relu(self.layers[l](x))
        return x


def self_test(pp_scheme="1f1b", VPP=2, NMB=None, device=None, verbose=True):
    """Pipeline vs serial on the toy model.  Returns (max |out err|, max |input-grad err|) on the
    ranks that own the respective tensors (else None)."""
    import torch.distributed as dist
    from .mapper import ParallelDpPpEpTpMapper
    rank, world = dist.get_rank(), dist.get_world_size()
    device = device or torch.device("cpu")
    PP = world
    NMB = NMB or 2 * PP
    MBS, S, H = 2, 4, 64
    cfg = Config(num_hidden_layers=2 * PP * VPP, hidden_size=H, pipeline_parallelism=PP, virtual_pipeline_parallelism=VPP)
    pmap = ParallelDpPpEpTpMapper(1, PP, 1, 1, rank=rank, create_groups=True)
    model = Model(cfg, pmap).to(device)
    trainer = ParallelTrainer(cfg, model, pmap, NMB * MBS, MBS, S, 1, torch.float32, device, pp_scheme=pp_scheme)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(NMB * MBS, S, H, generator=g).to(device)
    gout = torch.randn(NMB * MBS, S, H, generator=g).to(device)
    # the first stage feeds activations (not token ids): wrap them as a leaf to read the input gradient
    x_in = x.clone().requires_grad_(True)
    out = trainer.step(input=x_in if pmap.is_first_stage_rank else None, labels=None,
                       output_grad=gout if pmap.is_last_stage_rank else None, output_logits=True)
    # serial reference
    full = Config(num_hidden_layers=cfg.num_hidden_layers, hidden_size=H)
    serial = Model(full, ParallelDpPpEpTpMapper()).to(device)
    xs = x.clone().requires_grad_(True)
    ys = serial(xs)
    ys.backward(gout)
    out_err = (out.logits - ys).abs().max().item() if pmap.is_last_stage_rank else None
    grad_err = (x_in.grad - xs.grad).abs().max().item() if pmap.is_first_stage_rank else None
    if verbose:
        print(f"rank {rank}: out err {out_err}, input grad err {grad_err}", flush=True)
    return out_err, grad_err


if __name__ == "__main__":
    from .dutils import setup_distributed
    setup_distributed("gloo" if not torch.cuda.is_available() else "nccl")
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    self_test(device=dev)
