"""Single-GPU training-engine checks: kernel path against the plain PyTorch path, and the direct
weight-gradient stores against autograd's accumulate route."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from optimus_lm_b200.engine import EngineArgs, TrainEngine

MODEL = "allenai/OLMoE-1B-7B-0924--L2-SH0.125-SA0.25-SE0.125-SC0.25-SI0.5"   # d=256, 4 heads, 8 experts top-2, ffn 512


def _run(steps=4, gas=1, **kw):
    torch.manual_seed(0)
    args = EngineArgs(model_choice=MODEL, dtype="bf16", batch_size=2, context_size=256, optimizer="pgshard",
                      warmup_steps=0, lr=1e-3, opt_grad_acc_steps=gas, use_fast_moe=True, use_merged_mlp_in_fast_moe=True,
                      config_overrides={"output_router_logits": True}, **kw)
    eng = TrainEngine(args)
    g = torch.Generator().manual_seed(1)
    out = []
    for _ in range(steps * gas):
        ids = torch.randint(0, 50280, (2, 256), generator=g)
        o = eng.train_step(ids)
        out.append((float(o.loss), None if o.grad_norm is None else float(o.grad_norm)))
    assert eng.check_device_status() == 0
    flat = torch.cat([f.flat_param.float().cpu() for f in eng.optimizer.families])
    return out, flat, eng


@pytest.mark.parametrize("gas", [1, 2])
def test_direct_weight_gradients_match_autograd_accumulation(gas):
    a, pa, ea = _run(gas=gas, use_direct_grads=True)
    b, pb, eb = _run(gas=gas, use_direct_grads=False)
    assert len(ea.optimizer._direct) > 0 and not getattr(eb.optimizer, "_direct", None)
    for (la, ga), (lb, gb) in zip(a, b):
        assert abs(la - lb) < 2e-3, (a, b)
        if ga is not None:
            assert abs(ga - gb) <= 2e-2 * max(1.0, abs(gb)), (a, b)
    # Weights after the same steps.  One micro-batch per step: bit-identical gradients.  Two: the GEMM adds the
    # second gradient in fp32 and rounds once, autograd rounds each and their sum; early AdamW steps turn such a
    # last-bit difference of a near-zero gradient into a full +-lr move, so compare the bulk, not the maximum.
    d = (pa - pb).abs()
    if gas == 1:
        assert d.max().item() < 2e-3
    else:
        assert d.mean().item() < 1e-4 and d.max().item() < 1e-2


def test_loss_decreases_on_a_repeated_batch():
    torch.manual_seed(0)
    args = EngineArgs(model_choice=MODEL, dtype="bf16", batch_size=2, context_size=256, optimizer="unsharded",
                      warmup_steps=0, lr=2e-3)
    eng = TrainEngine(args)
    ids = torch.randint(0, 50280, (2, 256))
    losses = [float(eng.train_step(ids).loss) for _ in range(8)]
    assert losses[-1] < losses[0] - 0.5, losses
    assert eng.check_device_status() == 0


FAMILIES = [
    ("allenai/OLMo-1B-hf--L2", dict(optimizer="shard")),
    ("meta-llama/Llama-3.2-1B--L2", dict(optimizer="shard")),
    ("deepseek-ai/DeepSeek-V3--L3-DL1-N16-K4-MI512-A16-SE1-H1024-I2048",
     dict(optimizer="pgshard", use_fast_moe=True, use_merged_mlp_in_fast_moe=True)),
]


@pytest.mark.parametrize("model,kw", FAMILIES, ids=["olmo", "llama", "deepseek_v3"])
def test_other_families_train_on_the_kernel_path(model, kw, monkeypatch):
    """OLMo, Llama and DeepSeek-V3 (no QK-norm between projection and RoPE, MLA's partial interleaved RoPE) step
    through the kernels, and their first loss equals the plain PyTorch path's on the same weights and batch."""
    def first_losses(n):
        torch.manual_seed(0)
        eng = TrainEngine(EngineArgs(model_choice=model, dtype="bf16", batch_size=2, context_size=512, warmup_steps=0,
                                     lr=1e-3, seed=0, **kw))
        g = torch.Generator().manual_seed(5)
        ids = torch.randint(0, 32000, (2, 512), generator=g)
        out = [float(eng.train_step(ids).loss) for _ in range(n)]
        assert eng.check_device_status() == 0
        del eng
        torch.cuda.empty_cache()
        return out

    ker = first_losses(4)
    monkeypatch.setenv("OLB_DISABLE_KERNELS", "1")
    ref = first_losses(1)
    assert abs(ker[0] - ref[0]) < 3e-2, (ker, ref)
    assert ker[-1] < ker[0] - 0.3, ker


def test_updates_under_the_backward_match_the_plain_step():
    """AdamW of a finished layer on a side stream during the backward (clipping inactive) against the same updates
    all done in ``step``: same parameters bit for bit, same gradient norm up to summation order."""
    def run(early):
        torch.manual_seed(0)
        eng = TrainEngine(EngineArgs(model_choice=MODEL, dtype="bf16", batch_size=2, context_size=256, optimizer="pgshard",
                                     warmup_steps=100, lr=1e-3, use_fast_moe=True, use_merged_mlp_in_fast_moe=True,
                                     use_early_updates=early, config_overrides={"output_router_logits": True}))
        assert eng._early == early
        g = torch.Generator().manual_seed(1)
        out = []
        for _ in range(4):
            o = eng.train_step(torch.randint(0, 50280, (2, 256), generator=g))
            out.append((float(o.loss), float(o.grad_norm)))
        assert eng.check_device_status() == 0
        return out, torch.cat([f.flat_param.float().cpu() for f in eng.optimizer.families])

    a, pa = run(True)
    b, pb = run(False)
    assert torch.equal(pa, pb)
    for (la, na), (lb, nb) in zip(a, b):
        assert la == lb and abs(na - nb) <= 1e-4 * abs(nb), (a, b)


def test_per_expert_fast_path_matches_merged_weights():
    """``--use_fast_moe`` without merged weights stacks the experts' parameters and runs the same grouped GEMMs: the
    same losses as the merged layout (initial values depend on a tensor's serial name only)."""
    def run(merged):
        torch.manual_seed(0)
        eng = TrainEngine(EngineArgs(model_choice=MODEL, dtype="bf16", batch_size=2, context_size=256, optimizer="pgshard",
                                     warmup_steps=100, lr=1e-3, use_fast_moe=True, use_merged_mlp_in_fast_moe=merged,
                                     config_overrides={"output_router_logits": True}))
        g = torch.Generator().manual_seed(1)
        out = [float(eng.train_step(torch.randint(0, 50280, (2, 256), generator=g)).loss) for _ in range(4)]
        assert eng.check_device_status() == 0
        return out

    a, b = run(False), run(True)
    assert all(abs(x - y) < 2e-2 for x, y in zip(a, b)), (a, b)
