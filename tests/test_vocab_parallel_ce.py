"""Vocabulary-parallel LM head + cross entropy against the dense head and ``F.cross_entropy``."""
import pytest
import torch
import torch.nn.functional as F

from optimus_lm_b200.ops import functional as OF


def _dense(hidden, weight, labels):
    logits = hidden @ weight.t()
    V = logits.shape[-1]
    return F.cross_entropy(logits[:, :-1].reshape(-1, V), labels[:, 1:].reshape(-1))


def _worker(rank, world):
    import torch.distributed as dist
    from optimus_lm_b200.models.common.parallel_modules import VocabParallelLMHead
    torch.manual_seed(0)
    B, S, H, V = 2, 12, 32, 64
    full = torch.nn.Linear(H, V, bias=False)
    hidden0 = torch.randn(B, S, H)
    labels = torch.randint(0, V, (B, S))
    head = VocabParallelLMHead(H, V, tensor_parallelism=world, tp_ind=rank, group=dist.group.WORLD)
    head.set_parameters_from_full_module(full)
    h1 = hidden0.clone().requires_grad_()
    loss = head.loss(h1, labels)
    loss.backward()
    h2 = hidden0.clone().requires_grad_()
    want = _dense(h2, full.weight, labels)
    want.backward()
    assert torch.allclose(loss, want, atol=1e-5), (loss.item(), want.item())
    assert torch.allclose(h1.grad, h2.grad, atol=1e-5)
    lo = rank * (V // world)
    assert torch.allclose(head.weight.grad, full.weight.grad[lo:lo + V // world], atol=1e-5)


def test_vocab_parallel_head_matches_dense_head_two_ranks():
    from dist_utils import run_distributed
    run_distributed(_worker, 2)


def test_single_rank_and_ignored_rows():
    torch.manual_seed(1)
    logits = torch.randn(3, 7, 40, requires_grad=True)
    labels = torch.randint(0, 40, (3, 7))
    loss = OF.vocab_parallel_cross_entropy(logits, labels, 0, 40)
    want = F.cross_entropy(logits[:, :-1].reshape(-1, 40), labels[:, 1:].reshape(-1))
    assert torch.allclose(loss, want, atol=1e-6)
    g, = torch.autograd.grad(loss, logits)
    gw, = torch.autograd.grad(want, logits)
    assert torch.allclose(g, gw, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,V,shards", [(64, 1024, 2), (300, 50304, 4), (17, 264, 3)])
def test_kernels_on_vocabulary_slices(rows, V, shards):
    """The slice kernels on one GPU: statistics of every slice merged by hand give the full log-sum-exp, and every
    slice's gradient is the matching slice of the dense gradient."""
    from optimus_lm_b200.ops import extension
    C = extension()
    g = torch.Generator(device="cuda").manual_seed(5)
    logits = (torch.randn(rows, V, device="cuda", generator=g) * 3).to(torch.bfloat16)
    labels = torch.randint(0, V, (rows,), device="cuda", generator=g)
    labels[::7] = -100
    per = (V // shards) // 8 * 8
    bounds = [i * per for i in range(shards)] + [V]
    stats = []
    for i in range(shards):
        sl = logits[:, bounds[i]:bounds[i + 1]]
        if sl.data_ptr() % 16:
            sl = sl.contiguous()
        pm, ps, pt = (torch.empty(rows, dtype=torch.float32, device="cuda") for _ in range(3))
        C.ce_partial_fwd(sl, labels, bounds[i], pm, ps, pt)
        stats.append((pm, ps, pt))
    gmax = torch.stack([s[0] for s in stats]).max(dim=0).values
    ssum = sum(s[1] * torch.exp(s[0] - gmax) for s in stats)
    lse = gmax + torch.log(ssum)
    tgt = sum(s[2] for s in stats)
    lf = logits.float()
    assert torch.allclose(lse, torch.logsumexp(lf, dim=1), atol=2e-3, rtol=1e-4)
    valid = labels >= 0
    want_t = torch.where(valid, lf.gather(1, labels.clamp(min=0)[:, None])[:, 0], torch.zeros_like(lse))
    assert torch.equal(tgt, want_t)
    scale = torch.tensor([0.37], device="cuda")
    dense = torch.softmax(lf, dim=1)
    dense[valid.nonzero()[:, 0], labels[valid]] -= 1.0
    dense = dense * valid[:, None] * 0.37
    for i in range(shards):
        sl = logits[:, bounds[i]:bounds[i + 1]].contiguous()
        d = torch.empty_like(sl)
        C.ce_partial_bwd(sl, labels, bounds[i], V, lse, scale, d)
        assert torch.allclose(d.float(), dense[:, bounds[i]:bounds[i + 1]], atol=4e-3), i
    assert OF.check_status("cuda") == 0
