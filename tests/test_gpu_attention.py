"""Flash-attention kernels against an fp32 eager reference of the same op."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from optimus_lm_b200.ops import functional as OF
from optimus_lm_b200.ops import attention as OA


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _mk(B, S, Hq, Hkv, D, Dv, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(B, S, Hq, D, device="cuda", generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, device="cuda", generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, Dv, device="cuda", generator=g).to(torch.bfloat16)
    return q, k, v


@pytest.mark.parametrize("B,S,Hq,Hkv,D,Dv", [(1, 128, 1, 1, 128, 128), (2, 512, 4, 4, 128, 128), (1, 1024, 4, 2, 128, 128),
                                             (2, 384, 2, 2, 64, 64), (1, 512, 4, 4, 192, 128)])
def test_flash_attention_forward(B, S, Hq, Hkv, D, Dv):
    q, k, v = _mk(B, S, Hq, Hkv, D, Dv)
    scale = D ** -0.5
    o = OA.flash_attention(q, k, v, scale=scale)
    ref = OF.attention_reference(q.float(), k.float(), v.float(), scale, True)
    assert _rel(o, ref) < 2e-2, _rel(o, ref)
    assert OF.check_status("cuda") == 0


@pytest.mark.parametrize("B,S,Hq,Hkv,D,Dv", [(1, 256, 1, 1, 128, 128), (2, 2048, 4, 2, 128, 128), (1, 1280, 2, 2, 64, 64),
                                             (1, 768, 2, 2, 192, 128)])
def test_flash_attention_forward_two_tile_kernel(B, S, Hq, Hkv, D, Dv):
    # the kernel with two query tiles per CTA against the fp32 oracle (element-wise as well as in norm) and against
    # the single-tile kernel, output and log-sum-exp; long sequences wrap the K/V ring several times
    q, k, v = _mk(B, S, Hq, Hkv, D, Dv, seed=7)
    scale = D ** -0.5
    C = OF.extension()
    outs = []
    for variant in (1, 2):
        o = torch.empty(B, S, Hq, Dv, dtype=torch.bfloat16, device="cuda")
        lse = torch.empty(B, Hq, S, dtype=torch.float32, device="cuda")
        C.attn_fwd(q, k, v, o, lse, scale, OF.status_word("cuda"), variant)
        outs.append((o, lse))
    assert OF.check_status("cuda") == 0
    ref = OF.attention_reference(q.float(), k.float(), v.float(), scale, True)
    o2, lse2 = outs[1]
    assert _rel(o2, ref) < 2e-2, _rel(o2, ref)
    assert (o2.float() - ref).abs().max().item() < 4e-2
    assert (o2.float() - outs[0][0].float()).abs().max().item() < 2e-2
    assert (lse2 - outs[0][1]).abs().max().item() < 1e-3


def test_flash_attention_strided_views_and_lse():
    # q/k/v as slices of wider tensors (the MLA layout) and the saved log-sum-exp
    B, S, H = 1, 256, 2
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(B, S, H, 3 * 128, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v = qkv[..., :128], qkv[..., 128:256], qkv[..., 256:]
    C = OF.extension()
    o = torch.empty(B, S, H, 128, dtype=torch.bfloat16, device="cuda")
    lse = torch.empty(B, H, S, dtype=torch.float32, device="cuda")
    C.attn_fwd(q, k, v, o, lse, 128 ** -0.5, OF.status_word("cuda"))
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * 128 ** -0.5
    s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    assert _rel(lse, torch.logsumexp(s, -1)) < 1e-3
    ref = torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v.float())
    assert _rel(o, ref) < 2e-2
    assert OF.check_status("cuda") == 0


@pytest.mark.parametrize("B,S,Hq,Hkv,D,Dv", [(1, 128, 1, 1, 128, 128), (1, 256, 2, 2, 128, 128), (1, 512, 4, 2, 128, 128),
                                             (2, 1024, 2, 2, 128, 128), (1, 384, 2, 2, 64, 64), (1, 256, 2, 2, 192, 128),
                                             (1, 640, 3, 3, 192, 128)])
def test_flash_attention_backward(B, S, Hq, Hkv, D, Dv):
    from optimus_lm_b200.ops._ext import extension
    assert hasattr(extension(), "attn_bwd"), "backward kernels are not in the built extension"
    q, k, v = _mk(B, S, Hq, Hkv, D, Dv, seed=1)
    scale = D ** -0.5
    g = torch.Generator(device="cuda").manual_seed(9)
    do = torch.randn(B, S, Hq, Dv, device="cuda", generator=g).to(torch.bfloat16)
    qa, ka, va = (t.clone().requires_grad_() for t in (q, k, v))
    OA.flash_attention(qa, ka, va, scale=scale).backward(do)
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    OF.attention_reference(qr, kr, vr, scale, True).backward(do.float())
    assert _rel(qa.grad, qr.grad) < 3e-2 and _rel(ka.grad, kr.grad) < 3e-2 and _rel(va.grad, vr.grad) < 3e-2
    assert OF.check_status("cuda") == 0


def test_flash_attention_backward_strided_and_deterministic():
    # q / k / v / dO as slices of wider tensors; two runs must agree bit for bit (single writer per element)
    B, S, H, D = 1, 512, 2, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    big = torch.randn(B, S, H, 3 * D + 64, device="cuda", generator=g).to(torch.bfloat16)
    q, k, v = big[..., :D], big[..., D:2 * D], big[..., 2 * D + 64:3 * D + 64]
    do_big = torch.randn(B, S, H, 2 * D, device="cuda", generator=g).to(torch.bfloat16)
    do = do_big[..., D:]
    grads = []
    for _ in range(2):
        qa, ka, va = (t.detach().clone().requires_grad_() for t in (q, k, v))
        # keep the strided layout: operate on views of a leaf
        leaf = big.detach().clone().requires_grad_()
        o = OA.flash_attention(leaf[..., :D], leaf[..., D:2 * D], leaf[..., 2 * D + 64:3 * D + 64])
        o.backward(do)
        grads.append(leaf.grad.clone())
    assert torch.equal(grads[0], grads[1])
    ref = big.float().detach().requires_grad_()
    OF.attention_reference(ref[..., :D], ref[..., D:2 * D], ref[..., 2 * D + 64:3 * D + 64], D ** -0.5, True).backward(do.float())
    assert _rel(grads[0], ref.grad) < 3e-2
    assert OF.check_status("cuda") == 0
