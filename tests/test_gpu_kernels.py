"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from optimus_lm_b200.ops import functional as OF


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    assert OF.check_status("cuda") == 0, "a kernel reported a timeout / overflow in the status word"


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (384, 128, 512), (1000, 264, 200),
                                   (4096, 2048, 2048), (300, 64, 128), (128, 8, 256)])
def test_gemm_nt(M, N, K):
    a, b = bf(M, K, seed=1), bf(N, K, seed=2)
    c = OF.gemm(a, b, M, N, K)
    ref = a.float() @ b.float().t()
    assert rel_err(c, ref) < 1e-2


@pytest.mark.parametrize("block_n", [64, 128, 256])
def test_gemm_block_n(block_n):
    M, N, K = 512, 512, 320
    a, b = bf(M, K, seed=1), bf(N, K, seed=2)
    c = OF.gemm(a, b, M, N, K, block_n=block_n)
    assert rel_err(c, a.float() @ b.float().t()) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (512, 320, 192), (2048, 1024, 2048)])
def test_gemm_nn_dgrad(M, N, K):
    # dX[M,N] = dY[M,K] @ W[K,N]  (B is MN-major)
    a, w = bf(M, K, seed=3), bf(K, N, seed=4)
    c = OF.gemm(a, w, M, N, K, b_mn_major=True)
    assert rel_err(c, a.float() @ w.float()) < 1e-2


@pytest.mark.parametrize("M,N,K", [(256, 256, 256), (320, 512, 1000), (1024, 2048, 4096)])
def test_gemm_tn_wgrad(M, N, K):
    # dW[M,N] = dY[K,M]^T @ X[K,N]  (both MN-major)
    dy, x = bf(K, M, seed=5), bf(K, N, seed=6)
    c = OF.gemm(dy, x, M, N, K, a_mn_major=True, b_mn_major=True)
    assert rel_err(c, dy.float().t() @ x.float()) < 1e-2


def test_gemm_accumulate_and_fp32_out():
    M, N, K = 256, 256, 128
    a, b = bf(M, K, seed=1), bf(N, K, seed=2)
    c0 = bf(M, N, seed=7)
    c = c0.clone()
    OF.gemm(a, b, M, N, K, out=c, accumulate=True)
    assert rel_err(c, c0.float() + a.float() @ b.float().t()) < 1e-2
    c32 = OF.gemm(a, b, M, N, K, out_dtype=torch.float32)
    assert rel_err(c32, a.float() @ b.float().t()) < 1e-5
    # strided output (columns of a wider buffer)
    wide = torch.zeros(M, 2 * N, dtype=torch.bfloat16, device="cuda")
    OF.gemm(a, b, M, N, K, out=wide[:, N:])
    assert rel_err(wide[:, N:], a.float() @ b.float().t()) < 1e-2
    assert wide[:, :N].abs().max().item() == 0


def test_linear_autograd():
    x = bf(4, 96, 256, seed=1).requires_grad_()
    w = bf(512, 256, seed=2, scale=0.05).requires_grad_()
    y = OF.linear(x, w)
    g = bf(4, 96, 512, seed=3)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = F.linear(xr, wr)
    yr.backward(g.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(x.grad, xr.grad) < 1e-2 and rel_err(w.grad, wr.grad) < 1e-2


# ------------------------------------------------------------------ grouped GEMM + MoE
def _routing(T, E, K, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    logits = torch.randn(T, E, device="cuda", generator=g)
    w, idx = torch.topk(torch.softmax(logits, -1), K, dim=-1)
    return w.float().contiguous(), idx.to(torch.int32).contiguous()


@pytest.mark.parametrize("T,E,K,e_start,E_loc", [(300, 8, 2, 0, 8), (1024, 64, 8, 0, 64), (515, 16, 4, 8, 8),
                                                 (64, 8, 2, 0, 8)])
def test_moe_index(T, E, K, e_start, E_loc):
    _, idx = _routing(T, E, K)
    cap = OF.moe_capacity_rows(T, K, E_loc)
    ix = OF.MoEIndex(idx, e_start, E_loc, cap)
    torch.cuda.synchronize()
    row_of, src_of, k_of = ix.row_of.cpu(), ix.src_of.cpu(), ix.k_of.cpu()
    offs, counts, meta = ix.offsets.cpu(), ix.counts.cpu(), ix.meta.cpu()
    idx_c = idx.cpu()
    for le in range(E_loc):
        assert counts[le].item() == (idx_c == e_start + le).sum().item()
        assert offs[le].item() % OF.ROW_PAD == 0
        assert offs[le + 1].item() - offs[le].item() == -(-counts[le].item() // OF.ROW_PAD) * OF.ROW_PAD
    assert meta[0].item() * 128 == offs[E_loc].item()
    for i in range(meta[0].item()):
        e = meta[1 + i].item()
        assert offs[e] <= i * 128 < offs[e + 1]
    local = (idx_c >= e_start) & (idx_c < e_start + E_loc)
    assert ((row_of >= 0) == local).all()
    t_ids, k_ids = torch.where(local)
    rows = row_of[t_ids, k_ids].long()
    assert rows.unique().numel() == rows.numel()
    assert (src_of[rows] == t_ids.int()).all() and (k_of[rows] == k_ids.int()).all()
    e_of_row = idx_c[t_ids, k_ids].long() - e_start
    assert ((rows >= offs[e_of_row]) & (rows < offs[e_of_row] + counts[e_of_row])).all()
    used = torch.zeros(cap, dtype=torch.bool)
    used[rows] = True
    assert (src_of[~used] == -1).all()
    # deterministic
    ix2 = OF.MoEIndex(idx, e_start, E_loc, cap)
    assert torch.equal(ix2.row_of, ix.row_of)


def test_grouped_gemms():
    T, E, K, H, I = 700, 8, 2, 256, 512
    _, idx = _routing(T, E, K)
    cap = OF.moe_capacity_rows(T, K, E)
    ix = OF.MoEIndex(idx, 0, E, cap)
    x = bf(T, H, seed=1)
    w = bf(E, I, H, seed=2, scale=0.05)
    C = OF.extension()
    xp = torch.empty(cap, H, dtype=torch.bfloat16, device="cuda")
    C.moe_gather_rows(x, ix.src_of, ix.meta, xp)
    nrows = ix.meta[0].item() * 128
    src = ix.src_of[:nrows].long()
    ref_xp = torch.where(src[:, None] >= 0, x[src.clamp(min=0)].float(), torch.zeros(1, device="cuda"))
    assert torch.equal(xp[:nrows].float(), ref_xp)
    y = OF.grouped_linear_fwd(xp, w, ix)
    offs = ix.offsets.cpu().tolist()
    for e in range(E):
        a, b = offs[e], offs[e + 1]
        if b > a:
            assert rel_err(y[a:b], xp[a:b].float() @ w[e].float().t()) < 1e-2
    dy = bf(cap, I, seed=3)
    dy[nrows:] = 0
    dy[:nrows][src < 0] = 0
    dx = OF.grouped_linear_dgrad(dy, w, ix)
    dw = OF.grouped_linear_wgrad(dy, xp, ix, I, H)
    for e in range(E):
        a, b = offs[e], offs[e + 1]
        if b > a:
            assert rel_err(dx[a:b], dy[a:b].float() @ w[e].float()) < 1e-2
            assert rel_err(dw[e], dy[a:b].float().t() @ xp[a:b].float()) < 1e-2
        else:
            assert dw[e].abs().max().item() == 0
    # gate and up input gradients in one launch: K-concatenated B operand
    w2 = bf(E, I, H, seed=4, scale=0.05)
    dh = torch.cat([dy, bf(cap, I, seed=5)], dim=1).contiguous()
    dh[nrows:] = 0
    dh[:nrows][src < 0] = 0
    dx2 = OF.grouped_linear_dgrad_pair(dh, w, w2, ix)
    for e in range(E):
        a, b = offs[e], offs[e + 1]
        if b > a:
            want = dh[a:b, :I].float() @ w[e].float() + dh[a:b, I:].float() @ w2[e].float()
            assert rel_err(dx2[a:b], want) < 1e-2


def test_gemm_k_concatenated_b():
    M, N, K1, K2 = 384, 320, 192, 128
    a = bf(M, K1 + K2, seed=1)
    b1, b2 = bf(N, K1, seed=2), bf(N, K1, seed=3)   # K-major B: [N, K]; both halves must share a layout
    # K-major operands: second half of K comes from b2 (only its first K2 columns are read)
    y = OF.gemm(a, b1, M, N, K1 + K2, b2=b2, k_split=K1)
    want = a[:, :K1].float() @ b1.float().t() + a[:, K1:].float() @ b2[:, :K2].float().t()
    assert rel_err(y, want) < 1e-2
    # MN-major B ([K, N]) as in an input-gradient GEMM
    c1, c2 = bf(K1, N, seed=4), bf(K1, N, seed=5)
    y = OF.gemm(a, c1, M, N, K1 + K2, b_mn_major=True, b2=c2, k_split=K1)
    want = a[:, :K1].float() @ c1.float() + a[:, K1:].float() @ c2[:K2].float()
    assert rel_err(y, want) < 1e-2


@pytest.mark.parametrize("n,me,rows,N,K,b_mn", [(2, 0, 256, 512, 320, False), (4, 2, 1024, 1024, 2048, False),
                                                 (8, 7, 512, 384, 1024, True), (1, 0, 256, 128, 128, False)])
def test_gemm_with_fused_all_gather(n, me, rows, N, K, b_mn):
    """The all-gather variant of the GEMM with the "peers" standing in this GPU's memory: the stager warps copy the
    other slices into the gathered operand while the tiles of the local rows run, the producer waits per row block."""
    from optimus_lm_b200.ops import extension
    M = n * rows
    full = bf(M, K, seed=11)
    slices = [full[r * rows:(r + 1) * rows].clone() for r in range(n)]
    gathered = torch.full((M, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    gathered[me * rows:(me + 1) * rows] = slices[me]
    b = bf(K, N, seed=12) if b_mn else bf(N, K, seed=12)
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    flags = torch.empty(M // 128, dtype=torch.int32, device="cuda")
    extension().gemm_peer(gathered, [t.data_ptr() for t in slices], b, c, M, N, K, b_mn, me, flags,
                          OF.status_word("cuda"))
    want = full.float() @ (b.float() if b_mn else b.float().t())
    assert torch.equal(gathered, full)
    assert rel_err(c, want) < 1e-2
    counts = flags.tolist()
    assert all(v == (0 if i * 128 // rows == me else 128) for i, v in enumerate(counts)), counts


@pytest.mark.parametrize("n,me,rows,N,K,b_mn,split", [(2, 1, 256, 512, 320, False, 0), (4, 0, 1024, 1024, 1024, True, 512),
                                                       (8, 3, 256, 328, 256, False, 0), (1, 0, 256, 128, 128, False, 0)])
def test_gemm_with_fused_reduce_scatter_push(n, me, rows, N, K, b_mn, split):
    """The reduce-scatter variant of the GEMM with the peers' receive slots standing in this GPU's memory: every
    finished row that belongs to another peer is copied to that peer's slot by the stager warps."""
    from optimus_lm_b200.ops import extension
    M = n * rows
    a = bf(M, K, seed=21)
    b = bf(K if not split else split, N, seed=22) if b_mn else bf(N, K, seed=22)
    b2 = bf(split, N, seed=23) if split else None
    part = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    slots = [torch.full((rows, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    flags = torch.empty(M // 128, dtype=torch.int32, device="cuda")
    extension().gemm_push(a, b, b2, split, part, [t.data_ptr() for t in slots], M, N, K, b_mn, me, flags,
                          OF.status_word("cuda"))
    if split:
        want = a[:, :split].float() @ b.float() + a[:, split:].float() @ b2[:K - split].float()
    else:
        want = a.float() @ (b.float() if b_mn else b.float().t())
    assert rel_err(part, want) < 1e-2
    for r in range(n):
        if r == me:
            assert torch.isnan(slots[r].float()).all()          # nothing is sent to oneself
        else:
            assert torch.equal(slots[r], part[r * rows:(r + 1) * rows]), r


@pytest.mark.parametrize("n,T,E_loc,K,H,I", [(2, 256, 4, 2, 256, 128), (4, 512, 8, 4, 512, 256), (1, 384, 8, 8, 320, 64)])
def test_grouped_gemm_with_fused_combine_push(n, T, E_loc, K, H, I):
    """The expert-parallel combine variant of the grouped GEMM with the token owners' receive buffers standing in
    this GPU's memory: every routed row of the output lands in slot [token, k] of its owner's buffer."""
    from optimus_lm_b200.ops import extension
    E = n * E_loc                                            # this "rank" owns experts [E_loc, 2 * E_loc) when n > 1
    e_start = E_loc if n > 1 else 0
    g = torch.Generator(device="cuda").manual_seed(3)
    idx_all = torch.stack([torch.randperm(E, device="cuda", generator=g)[:K] for _ in range(n * T)]).to(torch.int32)
    cap = OF.moe_capacity_rows(n * T, K, E_loc)
    ix = OF.MoEIndex(idx_all, e_start, E_loc, cap)
    act = bf(cap, I, seed=31)
    wd = bf(E_loc, H, I, seed=32, scale=0.1)
    ys = torch.empty(cap, H, dtype=torch.bfloat16, device="cuda")
    recv = [torch.full((T, K, H), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    flags = torch.empty(cap // 128 + 1, dtype=torch.int32, device="cuda")
    extension().gemm_ep_push(act, wd.view(E_loc * H, I), ys, [t.data_ptr() for t in recv], ix.meta, ix.src_of, ix.k_of,
                             cap, H, I, H, E_loc, T, K, 0, flags, OF.status_word("cuda"))
    want = OF.grouped_linear_fwd(act, wd, ix)
    used = int(ix.meta[0].item()) * 128
    src = ix.src_of[:used].long()
    rows = torch.nonzero(src >= 0).flatten()
    assert rows.numel() == int(((idx_all >= e_start) & (idx_all < e_start + E_loc)).sum().item())
    assert torch.equal(ys[rows], want[rows])
    owner, tok, k = src[rows] // T, src[rows] % T, ix.k_of[:used].long()[rows]
    got = torch.stack(recv)[owner, tok, k]
    assert torch.equal(got, ys[rows])
    written = torch.zeros(n, T, K, dtype=torch.bool, device="cuda")
    written[owner, tok, k] = True
    assert torch.isnan(torch.stack(recv).float()).all(dim=-1).eq(~written).all()   # nothing else was touched


@pytest.mark.parametrize("n,T,E_loc,K,H,I", [(1, 700, 8, 2, 256, 512), (2, 256, 4, 2, 256, 128), (4, 512, 8, 4, 512, 256)])
def test_gateup_swiglu_launch_with_fused_dispatch(n, T, E_loc, K, H, I, monkeypatch):
    """One launch = gather of the routed rows (from n token buffers standing in this GPU's memory) + gate and up
    projections + routing-weighted SwiGLU.  Checked bit for bit against the separate kernels, and element-wise against
    fp32 torch."""
    monkeypatch.setattr(OF, "_GATHER_IN_KERNEL_LOCAL", True)   # the in-kernel gather also with a single token buffer
    E = n * E_loc
    e_start = E_loc if n > 1 else 0
    g = torch.Generator(device="cuda").manual_seed(5)
    idx_all = torch.stack([torch.randperm(E, device="cuda", generator=g)[:K] for _ in range(n * T)]).to(torch.int32)
    w_all = torch.rand(n * T, K, device="cuda", generator=g)
    xs = [bf(T, H, seed=40 + r) for r in range(n)]
    wg, wu = bf(E_loc, I, H, seed=2, scale=0.05), bf(E_loc, I, H, seed=3, scale=0.05)
    cap = OF.moe_capacity_rows(n * T, K, E_loc)
    ix = OF.MoEIndex(idx_all, e_start, E_loc, cap)
    xp, h, act = OF.grouped_gateup_swiglu([t.data_ptr() for t in xs], H, T, w_all, wg, wu, ix)
    used = int(ix.meta[0].item()) * 128
    src = ix.src_of[:used].long()
    x_cat = torch.cat(xs)
    want_xp = torch.where((src >= 0)[:, None], x_cat[src.clamp(min=0)], torch.zeros((), dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(xp[:used], want_xp)
    hg = OF.grouped_linear_fwd(xp, wg, ix)
    hu = OF.grouped_linear_fwd(xp, wu, ix)
    assert torch.equal(h[:used, :I], hg[:used]) and torch.equal(h[:used, I:], hu[:used])
    act2 = torch.empty_like(act)
    from optimus_lm_b200.ops import extension
    extension().swiglu_rowscale_fwd(h[:, :I], h[:, I:], ix.src_of, ix.k_of, w_all, ix.meta, act2)
    assert (act[:used].float() - act2[:used].float()).abs().max().item() <= 1e-2 * act2[:used].float().abs().max().item() + 1e-6
    assert rel_err(act[:used], act2[:used]) < 2e-3
    # against fp32 torch, element by element
    rows = torch.nonzero(src >= 0).flatten()
    e_of = ix.meta[1:1 + used // 128].long().repeat_interleave(128)[rows]
    xr = x_cat[src[rows]].float()
    gr = torch.einsum("rh,rih->ri", xr, wg.float()[e_of])
    ur = torch.einsum("rh,rih->ri", xr, wu.float()[e_of])
    wr = w_all[src[rows], ix.k_of[:used].long()[rows]]
    want = wr[:, None] * F.silu(gr) * ur
    got = act[rows].float()
    assert rel_err(got, want) < 1e-2
    assert (got - want).abs().max().item() < 0.05 * want.abs().max().item() + 1e-3
    assert act[:used][src < 0].abs().max().item() == 0 if (src < 0).any() else True


def test_dense_gateup_swiglu_launch():
    """The same epilogue on a dense MLP (no routing weights, no gather)."""
    from optimus_lm_b200.ops import extension
    M, H, I = 1000, 256, 384
    x, wg, wu = bf(M, H, seed=1), bf(I, H, seed=2, scale=0.05), bf(I, H, seed=3, scale=0.05)
    h = torch.empty(M, 2 * I, dtype=torch.bfloat16, device="cuda")
    act = torch.empty(M, I, dtype=torch.bfloat16, device="cuda")
    extension().gemm_gateup_swiglu(x, wg, wu, h, act, M, I, H, None, None, None, None, 1, [], 0, 0, None,
                                   OF.status_word("cuda"))
    assert torch.equal(h[:, :I], OF.gemm(x, wg, M, I, H)) and torch.equal(h[:, I:], OF.gemm(x, wu, M, I, H))
    want = F.silu(h[:, :I].float()) * h[:, I:].float()
    assert (act.float() - want).abs().max().item() < 1e-2 * want.abs().max().item() + 1e-6
    ref = F.silu(x.float() @ wg.float().t()) * (x.float() @ wu.float().t())
    assert rel_err(act, ref) < 1e-2


@pytest.mark.parametrize("n,T,E_loc,K,H,I", [(1, 700, 8, 2, 256, 512), (4, 512, 8, 4, 512, 256)])
def test_down_dgrad_launch_with_fused_gather(n, T, E_loc, K, H, I):
    E = n * E_loc
    e_start = E_loc if n > 1 else 0
    g = torch.Generator(device="cuda").manual_seed(6)
    idx_all = torch.stack([torch.randperm(E, device="cuda", generator=g)[:K] for _ in range(n * T)]).to(torch.int32)
    ds = [bf(T, H, seed=50 + r) for r in range(n)]
    wd = bf(E_loc, H, I, seed=4, scale=0.05)
    ix = OF.MoEIndex(idx_all, e_start, E_loc, OF.moe_capacity_rows(n * T, K, E_loc))
    dyp, dact = OF.grouped_gather_dgrad([t.data_ptr() for t in ds], H, T, wd, ix)
    used = int(ix.meta[0].item()) * 128
    src = ix.src_of[:used].long()
    want_dyp = torch.where((src >= 0)[:, None], torch.cat(ds)[src.clamp(min=0)],
                           torch.zeros((), dtype=torch.bfloat16, device="cuda"))
    assert torch.equal(dyp[:used], want_dyp)
    assert torch.equal(dact[:used], OF.grouped_linear_dgrad(dyp, wd, ix)[:used])


@pytest.mark.parametrize("n,T,E_loc,K,H,I", [(1, 700, 8, 2, 256, 512), (4, 512, 8, 4, 512, 256)])
def test_down_dgrad_launch_with_swiglu_backward_epilogue(n, T, E_loc, K, H, I, monkeypatch):
    """Gather + d(act) = d(y) wd + SwiGLU backward in one launch against the three separate kernels."""
    from optimus_lm_b200.ops import extension
    C = extension()
    monkeypatch.setattr(OF, "_FUSE_SWIGLU_BWD", True)          # the fused epilogue is opt-in
    monkeypatch.setattr(OF, "_GATHER_IN_KERNEL_LOCAL", True)   # also with a single token buffer
    E = n * E_loc
    e_start = E_loc if n > 1 else 0
    g = torch.Generator(device="cuda").manual_seed(7)
    idx_all = torch.stack([torch.randperm(E, device="cuda", generator=g)[:K] for _ in range(n * T)]).to(torch.int32)
    w_all = torch.rand(n * T, K, device="cuda", generator=g)
    ds = [bf(T, H, seed=50 + r) for r in range(n)]
    wd = bf(E_loc, H, I, seed=4, scale=0.05)
    ix = OF.MoEIndex(idx_all, e_start, E_loc, OF.moe_capacity_rows(n * T, K, E_loc))
    h = bf(ix.rows, 2 * I, seed=77)
    dw = torch.zeros(n * T, K, device="cuda")
    dyp, dh = OF.grouped_down_dgrad_swiglu_bwd([t.data_ptr() for t in ds], H, T, wd, h, w_all, ix, dw)
    used = int(ix.meta[0].item()) * 128
    dyp2, dact = OF.grouped_gather_dgrad([t.data_ptr() for t in ds], H, T, wd, ix)
    dh2 = torch.empty_like(h)
    dw2 = torch.zeros_like(dw)
    C.swiglu_rowscale_bwd(dact, h[:, :I], h[:, I:], ix.src_of, ix.k_of, w_all, ix.meta, dh2[:, :I], dh2[:, I:], dw2)
    assert torch.equal(dyp[:used], dyp2[:used])
    assert rel_err(dh[:used], dh2[:used]) < 2e-3
    assert (dh[:used].float() - dh2[:used].float()).abs().max().item() <= 1e-2 * dh2[:used].float().abs().max().item() + 1e-6
    assert rel_err(dw, dw2) < 1e-3
    assert (dw - dw2).abs().max().item() <= 1e-3 * dw2.abs().max().item() + 1e-6


def test_gate_up_dgrad_launch_with_fused_combine_push():
    """Backward combine: the K-concatenated input-gradient launch sends its rows to the token owners' buffers."""
    from optimus_lm_b200.ops import extension
    n, T, E_loc, K, H, I = 4, 512, 8, 4, 512, 256
    E, e_start = n * E_loc, E_loc
    g = torch.Generator(device="cuda").manual_seed(8)
    idx_all = torch.stack([torch.randperm(E, device="cuda", generator=g)[:K] for _ in range(n * T)]).to(torch.int32)
    cap = OF.moe_capacity_rows(n * T, K, E_loc)
    ix = OF.MoEIndex(idx_all, e_start, E_loc, cap)
    dh = bf(cap, 2 * I, seed=61)
    wg, wu = bf(E_loc, I, H, seed=2, scale=0.05), bf(E_loc, I, H, seed=3, scale=0.05)
    dxp = torch.empty(cap, H, dtype=torch.bfloat16, device="cuda")
    recv = [torch.full((T, K, H), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(n)]
    extension().gemm_ep_push(dh, wg.view(E_loc * I, H), dxp, [t.data_ptr() for t in recv], ix.meta, ix.src_of, ix.k_of,
                             cap, H, 2 * I, I, E_loc, T, K, 0, OF.stage_flags(dh.device, cap), OF.status_word("cuda"),
                             True, wu.view(E_loc * I, H), I)
    want = OF.grouped_linear_dgrad_pair(dh, wg, wu, ix)
    used = int(ix.meta[0].item()) * 128
    src = ix.src_of[:used].long()
    rows = torch.nonzero(src >= 0).flatten()
    assert torch.equal(dxp[rows], want[rows])
    owner, tok, k = src[rows] // T, src[rows] % T, ix.k_of[:used].long()[rows]
    assert torch.equal(torch.stack(recv)[owner, tok, k], dxp[rows])
    out = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    filled = torch.nan_to_num(recv[1], nan=0.0)
    extension().sum_slots(filled, out)
    assert (out.float() - filled.float().sum(1)).abs().max().item() <= 2e-2 * filled.float().sum(1).abs().max().item()


def test_index_overflow_sets_the_status_word():
    """A capacity-limited index that is too small reports ST_OVERFLOW (6); the host reads and clears it."""
    _, idx = _routing(1024, 8, 2)
    OF.MoEIndex(idx, 0, 8, 1024)                 # 2048 routed pairs cannot fit 1024 rows
    torch.cuda.synchronize()
    assert OF.check_status("cuda") == 6
    assert OF.check_status("cuda") == 0          # cleared by the read
    ix = OF.MoEIndex(idx, 0, 8, OF.moe_capacity_rows(1024, 2, 8))
    assert int(ix.counts.sum().item()) == 2048 and OF.check_status("cuda") == 0


def test_bounded_peer_wait_times_out_without_hanging():
    """A rendezvous whose partner never signals gives up after its limit, records ST_TIMEOUT_PEER (5) and returns:
    the context stays usable.  The partner's signal word is a word of this GPU's memory that nothing writes."""
    from optimus_lm_b200.ops import extension
    pads = [torch.zeros(16 * 64, dtype=torch.int32, device="cuda") for _ in range(2)]
    st = OF.status_word("cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    extension().symm_barrier([p.data_ptr() for p in pads], 0, 3, 1, st, 20_000_000)    # 20 ms limit
    t1.record()
    torch.cuda.synchronize()
    assert 10.0 < t0.elapsed_time(t1) < 2000.0
    assert OF.check_status("cuda") == 5
    assert int(pads[1][3 * 16 + 0].item()) == 1      # this rank did signal its partner
    x = torch.arange(1024, device="cuda").float()
    assert float(x.sum().item()) == 1023 * 1024 / 2   # the GPU still answers
    assert OF.check_status("cuda") == 0


@pytest.mark.parametrize("M,N,K,n", [(512, 512, 256, 2), (1024, 2304, 512, 4), (256, 2048, 2048, 8)])
def test_gemm_with_fused_parameter_all_gather(M, N, K, n):
    """y = x w^T where only this rank's part of w is current locally: the other parts are fetched from their owners'
    copies (standing in this GPU's memory) inside the launch, and w is complete afterwards."""
    from optimus_lm_b200.ops import extension
    me = 1 % n
    x = bf(M, K, seed=1)
    w_true = bf(N, K, seed=2, scale=0.05)
    part = (N * K // n + 511) // 512 * 512            # shard boundaries like the flat optimizer's: multiples of 512 elements
    copies, seg = [], []
    w_local = torch.full((N, K), float("nan"), dtype=torch.bfloat16, device="cuda")
    for r in range(n):
        lo, hi = min(r * part, N * K), min((r + 1) * part, N * K)
        c = torch.full((N * K,), float("nan"), dtype=torch.bfloat16, device="cuda")
        c[lo:hi] = w_true.view(-1)[lo:hi]             # rank r holds the current values of its own shard only
        copies.append(c)
        if r == me:
            w_local.view(-1)[lo:hi] = w_true.view(-1)[lo:hi]
            seg += [0, 0]
        else:
            seg += [lo, hi]
    y = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    extension().gemm_b_gather(x, w_local, y, M, N, K, [c.data_ptr() for c in copies], seg, me,
                              OF.stage_flags(x.device, N), OF.status_word("cuda"))
    assert torch.equal(w_local, w_true)
    assert torch.equal(y, OF.gemm(x, w_true, M, N, K))


def test_exact_row_count_sizes_the_expert_buffers():
    """With ``exact`` the activation buffers follow the routed count, not the worst case, and nothing is dropped."""
    n, T, E_loc, K = 8, 1024, 4, 2
    E = n * E_loc
    g = torch.Generator(device="cuda").manual_seed(9)
    idx_all = torch.stack([torch.randperm(E, device="cuda", generator=g)[:K] for _ in range(n * T)]).to(torch.int32)
    cap = OF.moe_capacity_rows(n * T, K, E_loc)
    ix = OF.MoEIndex(idx_all, 0, E_loc, cap, exact=True)
    mine = int((idx_all < E_loc).sum().item())
    assert mine <= ix.rows < cap and ix.rows % OF.ROW_GRANULE == 0 and ix.rows >= int(ix.meta[0].item()) * 128
    assert int((ix.row_of >= 0).sum().item()) == mine


@pytest.mark.parametrize("T,E,K,H,I,e_start,E_loc", [(512, 8, 2, 256, 512, 0, 8), (1000, 16, 4, 128, 256, 4, 8),
                                                     (2048, 64, 8, 512, 256, 0, 64)])
def test_moe_experts_fwd_bwd(T, E, K, H, I, e_start, E_loc):
    w, idx = _routing(T, E, K)
    x = bf(T, H, seed=1).requires_grad_()
    wg = bf(E_loc, I, H, seed=2, scale=0.05).requires_grad_()
    wu = bf(E_loc, I, H, seed=3, scale=0.05).requires_grad_()
    wd = bf(E_loc, H, I, seed=4, scale=0.05).requires_grad_()
    tw = w.clone().requires_grad_()
    out = OF.moe_experts(x, tw, idx, wg, wu, wd, e_start)
    g = bf(T, H, seed=5)
    out.backward(g)
    xr, wgr, wur, wdr, twr = [t.detach().float().requires_grad_() for t in (x, wg, wu, wd, tw)]
    ref = OF.moe_experts_reference(xr, twr, idx.long(), wgr, wur, wdr, e_start)
    ref.backward(g.float())
    assert rel_err(out, ref) < 2e-2
    assert rel_err(x.grad, xr.grad) < 2e-2
    assert rel_err(wg.grad, wgr.grad) < 2e-2 and rel_err(wu.grad, wur.grad) < 2e-2
    assert rel_err(wd.grad, wdr.grad) < 2e-2
    assert rel_err(tw.grad, twr.grad) < 2e-2


# ------------------------------------------------------------------ norms / activations / rope
@pytest.mark.parametrize("rows,cols", [(64, 256), (1000, 2048), (33, 7168)])
def test_rmsnorm(rows, cols):
    x = bf(rows, cols, seed=1).requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).to(torch.bfloat16).requires_grad_()
    y = OF.rms_norm(x, w, 1e-5)
    g = bf(rows, cols, seed=2)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = OF.rms_norm_reference(xr, wr, 1e-5)
    yr.backward(g.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(x.grad, xr.grad) < 1e-2 and rel_err(w.grad, wr.grad) < 1e-2


def test_layernorm_noaffine():
    x = bf(500, 2048, seed=1).requires_grad_()
    y = OF.layer_norm_noaffine(x, 1e-5)
    g = bf(500, 2048, seed=2)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = F.layer_norm(xr, (2048,), None, None, 1e-5)
    yr.backward(g.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(x.grad, xr.grad) < 1e-2


def test_swiglu():
    gte, up = bf(300, 1024, seed=1).requires_grad_(), bf(300, 1024, seed=2).requires_grad_()
    y = OF.swiglu(gte, up)
    g = bf(300, 1024, seed=3)
    y.backward(g)
    gr, ur = gte.detach().float().requires_grad_(), up.detach().float().requires_grad_()
    yr = F.silu(gr) * ur
    yr.backward(g.float())
    assert rel_err(y, yr) < 1e-2 and rel_err(gte.grad, gr.grad) < 1e-2 and rel_err(up.grad, ur.grad) < 1e-2


@pytest.mark.parametrize("interleaved,rot_offset,D", [(False, 0, 128), (False, 0, 64), (True, 128, 192)])
def test_rope(interleaved, rot_offset, D):
    B, S, Hn = 2, 256, 4
    rot = D - rot_offset
    inv = 1.0 / (10000 ** (torch.arange(0, rot, 2, device="cuda").float() / rot))
    fr = torch.outer(torch.arange(S, device="cuda").float(), inv)
    emb = torch.cat([fr, fr], -1)
    cos, sin = emb.cos().contiguous(), emb.sin().contiguous()
    x0 = bf(B, S, Hn, D, seed=1)
    xr = x0.float().requires_grad_()
    yr = OF.rope_reference(xr, cos, sin, rot_offset, rot, interleaved)
    g = bf(B, S, Hn, D, seed=2)
    yr.backward(g.float())
    x = x0.clone().requires_grad_()
    y = OF.rope(x * 1.0, cos, sin, rot_offset, rot, interleaved)
    y.backward(g)
    assert rel_err(y, yr) < 1e-2 and rel_err(x.grad, xr.grad) < 1e-2


# ------------------------------------------------------------------ router
@pytest.mark.parametrize("T,E,K,renorm", [(1000, 64, 8, False), (513, 8, 2, True), (256, 256, 8, False)])
def test_router_softmax_topk(T, E, K, renorm):
    logits = bf(T, E, seed=1, scale=2.0).requires_grad_()
    w, idx, stats = OF.router_softmax_topk(logits, K, renorm)
    lr = logits.detach().float().requires_grad_()
    wr, idxr = OF.router_softmax_topk_reference(lr, K, renorm)
    # same selected sets (order may differ only on exact ties)
    assert torch.equal(idx.long().sort(-1).values, idxr.sort(-1).values)
    sel_ref = torch.gather(torch.softmax(lr, -1), 1, idx.long()).detach()
    if renorm:
        sel_ref = sel_ref / sel_ref.sum(-1, keepdim=True)
    assert rel_err(w, sel_ref) < 1e-4
    g = torch.randn(T, K, device="cuda")
    w.backward(g)
    # reference gradient with matching order
    p = torch.softmax(lr, -1)
    sel = torch.gather(p, 1, idx.long())
    if renorm:
        sel = sel / sel.sum(-1, keepdim=True)
    sel.backward(g)
    assert rel_err(logits.grad, lr.grad) < 2e-2
    cnt = torch.bincount(idx.flatten().long(), minlength=E).float()
    assert torch.equal(stats[:E], cnt)
    assert rel_err(stats[E:2 * E], p.sum(0)) < 1e-4
    assert abs(stats[2 * E].item() - torch.logsumexp(lr, -1).pow(2).sum().item()) / stats[2 * E].item() < 1e-4


def test_router_aux_loss_matches_reference():
    T, E, K, L = 512, 16, 4, 3
    logits = [bf(T, E, seed=i, scale=1.5).requires_grad_() for i in range(L)]
    outs = [OF.router_softmax_topk(l, K, False) for l in logits]
    for layer_level in (False, True):
        for l in logits:
            l.grad = None
        aux = OF.router_aux_loss(logits, [o[1] for o in outs], [o[2] for o in outs], E, K, layer_level=layer_level,
                                 aux_coef=0.01, z_coef=0.001)
        aux.backward()
        refs = [l.detach().float().requires_grad_() for l in logits]
        fn = OF.layer_level_load_balancing_loss_reference if layer_level else OF.load_balancing_loss_reference
        ref = 0.01 * fn(tuple(refs), E, K) + 0.001 * OF.z_loss_reference(refs)
        ref.backward()
        assert abs(aux.item() - ref.item()) / abs(ref.item()) < 1e-3
        for a, b in zip(logits, refs):
            assert rel_err(a.grad, b.grad) < 3e-2


def test_router_sigmoid_group_topk():
    T, E, K, G, TG = 777, 256, 8, 8, 4
    logits = torch.randn(T, E, device="cuda")
    bias = 0.01 * torch.randn(E, device="cuda")
    C = OF.extension()
    w = torch.empty(T, K, device="cuda")
    idx = torch.empty(T, K, dtype=torch.int32, device="cuda")
    C.router_sigmoid_group_topk(logits, bias, K, G, TG, True, 2.5, w, idx)
    scores = logits.sigmoid()
    ch = scores + bias
    gs = ch.view(T, G, E // G).topk(2, dim=-1)[0].sum(-1)
    gi = gs.topk(TG, dim=-1)[1]
    gm = torch.zeros_like(gs).scatter_(1, gi, 1)
    sm = gm.unsqueeze(-1).expand(T, G, E // G).reshape(T, E)
    ch = ch.masked_fill(~sm.bool(), 0.0)
    ri = ch.topk(K, dim=-1)[1]
    rw = scores.gather(1, ri)
    rw = rw / (rw.sum(-1, keepdim=True) + 1e-20) * 2.5
    assert torch.equal(idx.long().sort(-1).values, ri.sort(-1).values)
    assert rel_err(w.sort(-1).values, rw.sort(-1).values) < 1e-5


# ------------------------------------------------------------------ loss / optimizer
@pytest.mark.parametrize("B,S,V", [(2, 64, 1024), (1, 128, 50304)])
def test_shifted_cross_entropy(B, S, V):
    logits = bf(B, S, V, seed=1, scale=2.0).requires_grad_()
    labels = torch.randint(0, V, (B, S), device="cuda")
    loss = OF.shifted_cross_entropy(logits, labels)
    loss.backward()
    lr = logits.detach().float().requires_grad_()
    ref = OF.shifted_cross_entropy_reference(lr, labels)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 1e-3 * abs(ref.item())
    assert rel_err(logits.grad, lr.grad) < 1e-2


def test_adamw_and_sumsq():
    n = 512 * 37
    g = bf(n, seed=1)
    master = torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    p = master.to(torch.bfloat16)
    mr, vr, pr, masr = m.clone(), v.clone(), p.clone(), master.clone()
    clip = torch.tensor([0.5], device="cuda")
    for step in (1, 2, 3):
        OF.adamw_step(g, master, m, v, p, 4e-4, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=0.25, clip_coef=clip)
        OF.adamw_step_reference(g, masr, mr, vr, pr, 4e-4, 0.9, 0.95, 1e-8, 0.1, step, grad_scale=0.25, clip_coef=clip)
    assert rel_err(master, masr) < 1e-6 and rel_err(m, mr) < 1e-6 and rel_err(v, vr) < 1e-6
    assert torch.equal(p, pr) or rel_err(p, pr) < 1e-3
    s = OF.sum_of_squares(g, 0.5)
    assert abs(s.item() - (g.float() * 0.5).pow(2).sum().item()) / s.item() < 1e-5
    s2 = OF.sum_of_squares(g, 0.5)
    assert torch.equal(s, s2)
    # the norm as a by-product of the update's own pass over the gradients (unclipped, scaled)
    acc = torch.full((1,), 3.0, device="cuda")
    OF.adamw_step(g, master, m, v, p, 4e-4, 0.9, 0.95, 1e-8, 0.1, 4, grad_scale=0.5, norm_out=acc)
    assert abs(acc.item() - 3.0 - s.item()) / s.item() < 1e-5


def test_kernels_package_entry_points():
    """The reference-named GEMM wrappers: NN, NT, TN, accumulate."""
    import optimus_lm_b200.kernels as K
    a, b_nk, b_kn = bf(256, 192, seed=1), bf(320, 192, seed=2), bf(192, 320, seed=3)
    assert rel_err(K.gemm(a, b_kn), a.float() @ b_kn.float()) < 1e-2
    assert rel_err(K.gemm_trans(a, b_nk), a.float() @ b_nk.float().t()) < 1e-2
    assert rel_err(K.linear_forward(a, b_nk), a.float() @ b_nk.float().t()) < 1e-2
    dy = bf(256, 320, seed=4)
    dx = K.linear_backward_input(dy, b_nk)
    assert rel_err(dx, dy.float() @ b_nk.float()) < 1e-2
    base = dx.clone()
    K.linear_backward_input_add(dy, b_nk, dx)
    assert rel_err(dx, 2 * base.float()) < 1e-2
    assert rel_err(K.linear_backward_weight(dy, a), dy.float().t() @ a.float()) < 1e-2


@pytest.mark.parametrize("v_start,rows", [(0, 1000), (300, 400)])
def test_embedding_fwd_bwd(v_start, rows):
    V, H, T = 1000, 256, 3000
    g = torch.Generator(device="cuda").manual_seed(0)
    ids = torch.randint(0, V, (3, T // 3), device="cuda", generator=g)
    ids[0, :50] = 7 + v_start          # a long run of one id
    w = bf(rows, H, seed=1).requires_grad_()
    pad = 5
    y = OF.embedding(ids, w, padding_idx=pad, v_start=v_start)
    local = ids - v_start
    inside = (local >= 0) & (local < rows)
    ref = torch.where(inside[..., None], w.detach().float()[local.clamp(0, rows - 1)], torch.zeros(1, device="cuda"))
    assert torch.equal(y.float(), ref)
    dy = bf(3, T // 3, H, seed=2)
    y.backward(dy)
    want = torch.zeros(rows, H, device="cuda")
    sel = inside & (local != pad)
    want.index_add_(0, local[sel], dy.float()[sel])
    assert rel_err(w.grad, want) < 1e-2
    assert w.grad[pad].abs().max().item() == 0
    # deterministic, and accumulation into an existing gradient buffer
    g1 = w.grad.clone()
    w.grad = None
    OF.embedding(ids, w, padding_idx=pad, v_start=v_start).backward(dy)
    assert torch.equal(w.grad, g1)
    h = OF.DirectGrad(torch.zeros_like(w))
    w._olb_direct = h
    for _ in range(2):
        OF.embedding(ids, w, padding_idx=pad, v_start=v_start).backward(dy)
    assert rel_err(h.buf, 2 * want) < 1e-2


# ------------------------------------------------------------------ reference custom-op interface, profiler shim
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_custom_op_kernels_match_their_tensor_programs(dtype):
    """The CUDA kernels behind the reference's custom-op entry points against the same functions on CPU tensors."""
    from optimus_lm_b200 import custom_ops as ops
    torch.manual_seed(0)
    T, K, E, e0, e1, H = 203, 4, 16, 4, 12, 64
    sel = torch.stack([torch.randperm(E)[:K] for _ in range(T)]).int()
    E_loc, TH = e1 - e0, (T + 7) // 8

    def pipeline(dev):
        s = sel.to(dev)
        ptc = torch.zeros((E_loc, TH), dtype=torch.int32, device=dev)
        cnt = torch.zeros(T, dtype=torch.int32, device=dev)
        ops.compute_partial_token_counts(s, ptc, cnt, e0, e1)
        pc = torch.zeros(E_loc * TH + 1, dtype=torch.int32, device=dev)
        pc[1:] = torch.cumsum(ptc.flatten(), 0).int()
        cum = torch.zeros(T + 1, dtype=torch.int32, device=dev)
        cum[1:] = torch.cumsum(cnt, 0).int()
        R = int(pc[-1])
        sei, ii, oi = (torch.empty(R, dtype=torch.int32, device=dev) for _ in range(3))
        incr = torch.zeros(E_loc * TH, dtype=torch.int32, device=dev)
        ops.compute_input_and_output_indices(s, pc, incr, cum, sei, ii, oi, e0, e1)
        g = torch.Generator().manual_seed(3)
        x = torch.randn(T, H, generator=g).to(dtype).to(dev)
        w = torch.rand(T, K, generator=g).to(dtype).to(dev)
        y = torch.randn(R, H, generator=g).to(dtype).to(dev)
        dout = torch.randn(T, H, generator=g).to(dtype).to(dev)
        xg = torch.empty(R, H, dtype=dtype, device=dev)
        ops.index_gather(x, ii, xg)
        out = torch.empty(T, H, dtype=dtype, device=dev)
        ops.reduce_ggemm_output(y, w, cum, sei, oi, out, False)
        dy = torch.zeros(R, H, dtype=dtype, device=dev)
        dw = torch.zeros(T, K, dtype=dtype, device=dev)
        ops.reduce_ggemm_output_backward(dout, y, w, cum, sei, ii, oi, dy, dw)
        dx = torch.empty(T, H, dtype=dtype, device=dev)
        ops.shuffle_sub_matrix_reduce(dy, cum, oi, dx)
        base = torch.zeros(T, H, dtype=dtype, device=dev)
        ops.index_add_op(y, base, ii)
        return [t.cpu() for t in (ptc, cnt, sei, ii, oi, xg, out, dy, dw, dx, base)]

    got, want = pipeline("cuda"), pipeline("cpu")
    for a, b in zip(got[:5], want[:5]):
        assert torch.equal(a, b)
    assert torch.equal(got[5], want[5])
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for a, b in zip(got[6:], want[6:]):
        assert (a.float() - b.float()).abs().max().item() <= tol * (b.float().abs().max().item() + 1.0)
    assert OF.check_status("cuda") == 0


def test_native_profiler_shim_marks_events_and_times_copies():
    from optimus_lm_b200.ops import extension
    C = extension()
    a = C.mark_event()
    src = torch.randn(64 * 1024 * 1024 // 4, device="cuda")
    dst = torch.empty_like(src)
    cp = C.async_memcpy(src, dst)
    b = C.mark_event()
    b.wait()
    assert torch.equal(src, dst)
    assert a.get_elapsed_time() >= 0 and a.get_start_time() > 0
    assert a.get_start_time() <= cp.get_start_time() <= cp.get_end_time() <= b.get_end_time()
    gbs = 2 * src.numel() * 4 / cp.get_elapsed_time()           # bytes per nanosecond = GB/s
    assert 100.0 < gbs < 20000.0, gbs
    assert cp.get_submit_time() > 0
