"""Compatibility entry points of the MoE custom-op interface against a naive per-token reference."""
import torch

from optimus_lm_b200 import custom_ops as ops


def _naive_index(sel, e0, e1):
    """Rows ordered by (expert, block of 8 tokens, token, k); slots token-major."""
    T, K = sel.shape
    pairs = [(int(sel[t, k]) - e0, t // 8, t, k) for t in range(T) for k in range(K) if e0 <= int(sel[t, k]) < e1]
    rows = sorted(range(len(pairs)), key=lambda i: (pairs[i][0], pairs[i][1], pairs[i][2], pairs[i][3]))
    row_of_pair = {p: r for r, p in enumerate(rows)}
    input_idx = [0] * len(pairs)
    out_idx, sel_idx = [], []
    for slot, (e, b, t, k) in enumerate(pairs):
        r = row_of_pair[slot]
        input_idx[r] = t
        out_idx.append(r)
        sel_idx.append(k)
    return input_idx, out_idx, sel_idx


def test_moe_index_pipeline_matches_naive():
    torch.manual_seed(0)
    T, K, E, e0, e1, H = 37, 3, 8, 2, 6, 16
    sel = torch.stack([torch.randperm(E)[:K] for _ in range(T)]).int()
    E_loc, TH = e1 - e0, (T + 7) // 8
    ptc = torch.zeros((E_loc, TH), dtype=torch.int32)
    cnt = torch.zeros(T, dtype=torch.int32)
    ops.compute_partial_token_counts(sel, ptc, cnt, e0, e1)
    assert int(ptc.sum()) == int(((sel >= e0) & (sel < e1)).sum()) == int(cnt.sum())
    pc = torch.zeros(E_loc * TH + 1, dtype=torch.int32)
    torch.cumsum(ptc.flatten(), 0, out=pc[1:])
    cum = torch.zeros(T + 1, dtype=torch.int32)
    torch.cumsum(cnt, 0, out=cum[1:])
    R = int(pc[-1])
    sei, ii, oi = (torch.empty(R, dtype=torch.int32) for _ in range(3))
    ops.compute_input_and_output_indices(sel, pc, torch.zeros(1, dtype=torch.int32), cum, sei, ii, oi, e0, e1)
    wi, wo, ws = _naive_index(sel, e0, e1)
    assert ii.tolist() == wi and oi.tolist() == wo and sei.tolist() == ws

    x = torch.randn(T, H)
    xg = torch.empty(R, H)
    ops.index_gather(x, ii, xg)
    assert torch.equal(xg, x[ii.long()])
    w = torch.rand(T, K)
    y = torch.randn(R, H)
    out = torch.empty(T, H)
    ops.reduce_ggemm_output(y, w, cum, sei, oi, out, False)
    want = torch.zeros(T, H)
    for t in range(T):
        for s in range(int(cum[t]), int(cum[t + 1])):
            want[t] += w[t, int(sei[s])] * y[int(oi[s])]
    assert torch.allclose(out, want, atol=1e-6)

    dout = torch.randn(T, H)
    dy, dw = torch.zeros(R, H), torch.zeros(T, K)
    ops.reduce_ggemm_output_backward(dout, y, w, cum, sei, ii, oi, dy, dw)
    dx = torch.empty(T, H)
    ops.shuffle_sub_matrix_reduce(dy, cum, oi, dx)
    wdy, wdw, wdx = torch.zeros(R, H), torch.zeros(T, K), torch.zeros(T, H)
    for t in range(T):
        for s in range(int(cum[t]), int(cum[t + 1])):
            r, k = int(oi[s]), int(sei[s])
            wdy[r] = w[t, k] * dout[t]
            wdw[t, k] = (y[r] * dout[t]).sum()
            wdx[t] += wdy[r]
    assert torch.allclose(dy, wdy, atol=1e-6) and torch.allclose(dw, wdw, atol=1e-5) and torch.allclose(dx, wdx, atol=1e-5)


def test_index_add_function_autograd():
    torch.manual_seed(1)
    e = torch.randn(5, 4, requires_grad=True)
    base = torch.zeros(7, 4)
    idx = torch.tensor([6, 0, 3, 0, 2], dtype=torch.int32)
    out = ops.IndexAddOpFunction.apply(e, base, idx)
    want = torch.zeros(7, 4).index_add(0, idx.long(), e.detach())
    assert torch.equal(out.detach(), want)
    g = torch.randn(7, 4)
    out.backward(g)
    assert torch.equal(e.grad, g[idx.long()])
    o = torch.empty(3, 8)
    ops.RMSNormOp(torch.randn(3, 8), torch.ones(8), o, 1e-5)
    assert torch.allclose(o.pow(2).mean(-1), torch.ones(3), atol=1e-3)
