"""Kernel micro-benchmarks (counterpart of the ``__main__`` blocks of the reference's
optimus/kernels/*.py): time the tcgen05 GEMMs, the grouped expert GEMMs and flash attention
against the library kernels with CUDA events, print TFLOP/s.

    python -m optimus_lm_b200.ops.bench_kernels [gemm|grouped|attention|all]
"""
import sys

import torch

from . import functional as OF
from . import attention as OA


def _time(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()  # > L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def bench_gemm():
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    for M, N, K in [(4096, 4096, 4096), (8192, 8192, 8192), (16384, 2048, 2048), (16384, 50304, 2048)]:
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        t1 = _time(lambda: OF.gemm(a, b, M, N, K, out=c), flush=flush)
        t2 = _time(lambda: torch.matmul(a, b.t(), out=c), flush=flush)
        fl = 2.0 * M * N * K
        print(f"gemm NT {M}x{N}x{K}: tcgen05 kernel {t1:.3f} ms ({fl / t1 * 1e-9:.0f} TFLOP/s) | cuBLAS {t2:.3f} ms "
              f"({fl / t2 * 1e-9:.0f} TFLOP/s)", flush=True)
    # the other two products of a projection at the model's shape: input gradient (NN) and weight gradient (TN)
    M, N, K = 16384, 2048, 2048
    dy = torch.randn(M, N, device="cuda").to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    dx = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
    dw = torch.empty(N, K, device="cuda", dtype=torch.bfloat16)
    fl = 2.0 * M * N * K
    t1 = _time(lambda: OF.gemm(dy, w, M, K, N, b_mn_major=True, out=dx), flush=flush)
    t2 = _time(lambda: torch.matmul(dy, w, out=dx), flush=flush)
    print(f"gemm NN (dgrad) {M}x{K}x{N}: tcgen05 kernel {t1:.3f} ms ({fl / t1 * 1e-9:.0f} TFLOP/s) | cuBLAS {t2:.3f} ms "
          f"({fl / t2 * 1e-9:.0f} TFLOP/s)", flush=True)
    t1 = _time(lambda: OF.gemm(dy, x, N, K, M, a_mn_major=True, b_mn_major=True, out=dw), flush=flush)
    t2 = _time(lambda: torch.matmul(dy.t(), x, out=dw), flush=flush)
    print(f"gemm TN (wgrad) {N}x{K}x{M}: tcgen05 kernel {t1:.3f} ms ({fl / t1 * 1e-9:.0f} TFLOP/s) | cuBLAS {t2:.3f} ms "
          f"({fl / t2 * 1e-9:.0f} TFLOP/s)", flush=True)


def bench_grouped():
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    T, E, K, H, I = 16384, 64, 8, 2048, 1024
    idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]).to(torch.int32)
    cap = OF.moe_capacity_rows(T, K, E)
    ix = OF.MoEIndex(idx, 0, E, cap)
    xp = torch.randn(cap, H, device="cuda").to(torch.bfloat16)
    w = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16)
    y = torch.empty(cap, I, device="cuda", dtype=torch.bfloat16)
    t = _time(lambda: OF.grouped_linear_fwd(xp, w, ix, out=y), flush=flush)
    fl = 2.0 * T * K * H * I
    print(f"grouped fwd  {T * K} rows x {H}->{I}, {E} experts: {t:.3f} ms ({fl / t * 1e-9:.0f} TFLOP/s)", flush=True)
    dy = torch.randn(cap, I, device="cuda").to(torch.bfloat16)
    t = _time(lambda: OF.grouped_linear_dgrad(dy, w, ix), flush=flush)
    print(f"grouped dgrad: {t:.3f} ms ({fl / t * 1e-9:.0f} TFLOP/s)", flush=True)
    t = _time(lambda: OF.grouped_linear_wgrad(dy, xp, ix, I, H), flush=flush)
    print(f"grouped wgrad: {t:.3f} ms ({fl / t * 1e-9:.0f} TFLOP/s)", flush=True)
    # the fused launches of the MoE layer, with and without the in-kernel row gather
    from ._ext import extension
    C = extension()
    x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    tw = torch.rand(T, K, device="cuda")
    wu = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16)
    wd = (torch.randn(E, H, I, device="cuda") * 0.02).to(torch.bfloat16)
    h = torch.empty(cap, 2 * I, device="cuda", dtype=torch.bfloat16)
    act = torch.empty(cap, I, device="cuda", dtype=torch.bfloat16)
    st = OF.status_word("cuda")
    t = _time(lambda: C.gemm_gateup_swiglu(xp, w.view(E * I, H), wu.view(E * I, H), h, act, cap, I, H, ix.meta, ix.src_of,
                                           ix.k_of, tw, E, [], 0, 0, None, st, ix.pair), flush=flush)
    print(f"gate|up + SwiGLU epilogue, operand in place: {t:.3f} ms ({2 * fl / t * 1e-9:.0f} TFLOP/s)", flush=True)
    t = _time(lambda: OF.grouped_gateup_swiglu([x.data_ptr()], H, T, tw, w, wu, ix), flush=flush)
    print(f"gate|up + SwiGLU epilogue + row gather     : {t:.3f} ms ({2 * fl / t * 1e-9:.0f} TFLOP/s)", flush=True)
    dout = torch.randn(T, H, device="cuda").to(torch.bfloat16)
    t = _time(lambda: OF.grouped_gather_dgrad([dout.data_ptr()], H, T, wd, ix), flush=flush)
    print(f"down dgrad + row gather                    : {t:.3f} ms ({fl / t * 1e-9:.0f} TFLOP/s)", flush=True)
    dw = torch.zeros(T, K, device="cuda")
    t = _time(lambda: OF.grouped_down_dgrad_swiglu_bwd([dout.data_ptr()], H, T, wd, h, tw, ix, dw), flush=flush)
    print(f"down dgrad + row gather + SwiGLU backward  : {t:.3f} ms ({fl / t * 1e-9:.0f} TFLOP/s)", flush=True)
    assert OF.check_status("cuda") == 0


def bench_attention():
    import torch.nn.functional as F
    for B, S, Hh, D, Dv in [(4, 4096, 16, 128, 128), (1, 4096, 128, 192, 128)]:
        q = torch.randn(B, S, Hh, D, device="cuda").to(torch.bfloat16)
        k = torch.randn(B, S, Hh, D, device="cuda").to(torch.bfloat16)
        v = torch.randn(B, S, Hh, Dv, device="cuda").to(torch.bfloat16)
        fl = 2.0 * B * Hh * S * S * (D + Dv) / 2
        t1 = _time(lambda: OA.flash_attention(q, k, v))
        msg = f"attention fwd B{B} S{S} H{Hh} D{D}/{Dv}: kernel {t1:.3f} ms ({fl / t1 * 1e-9:.0f} TFLOP/s)"
        C = OF.extension()
        o_ = torch.empty(B, S, Hh, Dv, dtype=torch.bfloat16, device="cuda")
        lse_ = torch.empty(B, Hh, S, dtype=torch.float32, device="cuda")
        st_ = OF.status_word(q.device)
        for variant, label in ((1, "one query tile per CTA"), (2, "two query tiles per CTA")):
            tv = _time(lambda: C.attn_fwd(q, k, v, o_, lse_, D ** -0.5, st_, variant))
            msg += f" | {label} {tv:.3f} ms ({fl / tv * 1e-9:.0f} TFLOP/s)"
        if D == Dv:
            qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
            t2 = _time(lambda: F.scaled_dot_product_attention(qh, kh, vh, is_causal=True))
            msg += f" | SDPA {t2:.3f} ms ({fl / t2 * 1e-9:.0f} TFLOP/s)"
        print(msg, flush=True)
        qa, ka, va = (t.clone().requires_grad_() for t in (q, k, v))
        o = OA.flash_attention(qa, ka, va)
        do = torch.randn_like(o)
        tb = _time(lambda: torch.autograd.grad(o, (qa, ka, va), do, retain_graph=True))
        print(f"attention bwd: {tb:.3f} ms ({2.5 * fl / tb * 1e-9:.0f} TFLOP/s)", flush=True)
    assert OF.check_status("cuda") == 0


def profile_case(name: str, launches: int = 4):
    """A few launches of ONE kernel on operands larger than L2 and well under a GB each: the case to
    put under a hardware profiler (``profile-gemm``, ``profile-grouped``, ``profile-attention``,
    ``profile-attention-bwd``, ``profile-gateup``, ``profile-gateup-nogather``, ``profile-dgrad-gather``, ``profile-ep``, ``profile-gemm-allgather``, ``profile-gemm-push``, ``profile-rs-adamw``,
    ``profile-rmsnorm-bwd``)."""
    torch.manual_seed(0)
    if name == "gemm":
        M = N = K = 8192
        a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fn = lambda: OF.gemm(a, b, M, N, K, out=c)
    elif name == "grouped":
        T, E, K, H, I = 16384, 64, 8, 2048, 1024
        idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]).to(torch.int32)
        ix = OF.MoEIndex(idx, 0, E, OF.moe_capacity_rows(T, K, E))
        xp = torch.randn(ix.cap, H, device="cuda").to(torch.bfloat16)
        w = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16)
        y = torch.empty(ix.cap, I, device="cuda", dtype=torch.bfloat16)
        fn = lambda: OF.grouped_linear_fwd(xp, w, ix, out=y)
    elif name in ("gateup", "gateup-nogather", "dgrad-gather"):
        # the fused launches of the MoE layer on half of the model's token count (operands ~1.5 GB in total)
        from ._ext import extension
        T, E, K, H, I = 8192, 64, 8, 2048, 1024
        idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]).to(torch.int32)
        ix = OF.MoEIndex(idx, 0, E, OF.moe_capacity_rows(T, K, E))
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16)
        tw = torch.rand(T, K, device="cuda")
        wg = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16)
        wu = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16)
        wd = (torch.randn(E, H, I, device="cuda") * 0.02).to(torch.bfloat16)
        if name == "gateup":
            fn = lambda: OF.grouped_gateup_swiglu([x.data_ptr()], H, T, tw, wg, wu, ix)
        elif name == "gateup-nogather":
            xp = torch.randn(ix.rows, H, device="cuda").to(torch.bfloat16)
            h = torch.empty(ix.rows, 2 * I, device="cuda", dtype=torch.bfloat16)
            act = torch.empty(ix.rows, I, device="cuda", dtype=torch.bfloat16)
            st = OF.status_word("cuda")
            fn = lambda: extension().gemm_gateup_swiglu(xp, wg.view(E * I, H), wu.view(E * I, H), h, act, ix.rows, I, H,
                                                        ix.meta, ix.src_of, ix.k_of, tw, E, [], 0, 0, None, st, ix.pair)
        else:
            fn = lambda: OF.grouped_gather_dgrad([x.data_ptr()], H, T, wd, ix)
    elif name == "attention":
        q, k, v = (torch.randn(4, 4096, 16, 128, device="cuda").to(torch.bfloat16) for _ in range(3))
        fn = lambda: OA.flash_attention(q, k, v)
    elif name == "attention-bwd":
        q, k, v = (torch.randn(4, 4096, 16, 128, device="cuda").to(torch.bfloat16).requires_grad_() for _ in range(3))
        o = OA.flash_attention(q, k, v)
        do = torch.randn_like(o)
        fn = lambda: torch.autograd.grad(o, (q, k, v), do, retain_graph=True)
    elif name == "ep":
        # The expert-parallel MoE function with a process group of ONE rank: the peer-memory kernels (row pulls,
        # combine, device barrier) run with this GPU as their only "peer", so that a single-process profiler can
        # look at them.  NVLink does not appear in such a capture; the multi-GPU timings are taken with CUDA events.
        import os
        import torch.distributed as dist
        from ..parallel.ep_alltoall import _FusedEPMoEFn
        from ..parallel.symm import SymmGroup
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29577")
        if not dist.is_initialized():
            dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        sg = SymmGroup.get(dist.group.WORLD)
        T, E, K, H, I = 16384, 64, 8, 2048, 1024
        x = torch.randn(T, H, device="cuda").to(torch.bfloat16).requires_grad_()
        idx = torch.stack([torch.randperm(E, device="cuda")[:K] for _ in range(T)]).to(torch.int32)
        tw = torch.rand(T, K, device="cuda")
        wg = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
        wu = (torch.randn(E, I, H, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
        wd = (torch.randn(E, H, I, device="cuda") * 0.02).to(torch.bfloat16).requires_grad_()
        cap = OF.moe_capacity_rows(T, K, E)
        go = torch.randn(T, H, device="cuda").to(torch.bfloat16)

        def fn():
            y = _FusedEPMoEFn.apply(x, tw, idx, wg, wu, wd, sg, 0, cap, False)
            y.backward(go)
    elif name in ("gemm-allgather", "gemm-push"):
        # The GEMM variants with a collective inside, with the four "peers" standing in this GPU's memory: the stager
        # warps, the per-row-block counters and the waits run exactly as between GPUs, only NVLink is missing.
        from ._ext import extension
        n, rows, N, K, me = 4, 2048, 8192, 4096, 1
        M = n * rows
        b = torch.randn(N, K, device="cuda").to(torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        flags = torch.empty(M // 128, dtype=torch.int32, device="cuda")
        st = OF.status_word("cuda")
        if name == "gemm-allgather":
            slices = [torch.randn(rows, K, device="cuda").to(torch.bfloat16) for _ in range(n)]
            gathered = torch.empty(M, K, device="cuda", dtype=torch.bfloat16)
            gathered[me * rows:(me + 1) * rows] = slices[me]
            ptrs = [t.data_ptr() for t in slices]
            fn = lambda: extension().gemm_peer(gathered, ptrs, b, c, M, N, K, False, me, flags, st)
        else:
            a = torch.randn(M, K, device="cuda").to(torch.bfloat16)
            slots = [torch.empty(rows, N, device="cuda", dtype=torch.bfloat16) for _ in range(n)]
            ptrs = [t.data_ptr() for t in slots]
            fn = lambda: extension().gemm_push(a, b, None, 0, c, ptrs, M, N, K, False, me, flags, st)
    elif name == "rs-adamw":
        # Reduce-scatter + AdamW + all-gather kernel with a process group of one rank (its only "peer" is itself).
        import os
        import torch.distributed as dist
        from ._ext import extension
        from ..parallel.symm import SymmGroup
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29578")
        if not dist.is_initialized():
            dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        sg = SymmGroup.get(dist.group.WORLD)
        C = extension()
        nel = 128 * 1024 * 1024
        grad, param = sg.empty((nel,), torch.bfloat16), sg.empty((nel,), torch.bfloat16)
        grad.local.normal_(0.0, 1e-3)
        param.local.normal_(0.0, 0.02)
        master = param.local.float()
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        partial = torch.empty(C.rs_adamw_blocks(nel), dtype=torch.float32, device="cuda")
        fn = lambda: C.rs_adamw(grad.ptrs, param.ptrs, 0, master, m, v, 4e-4, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, None,
                                partial, 1, False)
    elif name == "rmsnorm-bwd":
        x = torch.randn(16384, 2048, device="cuda").to(torch.bfloat16).requires_grad_()
        w = torch.ones(2048, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        y = OF.rms_norm(x, w, 1e-5)
        dy = torch.randn_like(y)
        fn = lambda: torch.autograd.grad(y, (x, w), dy, retain_graph=True)
    else:
        raise SystemExit(f"unknown profile case {name}")
    for _ in range(launches):
        fn()
    torch.cuda.synchronize()
    assert OF.check_status("cuda") == 0
    print(f"profile case {name}: {launches} launches done", flush=True)


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "all"
    if what.startswith("profile-"):
        profile_case(what[len("profile-"):])
        sys.exit(0)
    if what in ("gemm", "all"):
        bench_gemm()
    if what in ("grouped", "all"):
        bench_grouped()
    if what in ("attention", "all"):
        bench_attention()
