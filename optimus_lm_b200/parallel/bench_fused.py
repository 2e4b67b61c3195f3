"""Timings of the fused compute + collective paths against the same computation on NCCL collectives, with the
fraction of each path's roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29555 \
        -m optimus_lm_b200.parallel.bench_fused [ep,adamw,tp|all]

Every number is a CUDA-event time on the launching stream after warm-up, median of the iterations, maximum over
ranks.  The roofline of a path is the slower of (its FLOPs / the GEMM peak) and (the bytes that cross NVLink into
or out of one GPU / the peer-copy bandwidth); for the optimizer step the HBM traffic of the update takes the
place of the FLOPs.  The peaks are read from ``MEASURED_PEAKS.json`` at the repository root when it is there
(cuBLAS bf16 sustained rate, copy bandwidth), otherwise 1400 TFLOP/s and 6650 GB/s; NVLink peer copy: 770 GB/s per
direction.

  ep    : one OLMoE-1B-7B MoE layer (T=16384 tokens per rank, H=2048, 64 experts top-8, I=1024), forward +
          backward: peer-memory dispatch/combine (``parallel/ep_alltoall.py``) against the all-gather /
          reduce-scatter transport of the reference (optimus/models/common/moe.py:478-480, 607).
  adamw : gradient reduce-scatter + 1/N + norm partial + sharded AdamW + parameter all-gather as one kernel
          (``csrc/comm_p2p.cu: rs_adamw_kernel``) against ``reduce_scatter_tensor`` + the local AdamW kernel +
          ``all_gather_into_tensor`` (optimus/optimizers.py:364-365, 455-494).
  tp    : all-gather -> gate/up GEMM -> SwiGLU -> down GEMM -> reduce-scatter (``parallel/tp_fused.py``) against
          the NCCL collectives around local GEMMs (optimus/models/deepseek_v3/modeling_deepseek_v3.py:88-112).
"""
import json
import os
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    tf, bw, src = 1400.0, 6650.0, "fallback"
    try:
        with open(path) as f:
            d = json.load(f)
        tf = float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", tf)))
        bw = float(d.get("hbm_gbs", bw))
        src = "measured"
    except (OSError, ValueError):
        pass
    return tf, bw, src


def _time(fn, iters=8, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def _report(name, t_fused, t_nccl, flops, link_bytes, hbm_bytes=0.0):
    tf, bw, src = _peaks()
    t_compute = flops / (tf * 1e12) * 1e3
    t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e3
    t_hbm = hbm_bytes / (bw * 1e9) * 1e3
    roof = max(t_compute, t_link, t_hbm)
    if dist.get_rank() == 0:
        print(json.dumps({"path": name, "n_gpus": dist.get_world_size(), "fused_ms": round(t_fused, 3),
                          "nccl_ms": round(t_nccl, 3), "speedup": round(t_nccl / t_fused, 3),
                          "roofline_ms": {"compute": round(t_compute, 3), "nvlink": round(t_link, 3),
                                          "hbm": round(t_hbm, 3)},
                          "fraction_of_roofline": round(roof / t_fused, 3), "peaks": src}), flush=True)


def bench_ep():
    from ..mapper import ParallelDpPpEpTpMapper
    from ..models.common.moe import FastOlmoeParallelSparseMoeBlock
    from ..models.olmoe.configuration_olmoe import OlmoeParallelConfig
    rank, world = dist.get_rank(), dist.get_world_size()
    T, H, I, E, K = 16384, 2048, 1024, 64, 8
    pmap = ParallelDpPpEpTpMapper(1, 1, world, 1, rank=rank, create_groups=True)
    cfg = OlmoeParallelConfig(hidden_size=H, intermediate_size=I, num_experts=E, num_experts_per_tok=K,
                              expert_parallelism=world, use_fast_moe=True, use_merged_mlp_in_fast_moe=True,
                              output_router_logits=True)
    torch.manual_seed(0)
    blk = FastOlmoeParallelSparseMoeBlock(cfg, pmap).cuda().to(torch.bfloat16)
    with torch.no_grad():
        for p in blk.parameters():
            p.normal_(0.0, 0.02)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x = torch.randn(4, T // 4, H, device="cuda", generator=g).to(torch.bfloat16).requires_grad_()
    go = torch.randn(4, T // 4, H, device="cuda", generator=g).to(torch.bfloat16)

    def step():
        y, _ = blk(x)
        y.backward(go)

    res = {}
    for transport in ("allgather", "alltoall"):
        if world == 1 and transport == "allgather":
            continue
        blk.ep_transport = transport
        res[transport] = _time(step)
    from ..ops import functional as OF
    assert OF.check_status("cuda") == 0
    flops = 3 * 2.0 * T * K * 3 * H * I                       # forward + two backward GEMMs per projection
    # rows this rank pulls from the others: dispatch (fwd x, bwd dy) and combine (fwd y, bwd dx), balanced routing
    link = 4 * T * K * H * 2 * (world - 1) / world
    _report("ep_moe_layer_fwd_bwd", res["alltoall"], res.get("allgather", res["alltoall"]), flops, link)


def bench_adamw():
    from ..ops import functional as OF
    from ..ops._ext import extension
    from .symm import SymmGroup
    rank, world = dist.get_rank(), dist.get_world_size()
    C = extension()
    n = 512 * 1024 * 1024 // world * world                      # 512 Mi bf16 parameters (1 GiB), as one family
    shard = n // world
    sg = SymmGroup.get(dist.group.WORLD)
    grad = sg.empty((n,), torch.bfloat16)
    param = sg.empty((n,), torch.bfloat16)
    grad.local.normal_(0.0, 1e-3)
    param.local.normal_(0.0, 0.02)
    master = param.local[rank * shard:(rank + 1) * shard].float()
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    partial = torch.empty(C.rs_adamw_blocks(shard), dtype=torch.float32, device="cuda")
    hp = dict(lr=4e-4, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1)

    from .fused_optimizer import use_multimem
    nvls = use_multimem(world) and bool(grad.multicast_ptr and param.multicast_ptr)
    mcg, mcp = (grad.multicast_ptr, param.multicast_ptr) if nvls else (0, 0)
    if rank == 0:
        print(f"rs_adamw: {'multimem.ld_reduce / multimem.st through the NVSwitch' if nvls else 'plain peer loads and stores'}",
              flush=True)

    def fused():
        sg.barrier(8)
        C.rs_adamw(grad.ptrs, param.ptrs, rank * shard, master, m, v, hp["lr"], hp["beta1"], hp["beta2"], hp["eps"],
                   hp["wd"], 1, 1.0 / world, None, partial, 1, False, mcg, mcp)
        partial.sum()
        sg.barrier(9)

    g_shard = torch.empty(shard, dtype=torch.bfloat16, device="cuda")
    p_shard = torch.empty(shard, dtype=torch.bfloat16, device="cuda")

    def nccl():
        dist.reduce_scatter_tensor(g_shard, grad.local)
        OF.sum_of_squares(g_shard, 1.0 / world)
        OF.adamw_step(g_shard, master, m, v, p_shard, hp["lr"], hp["beta1"], hp["beta2"], hp["eps"], hp["wd"], 1,
                      grad_scale=1.0 / world)
        dist.all_gather_into_tensor(param.local, p_shard)

    t_f = _time(fused)
    t_n = _time(nccl)
    assert OF.check_status("cuda") == 0
    link = shard * 2.0 * (world - 1)                            # gradients in; the same number of parameter bytes out
    hbm = shard * (3 * 4 * 2 + 2 + 2)                           # master, m, v read + written; local gradient; parameter
    _report("rs_adamw_ag_512Mi_params", t_f, t_n, 0.0, link, hbm)


def bench_tp():
    from ..models.common.comms_ptfunctions import (forward_allgather_backward_reducescatter,
                                                   forward_reducescatter_backward_allgather)
    from ..ops import functional as OF
    from . import tp_fused
    rank, world = dist.get_rank(), dist.get_world_size()
    if world == 1:
        return
    T_loc, H, I_full = 4096, 7168, 18432                        # DeepSeek-V3 dense MLP, sequence 4096 per rank
    I = I_full // world // 128 * 128
    grp = dist.group.WORLD
    gen = torch.Generator(device="cuda").manual_seed(7 + rank)
    wg = (torch.randn(I, H, device="cuda", generator=gen) * 0.02).to(torch.bfloat16).requires_grad_()
    wu = (torch.randn(I, H, device="cuda", generator=gen) * 0.02).to(torch.bfloat16).requires_grad_()
    wd = (torch.randn(H, I, device="cuda", generator=gen) * 0.02).to(torch.bfloat16).requires_grad_()
    x = torch.randn(T_loc, H, device="cuda", generator=gen).to(torch.bfloat16).requires_grad_()
    go = torch.randn(T_loc, H, device="cuda", generator=gen).to(torch.bfloat16)
    assert tp_fused.usable(x, grp, (wg, wu, wd))

    def fused():
        tp_fused.ag_swiglu_mlp_rs(x, wg, wu, wd, rank, world, grp).backward(go)

    def nccl():
        xa = forward_allgather_backward_reducescatter.apply(x, rank, world, grp, False)
        h = OF.swiglu(OF.linear(xa, wg), OF.linear(xa, wu))
        forward_reducescatter_backward_allgather.apply(OF.linear(h, wd), rank, world, grp, False, False).backward(go)

    t_f = _time(fused)
    t_n = _time(nccl)
    assert OF.check_status("cuda") == 0
    flops = 3 * 2.0 * (T_loc * world) * 3 * H * I
    # forward: gather x, reduce-scatter y; backward: gather dy, reduce-scatter dx (bf16 rows of the other ranks)
    link = 4 * T_loc * (world - 1) * H * 2.0
    _report("tp_ag_swiglu_mlp_rs_fwd_bwd", t_f, t_n, flops, link)


def main():
    what = (sys.argv[1] if len(sys.argv) > 1 else "all").split(",")
    if "all" in what:
        what = ["ep", "adamw", "tp"]
    from ..dutils import setup_distributed
    setup_distributed("nccl", timeout_s=600)
    if "ep" in what:
        bench_ep()
    if "adamw" in what:
        bench_adamw()
    if "tp" in what:
        bench_tp()
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
