"""Multi-GPU tests (2, 4 and 8 ranks, one process per GPU, NCCL): the fused peer-memory paths against the
NCCL-only paths of the same computation.  A case is skipped when fewer GPUs are visible than it needs."""
import os
import socket
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, args, errq):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), OLB_SYMM_CANARY="1")     # guard bands around every symmetric buffer
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        globals()[fn_name](rank, world, *args)
        dist.barrier()
        torch.cuda.synchronize()
        from optimus_lm_b200.parallel.symm import SymmGroup
        assert SymmGroup.all_canaries_intact(), "a kernel wrote outside a symmetric buffer (guard band overwritten)"
    except Exception:
        errq.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def _run(fn_name, world, *args, timeout=600):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, args, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            errors.append((-1, "timeout"))
        elif p.exitcode != 0 and not errors:
            errors.append((-1, f"exit code {p.exitcode}"))
    assert not errors, "\n".join(f"[rank {r}]\n{tb}" for r, tb in errors)


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _max_err(a, b):
    """Largest element-wise difference relative to the reference's largest element: a few wrong rows show up here
    even when the norm-wise error stays small."""
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-12)).item()


WORLDS = [2, 4, 8]


# ----------------------------------------------------------------------------- workers
def w_symm_barrier_and_pull(rank, world):
    import torch.distributed as dist
    from optimus_lm_b200.ops import functional as OF
    from optimus_lm_b200.ops import extension
    from optimus_lm_b200.parallel.symm import SymmGroup
    sg = SymmGroup.get(dist.group.WORLD)
    st = sg.empty((world * 64, 256), torch.bfloat16)
    st.local.fill_(float(rank + 1))
    for _ in range(5):
        sg.barrier(0)
    out = torch.empty(64, 256, dtype=torch.bfloat16, device="cuda")
    extension().pull_reduce_rows(st.ptrs, rank * 64, 256, out)
    torch.cuda.synchronize()
    assert torch.all(out.float() == sum(range(1, world + 1)))
    assert OF.check_status("cuda") == 0


def w_fused_ep_vs_allgather(rank, world):
    import torch.distributed as dist
    from optimus_lm_b200.mapper import ParallelDpPpEpTpMapper
    from optimus_lm_b200.models.olmoe.configuration_olmoe import OlmoeParallelConfig
    from optimus_lm_b200.models.common.moe import FastOlmoeParallelSparseMoeBlock
    from optimus_lm_b200.ops import functional as OF
    pmap = ParallelDpPpEpTpMapper(1, 1, world, 1, rank=rank, create_groups=True)
    cfg = OlmoeParallelConfig(hidden_size=256, intermediate_size=512, num_experts=16, num_experts_per_tok=4,
                              expert_parallelism=world, use_fast_moe=True, use_merged_mlp_in_fast_moe=True,
                              output_router_logits=True, moe_capacity_factor=0.0)
    torch.manual_seed(0)
    blk = FastOlmoeParallelSparseMoeBlock(cfg, pmap).cuda().to(torch.bfloat16)
    with torch.no_grad():
        for name, p in blk.named_parameters():
            g = torch.Generator(device="cuda").manual_seed(hash(name) % 1000 + (rank if "experts" in name else 0))
            p.copy_(torch.randn(p.shape, device="cuda", generator=g) * 0.05)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    x0 = torch.randn(2, 96, 256, device="cuda", generator=g).to(torch.bfloat16)
    go = torch.randn(2, 96, 256, device="cuda", generator=g).to(torch.bfloat16)
    res = {}
    for transport in ("allgather", "alltoall"):
        blk.ep_transport = transport
        blk.zero_grad()
        x = x0.clone().requires_grad_()
        y, _ = blk(x)
        y.backward(go)
        res[transport] = (y.detach().clone(), x.grad.clone(), {n: p.grad.clone() for n, p in blk.named_parameters()})
    ya, xa, ga = res["allgather"]
    yb, xb, gb = res["alltoall"]
    assert _rel(yb, ya) < 2e-2, _rel(yb, ya)
    assert _rel(xb, xa) < 2e-2, _rel(xb, xa)
    assert _max_err(yb, ya) < 5e-2, _max_err(yb, ya)
    assert _max_err(xb, xa) < 5e-2, _max_err(xb, xa)
    for n in ga:
        assert _rel(gb[n], ga[n]) < 3e-2, (n, _rel(gb[n], ga[n]))
        assert _max_err(gb[n], ga[n]) < 8e-2, (n, _max_err(gb[n], ga[n]))
    assert OF.check_status("cuda") == 0


def w_capacity_overflow_is_reported(rank, world):
    """A fixed capacity below the routed load must raise ST_OVERFLOW (6) in the status word of the overloaded rank and
    leave the GPU usable; with the default (capacity factor 0) the same routing runs clean."""
    import torch.distributed as dist
    from optimus_lm_b200.mapper import ParallelDpPpEpTpMapper
    from optimus_lm_b200.models.olmoe.configuration_olmoe import OlmoeParallelConfig
    from optimus_lm_b200.models.common.moe import FastOlmoeParallelSparseMoeBlock
    from optimus_lm_b200.ops import functional as OF
    pmap = ParallelDpPpEpTpMapper(1, 1, world, 1, rank=rank, create_groups=True)
    seen = {}
    for factor in (0.25, 0.0):
        cfg = OlmoeParallelConfig(hidden_size=256, intermediate_size=512, num_experts=16, num_experts_per_tok=4,
                                  expert_parallelism=world, use_fast_moe=True, use_merged_mlp_in_fast_moe=True,
                                  output_router_logits=True, moe_capacity_factor=factor)
        torch.manual_seed(0)
        blk = FastOlmoeParallelSparseMoeBlock(cfg, pmap).cuda().to(torch.bfloat16)
        with torch.no_grad():
            for name, p in blk.named_parameters():
                g = torch.Generator(device="cuda").manual_seed(hash(name) % 1000)
                p.copy_(torch.randn(p.shape, device="cuda", generator=g) * 0.05)
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        x = torch.randn(4, 512, 256, device="cuda", generator=g).to(torch.bfloat16)
        y, _ = blk(x)
        torch.cuda.synchronize()
        st = torch.tensor([float(OF.check_status("cuda"))], device="cuda")
        dist.all_reduce(st, op=dist.ReduceOp.MAX)
        seen[factor] = int(st.item())
        assert torch.isfinite(y.float()).all() or factor > 0
    assert seen[0.25] == 6, seen        # a quarter of the balanced share cannot hold the routed rows
    assert seen[0.0] == 0, seen


def w_fused_optimizer_vs_nccl(rank, world):
    import copy
    import torch.distributed as dist
    from optimus_lm_b200.engine import EngineArgs, TrainEngine
    from optimus_lm_b200.ops import functional as OF
    losses = {}
    os.environ["OLB_PARAM_AG"] = "gemm"      # also the parameter all-gather inside the consuming GEMM (off by default)
    os.environ["OLB_MULTIMEM"] = "1" if world >= 4 else "0"     # and, from 4 ranks, the NVLS form of the update kernel
    for fused in (False, True):
        args = EngineArgs(model_choice="allenai/OLMoE-1B-7B-0924--L2-SH0.125-SA0.25-SE0.125-SC0.25-SI0.5",
                          batch_size=2, context_size=128, optimizer="pgshard", warmup_steps=2, expert_parallelism=world,
                          use_fused_ep_alltoall=fused, use_fused_optimizer=fused,
                          config_overrides={"vocab_size": 1024, "max_position_embeddings": 128,
                                            "output_router_logits": True})
        eng = TrainEngine(args)
        g = torch.Generator().manual_seed(5 + rank)
        out = []
        for s in range(5):
            tok = torch.randint(0, 1024, (2, 128), generator=g)
            o = eng.train_step(tok.cuda())
            out.append((o.loss.item(), o.grad_norm.item()))
        losses[fused] = out
        assert eng.check_device_status() == 0
    for (la, na), (lb, nb) in zip(losses[False], losses[True]):
        assert abs(la - lb) < 3e-2 * abs(la), (losses)
        assert abs(na - nb) < 5e-2 * abs(na) + 1e-3, (losses)


def w_tp_fused_mlp_vs_nccl(rank, world):
    """All-gather -> GEMM and GEMM -> reduce-scatter over peer memory against the NCCL collectives + local GEMMs."""
    import torch.distributed as dist
    from optimus_lm_b200.models.common.comms_ptfunctions import (forward_allgather_backward_reducescatter,
                                                                forward_reducescatter_backward_allgather)
    from optimus_lm_b200.ops import functional as OF
    from optimus_lm_b200.parallel import tp_fused
    T_loc, H, I = 256, 512, 384
    grp = dist.group.WORLD
    gen = torch.Generator(device="cuda").manual_seed(7)          # same weights' seed on every rank, sliced per rank
    wg_full = (torch.randn(world * I, H, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    wu_full = (torch.randn(world * I, H, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    wd_full = (torch.randn(H, world * I, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
    gen = torch.Generator(device="cuda").manual_seed(100 + rank)
    x0 = torch.randn(T_loc, H, device="cuda", generator=gen).to(torch.bfloat16)
    go = torch.randn(T_loc, H, device="cuda", generator=gen).to(torch.bfloat16)
    res = {}
    for fused in (False, True):
        wg = wg_full[rank * I:(rank + 1) * I].clone().requires_grad_()
        wu = wu_full[rank * I:(rank + 1) * I].clone().requires_grad_()
        wd = wd_full[:, rank * I:(rank + 1) * I].contiguous().clone().requires_grad_()
        x = x0.clone().requires_grad_()
        if fused:
            assert tp_fused.usable(x, grp, (wg, wu, wd))
            y = tp_fused.ag_swiglu_mlp_rs(x, wg, wu, wd, rank, world, grp)
        else:
            xa = forward_allgather_backward_reducescatter.apply(x, rank, world, grp, False)
            h = OF.swiglu(OF.linear(xa, wg), OF.linear(xa, wu))
            y = forward_reducescatter_backward_allgather.apply(OF.linear(h, wd), rank, world, grp, False, False)
        y.backward(go)
        res[fused] = [t.detach().clone() for t in (y, x.grad, wg.grad, wu.grad, wd.grad)]
    for name, a, b in zip(("y", "dx", "dwg", "dwu", "dwd"), res[False], res[True]):
        assert _rel(b, a) < 2e-2, (name, _rel(b, a))
    assert OF.check_status("cuda") == 0


def w_dense_tp_sequence_parallel_vs_allreduce(rank, world):
    """Llama under tensor parallelism: the sequence-parallel execution with all-gather -> GEMM / GEMM -> reduce-scatter
    launches against the reference form (replicated activations, all-reduces of the collective library)."""
    from optimus_lm_b200.engine import EngineArgs, TrainEngine
    runs = {}
    for fused in (False, True):
        if fused:
            os.environ.pop("OLB_DISABLE_TP_FUSED", None)
        else:
            os.environ["OLB_DISABLE_TP_FUSED"] = "1"
        eng = TrainEngine(EngineArgs(model_choice="meta-llama/Llama-3.2-1B--L2", dtype="bf16", context_size=512,
                                     batch_size=2, warmup_steps=0, lr=1e-3, seed=0, optimizer="shard",
                                     tensor_parallelism=world))
        g = torch.Generator().manual_seed(11)
        out = []
        for _ in range(4):
            ids = torch.randint(0, 32000, (2, 512), generator=g)
            o = eng.train_step(ids.cuda())
            out.append((float(o.loss), float(o.grad_norm)))
        assert eng.check_device_status() == 0
        runs[fused] = out
    os.environ.pop("OLB_DISABLE_TP_FUSED", None)
    for (la, na), (lb, nb) in zip(runs[False], runs[True]):
        assert abs(la - lb) < 3e-2 * abs(la), runs
        assert abs(na - nb) < 6e-2 * abs(na) + 1e-3, runs


LAYOUTS = {
    "olmo_dp2_shard": ("allenai/OLMo-1B-hf--L2", dict(optimizer="shard", batch_size=4)),
    "olmoe_pp2_1f1b": ("allenai/OLMoE-1B-7B-0924--L4-SH0.5-SI0.5",
                       dict(optimizer="pgshard", pipeline_parallelism=2, pp_scheme="1f1b", batch_size=4,
                            micro_batch_size=2, use_fast_moe=True, use_merged_mlp_in_fast_moe=True)),
    "deepseek_v3_ep2": ("deepseek-ai/DeepSeek-V3--L3-DL1-N16-K4-MI512-A16-SE1-H1024-I2048",
                        dict(optimizer="pgshard", expert_parallelism=2, batch_size=2, use_fast_moe=True,
                             use_merged_mlp_in_fast_moe=True)),
    "llama_tp2": ("meta-llama/Llama-3.2-1B--L2", dict(optimizer="shard", tensor_parallelism=2, batch_size=2)),
}


def w_family_layout(rank, world, name):
    """A few optimizer steps of a model family in a two-GPU layout on the kernel path: the loss of a repeated
    batch falls and no kernel reports an error."""
    from optimus_lm_b200.engine import EngineArgs, TrainEngine
    model, kw = LAYOUTS[name]
    eng = TrainEngine(EngineArgs(model_choice=model, dtype="bf16", context_size=512, warmup_steps=0, lr=1e-3, seed=0, **kw))
    g = torch.Generator().manual_seed(11 + 7 * eng.pmap.dp_ind)   # one batch per data-parallel replica
    ids = torch.randint(0, 32000, (kw["batch_size"], 512), generator=g)
    losses = []
    for _ in range(5):
        o = eng.train_step(ids.cuda())
        if o.loss is not None:
            losses.append(float(o.loss))
    assert eng.check_device_status() == 0
    if losses:       # ranks that are not on the last pipeline stage see no loss
        assert all(l == l for l in losses) and losses[-1] < losses[0] - 0.3, losses


# ----------------------------------------------------------------------------- tests
@pytest.mark.parametrize("world", WORLDS)
def test_symm_barrier_and_pull_reduce(world):
    _run("w_symm_barrier_and_pull", world)


@pytest.mark.parametrize("world", WORLDS)
def test_fused_ep_moe_matches_allgather_transport(world):
    _run("w_fused_ep_vs_allgather", world)


def test_capacity_overflow_is_reported_and_default_cannot_overflow():
    _run("w_capacity_overflow_is_reported", 2)


@pytest.mark.parametrize("world", WORLDS)
def test_fused_engine_matches_nccl_engine(world):
    _run("w_fused_optimizer_vs_nccl", world)


@pytest.mark.parametrize("world", WORLDS)
def test_tp_fused_mlp_matches_nccl_path(world):
    _run("w_tp_fused_mlp_vs_nccl", world)


@pytest.mark.parametrize("world", WORLDS)
def test_dense_tensor_parallel_sequence_parallel_form_matches_allreduce_form(world):
    _run("w_dense_tp_sequence_parallel_vs_allreduce", world)


@pytest.mark.parametrize("name", list(LAYOUTS))
def test_model_families_in_two_gpu_layouts(name):
    _run("w_family_layout", 2, name)
