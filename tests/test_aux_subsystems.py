"""Checkpoint / resume, learning-rate schedule, dataset indexing and host-side failure detection.

Failures are injected on the host only: a rank that raises or never joins, a checkpoint whose completion
marker is missing; nothing here needs (or touches) a GPU."""
import math
import os
import types

import numpy as np
import pytest
import torch

from optimus_lm_b200 import checkpoint as ckpt
from optimus_lm_b200.engine import EngineArgs, TrainEngine, get_learning_rate

MODEL = "allenai/OLMoE-1B-7B-0924--L2-SH0.0625-SA0.25-SE0.125-SC0.25-SI0.25"
OVR = {"vocab_size": 512, "max_position_embeddings": 64}
SEQ = 32


def _engine(**kw):
    args = EngineArgs(model_choice=MODEL, dtype="fp32", context_size=SEQ, lr=1e-3, warmup_steps=0, batch_size=2,
                      config_overrides=OVR, use_fused_ep_alltoall=False, **kw)
    return TrainEngine(args, device=torch.device("cpu"))


def _tokens(n):
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, 512, (n, 2, SEQ), generator=g)


# ---------------------------------------------------------------- learning-rate schedule


def test_lr_schedule_warmup_cosine_linear_constant_and_grad_accumulation():
    a = types.SimpleNamespace(lr=4e-4, min_lr=4e-5, warmup_steps=10, opt_grad_acc_steps=1, lr_schedule="cosine",
                              lr_train_steps=None)
    assert get_learning_rate(0, 110, a) == pytest.approx(4e-5)
    assert get_learning_rate(5, 110, a) == pytest.approx(4e-5 + (4e-4 - 4e-5) * 0.5)
    assert get_learning_rate(10, 110, a) == pytest.approx(4e-4)
    mid = 4e-5 + 0.5 * (1 + math.cos(math.pi * 0.5)) * (4e-4 - 4e-5)
    assert get_learning_rate(60, 110, a) == pytest.approx(mid)
    assert get_learning_rate(110, 110, a) == pytest.approx(4e-5)
    a.lr_schedule = "linear"
    assert get_learning_rate(60, 110, a) == pytest.approx(4e-5 + 0.5 * (4e-4 - 4e-5))
    a.lr_schedule = "constant"
    assert get_learning_rate(60, 110, a) == pytest.approx(4e-4)
    # the schedule runs on optimizer steps: two micro-steps share one value
    a.lr_schedule, a.opt_grad_acc_steps = "cosine", 2
    assert get_learning_rate(10, 220, a) == get_learning_rate(11, 220, a) == pytest.approx(4e-5 + (4e-4 - 4e-5) * 0.5)
    # lr_train_steps decouples the decay horizon from the number of steps actually run
    a.opt_grad_acc_steps, a.lr_train_steps = 1, 210
    assert get_learning_rate(110, 110, a) == pytest.approx(4e-5 + 0.5 * (1 + math.cos(math.pi * 0.5)) * (4e-4 - 4e-5))
    a.lr_schedule = "nope"
    with pytest.raises(ValueError):
        get_learning_rate(50, 110, a)


# ---------------------------------------------------------------- checkpoint / resume


@pytest.mark.parametrize("optimizer", ["unsharded", "pgshard"])
def test_resume_continues_the_loss_curve_exactly(tmp_path, optimizer):
    data = _tokens(6)
    torch.manual_seed(0)
    e = _engine(optimizer=optimizer)
    ref = [e.train_step(data[s]).loss.item() for s in range(6)]

    torch.manual_seed(0)
    e1 = _engine(optimizer=optimizer)
    for s in range(3):
        e1.train_step(data[s])
    name = ckpt.save_checkpoint(str(tmp_path), e1.model, e1.optimizer, e1.pmap, 2, rank=0, verbose=False)
    assert name == "checkpoint1" and ckpt.read_marker(str(tmp_path), name) == 3

    torch.manual_seed(123)  # a different init: everything must come from the files
    e2 = _engine(optimizer=optimizer, seed=5)
    step, got = ckpt.load_checkpoint(str(tmp_path), e2.model, e2.optimizer, e2.pmap, rank=0, verbose=False)
    assert (step, got) == (3, "checkpoint1")
    e2.step_id = step
    cont = [e2.train_step(data[s]).loss.item() for s in range(3, 6)]
    assert cont == pytest.approx(ref[3:], abs=1e-6)


def test_hot_checkpoints_alternate_and_an_unfinished_one_is_ignored(tmp_path):
    e = _engine(optimizer="unsharded")
    exp = str(tmp_path)
    assert ckpt.load_checkpoint(exp, e.model, e.optimizer, e.pmap, rank=0, verbose=False) == (0, None)
    assert ckpt.save_checkpoint(exp, e.model, e.optimizer, e.pmap, 9, rank=0, verbose=False) == "checkpoint1"
    assert ckpt.save_checkpoint(exp, e.model, e.optimizer, e.pmap, 19, rank=0, verbose=False) == "checkpoint2"
    assert ckpt.save_checkpoint(exp, e.model, e.optimizer, e.pmap, 29, rank=0, verbose=False) == "checkpoint1"
    assert ckpt.choose_checkpoint_for_reading(exp) == "checkpoint1"
    # a writer that died before the marker was written: the other checkpoint is the one to resume from
    os.remove(os.path.join(exp, "checkpoints", "checkpoint1", ckpt.MARKER))
    assert ckpt.choose_checkpoint_for_reading(exp) == "checkpoint2"
    step, name = ckpt.load_checkpoint(exp, e.model, e.optimizer, e.pmap, rank=0, verbose=False)
    assert (step, name) == (20, "checkpoint2")
    assert ckpt.cold_checkpoint_name(61499, e.pmap, 8, 4096).startswith("step61500-tokens")


def _dp_resume_worker(rank, world, exp, ref):
    import torch.distributed as dist
    data = _tokens(6)
    e = _engine(optimizer="pgshard", data_parallelism=world)
    for s in range(3):
        e.train_step(data[s])
    ckpt.save_checkpoint(exp, e.model, e.optimizer, e.pmap, 2, rank=rank, verbose=False)
    e2 = _engine(optimizer="pgshard", data_parallelism=world, seed=9)
    step, _ = ckpt.load_checkpoint(exp, e2.model, e2.optimizer, e2.pmap, rank=rank, use_broadcast=True, verbose=False)
    assert step == 3
    e2.step_id = step
    for s in range(3, 6):
        loss = e2.train_step(data[s]).loss.detach().clone()
        dist.all_reduce(loss)
        assert abs(loss.item() / world - ref[s]) < 1e-5
    if rank == 0:
        files = sorted(os.listdir(os.path.join(exp, "checkpoints", "checkpoint1")))
        assert "optimizer_checkpoint_shard-0.pth" in files and "optimizer_checkpoint_shard-1.pth" in files


def test_sharded_optimizer_state_resumes_under_data_parallelism(tmp_path):
    from dist_utils import run_distributed
    torch.manual_seed(0)
    data = _tokens(6)
    e = _engine(optimizer="unsharded")
    ref = [e.train_step(data[s]).loss.item() for s in range(6)]   # both DP ranks see the same batch
    run_distributed(_dp_resume_worker, 2, str(tmp_path), ref)


def _buffer_broadcast_worker(rank, world, exp):
    """A persistent buffer (the stand-in for DeepSeek-V3's routing bias) must reach the replicas that do not read
    the model file when the parameters travel over the data-parallel group."""
    import torch.distributed as dist
    for allreduce in (False, True):
        e = _engine(optimizer="pgshard", data_parallelism=world)
        e.model.register_buffer("routing_bias", torch.full((4,), 0.25 if rank == 0 else -1.0))
        # every rank writes its part of the checkpoint through the regular path; only dp_ind 0's model file is read
        ckpt.save_checkpoint(exp, e.model, e.optimizer, e.pmap, 0, rank=rank, verbose=False)
        e2 = _engine(optimizer="pgshard", data_parallelism=world, seed=5)
        e2.model.register_buffer("routing_bias", torch.full((4,), 7.0))
        ckpt.load_checkpoint(exp, e2.model, e2.optimizer, e2.pmap, rank=rank, use_broadcast=True,
                             use_allreduce_in_broadcast=allreduce, verbose=False)
        assert torch.equal(e2.model.routing_bias, torch.full((4,), 0.25)), (rank, allreduce, e2.model.routing_bias)


def test_broadcast_load_carries_persistent_buffers(tmp_path):
    from dist_utils import run_distributed
    run_distributed(_buffer_broadcast_worker, 2, str(tmp_path))


# ---------------------------------------------------------------- datasets


def test_data_parallel_indexing_and_sharded_dataset_agree(tmp_path):
    from optimus_lm_b200.datasets import (PclDataPrallelDataset, PclShardedDataParallelDataset, SyntheticTokenDataset,
                                          write_synthetic_dataset_dir)
    from optimus_lm_b200 import data_prep
    C = 16
    ddir = write_synthetic_dataset_dir(str(tmp_path), vocab_size=100, context_size=C, num_files=3, instances_per_file=10)
    layout = types.SimpleNamespace()
    a0 = PclDataPrallelDataset(ddir, 3, C, dp_size=2, dp_ind=0)
    a1 = PclDataPrallelDataset(ddir, 3, C, dp_size=2, dp_ind=1)
    full = PclDataPrallelDataset(ddir, 3, C)
    assert full.num_instances == 10 + 11 + 12
    # rank r of d sees the serial instances r, r+d, r+2d, ...
    assert np.array_equal(a0[3], full[6]) and np.array_equal(a1[3], full[7])
    a0.set_base_dp_idx(5)
    assert np.array_equal(a0[0], full[10])
    s = SyntheticTokenDataset(100, C, dp_size=2, dp_ind=1, seed=1)
    assert s[4].shape == (C,) and np.array_equal(s[4], SyntheticTokenDataset(100, C, dp_size=2, dp_ind=1, seed=1)[4])
    assert not np.array_equal(s[4], s[5])


# ---------------------------------------------------------------- failure detection (host side)


def test_soft_failure_report_lists_the_nodes_of_bad_ranks(tmp_path, monkeypatch):
    import dist_train
    monkeypatch.setenv("OPTIMUS_LAUNCH_INFO_DIR", str(tmp_path))
    monkeypatch.setenv("PBS_JOBID", "777.sched")
    pmap = types.SimpleNamespace(rank_to_node_list=["nodeA", "nodeA", "nodeB", "nodeC"])
    flags = torch.tensor([0, 0, 1, 1])
    dist_train.report_soft_failures(flags, pmap, rank=1, world_size=4)       # only rank 0 writes
    assert not os.path.exists(tmp_path / "777")
    dist_train.report_soft_failures(flags, pmap, rank=0, world_size=4)
    assert (tmp_path / "777" / "failed_soft_nodes.txt").read_text().split() == ["nodeB", "nodeC"]
    # the launcher's screen reads the same file
    from optimus_lm_b200 import launcher
    assert launcher.read_soft_failures(str(tmp_path / "777")) == ["nodeB", "nodeC"]


def _absent_rank_worker(rank, world):
    import datetime
    import torch.distributed as dist
    # a second group with a short timeout, as the driver's --dist_timeout_s sets for the whole job
    g = dist.new_group(ranks=list(range(world)), backend="gloo", timeout=datetime.timedelta(seconds=3))
    t = torch.ones(1)
    dist.all_reduce(t, group=g)           # everybody is here: works
    assert t.item() == world
    if rank == 1:
        return                            # this rank stops taking part between steps
    with pytest.raises(Exception):
        dist.all_reduce(t, group=g)       # the survivor's next collective ends with an error, not a hang


def test_a_rank_that_stops_is_detected_by_the_collective_timeout():
    from dist_utils import run_distributed
    import time
    t0 = time.time()
    run_distributed(_absent_rank_worker, 2)
    assert time.time() - t0 < 120


def _raising_worker(rank, world):
    if rank == 1:
        raise RuntimeError("injected failure on rank 1")


def test_a_rank_that_raises_is_reported_by_the_spawn_helper():
    from dist_utils import run_distributed
    with pytest.raises(AssertionError, match="injected failure on rank 1"):
        run_distributed(_raising_worker, 2)


def test_torch_adamw_path_and_hf_model_path():
    """``--opt_use_pt_optimizer`` (torch.optim.AdamW through the engine) and ``--use_hf_model`` (the transformers
    implementation built without the hub) both train: the loss of a repeated batch falls."""
    from optimus_lm_b200.engine import EngineArgs, TrainEngine
    torch.manual_seed(0)
    tag = "allenai/OLMoE-1B-7B-0924--L2-SH0.0625-SA0.25-SE0.125-SC0.0625-SI0.125"
    over = {"vocab_size": 256, "max_position_embeddings": 64}
    ids = torch.randint(0, 256, (2, 32))
    for hf in (False, True):
        eng = TrainEngine(EngineArgs(model_choice=tag, dtype="fp32", batch_size=2, context_size=32, optimizer="pt",
                                     warmup_steps=0, lr=3e-3, use_hf_model=hf, config_overrides=over))
        losses = [float(eng.train_step(ids).loss) for _ in range(6)]
        assert losses[-1] < losses[0] - 0.2, (hf, losses)
        if hf:
            import transformers
            assert isinstance(eng.model, transformers.PreTrainedModel)
