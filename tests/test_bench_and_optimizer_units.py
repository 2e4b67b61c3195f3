"""Small host-side checks: the named benchmark configurations, the bookkeeping of optimizer updates that ran early,
and the gradient norm taken as a by-product of the AdamW pass."""
import importlib.util
import os

import pytest
import torch

from optimus_lm_b200.ops import functional as OF

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_named_configurations():
    b = _bench()
    kw, mb, seq, vocab, metric, tag = b.named_config("olmoe_ep", 8)
    assert (kw["expert_parallelism"], kw["optimizer"], mb, seq, vocab, tag) == (8, "pgshard", 4, 4096, 50304, "ep8")
    assert metric == b.METRIC
    kw, mb, seq, vocab, metric, tag = b.named_config("olmo1b_dp", 8)
    assert (kw["data_parallelism"], kw["optimizer"], mb, seq, tag) == (8, "shard", 8, 2048, "dp8")
    kw, mb, seq, _, _, tag = b.named_config("olmoe_pp_ep", 8)
    assert (kw["pipeline_parallelism"], kw["expert_parallelism"], kw["micro_batch_size"], mb, tag) == (4, 2, 4, 32, "pp4xep2")
    kw, *_ , tag = b.named_config("olmoe_pp_ep", 2)
    assert (kw["pipeline_parallelism"], kw["expert_parallelism"], tag) == (2, 1, "pp2xep1")
    with pytest.raises(AssertionError):
        b.named_config("dsv3_reduced_ep", 2)      # 34 G expert parameters do not fit fewer than 8 GPUs
    with pytest.raises(SystemExit):
        b.named_config("nope", 1)


def test_pending_ranges_are_the_complement_of_early_updates():
    from optimus_lm_b200.optimizers import _FlatAdamWEngine, _Slice

    class Fam:
        pass

    eng = _FlatAdamWEngine.__new__(_FlatAdamWEngine)
    fam, sl = Fam(), _Slice(0, 1000, 1000, 0)
    assert eng._pending_ranges(fam, sl) == [(0, 1000)]
    eng._early_done = {id(fam): [(600, 800), (100, 200)]}
    assert eng._pending_ranges(fam, sl) == [(0, 100), (200, 600), (800, 1000)]
    eng._early_done = {id(fam): [(0, 400), (400, 1000)]}
    assert eng._pending_ranges(fam, sl) == []


def test_adamw_norm_by_product_on_the_plain_path():
    torch.manual_seed(0)
    n = 64
    g = torch.randn(n)
    master, m, v = torch.randn(n), torch.zeros(n), torch.zeros(n)
    p = master.clone()
    acc = torch.full((1,), 2.0)
    OF.adamw_step(g, master, m, v, p, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, grad_scale=0.5, norm_out=acc)
    assert torch.allclose(acc, 2.0 + (g * 0.5).pow(2).sum().reshape(1))
    assert torch.equal(p, master)


@pytest.mark.parametrize("dp", [2, 3, 4, 5, 6, 7, 8])
def test_fused_step_alignment_predicate(dp):
    """The fused reduce-scatter + AdamW kernel moves 16-byte vectors: sub-sharded chunks whose per-rank part is not a
    multiple of 8 elements (DP 3, 5, 6, 7 with a power-of-two chunk limit) must be left to the NCCL path."""
    from optimus_lm_b200.optimizers import _Family, _FamilySpec
    from optimus_lm_b200.parallel.fused_optimizer import slices_aligned

    params = [torch.nn.Parameter(torch.zeros(4096)), torch.nn.Parameter(torch.zeros(1000))]
    sub = _Family(_FamilySpec("", params, None, dp, dp - 1, 1.0, chunk_limit=2048, chunk_round=1), torch.bfloat16, "cpu",
                  512, keep_state=False)
    part = (2048 // dp * dp) // dp
    assert slices_aligned([sub]) == (part % 8 == 0 and ((dp - 1) * part) % 8 == 0)
    # the plain sharded layout rounds every shard to 512 elements and is always aligned
    params = [torch.nn.Parameter(torch.zeros(4096)), torch.nn.Parameter(torch.zeros(1000))]
    plain = _Family(_FamilySpec("", params, None, dp, dp - 1, 1.0), torch.bfloat16, "cpu", 512, keep_state=False)
    assert slices_aligned([plain])


def test_debug_shapes_do_not_carry_the_benchmark_metric_name():
    import types
    b = _bench()
    opts = types.SimpleNamespace(config="olmoe_ep", seq_len=b.SEQ_LEN, micro_batch=b.MICRO_BATCH, layers=0)
    assert b.metric_name(b.METRIC, opts) == b.METRIC
    for change in (dict(seq_len=1024), dict(micro_batch=1), dict(layers=4)):
        o = types.SimpleNamespace(**{**vars(opts), **change})
        assert b.metric_name(b.METRIC, o).startswith("DEBUG")
    # both arms describe the measured configuration with the same record
    kw, mb, seq, vocab, metric, tag = b.named_config("olmoe_ep", 8)
    rec = b.result_config(opts, kw, 8 * mb * seq, tag)
    assert rec["model"] == "OLMoE-1B-7B" and rec["global_batch"] == 32 and rec["parallelism"] == "ep8"


def test_step_profile_kernel_table_sums_device_events_only():
    """The step profiler's table: device events are summed per kernel name, host events are left out, rows come longest
    first and the total covers every kernel, also those below the cut."""
    from types import SimpleNamespace

    import torch

    from optimus_lm_b200.utils.step_profile import kernel_table

    cuda, cpu = torch.autograd.DeviceType.CUDA, torch.autograd.DeviceType.CPU
    ev = [SimpleNamespace(device_type=cuda, name="gemm", device_time_total=100.0),
          SimpleNamespace(device_type=cuda, name="gemm", device_time_total=50.0),
          SimpleNamespace(device_type=cuda, name="adamw", device_time_total=400.0),
          SimpleNamespace(device_type=cuda, name="rope", device_time_total=5.0),
          SimpleNamespace(device_type=cpu, name="aten::mm", device_time_total=999.0)]
    total, rows = kernel_table(ev, top=2)
    assert total == 555.0
    assert rows == [(400.0, 1, "adamw"), (150.0, 2, "gemm")]
