"""Serial store -> sharded model files -> serial again, for every model family and layout kind.

The oracle is the in-memory seeded initialiser (``engine.init_weights``): a shard filled from the
per-tensor files must equal the same shard initialised directly, and scattering all shards back
must reproduce the store.
"""
import os

import pytest
import torch

from optimus_lm_b200 import model_generation as mg
from optimus_lm_b200 import model_io
from optimus_lm_b200.engine import build_model, init_weights
from optimus_lm_b200.mapper import ParallelDpPpEpTpMapper

OLMOE = "allenai/OLMoE-1B-7B-0924--L4-SH0.0625-SA0.25-SE0.125-SC0.25-SI0.25"
DSV3 = "deepseek-ai/DeepSeek-V3--L3-DL1-N8-K2-MI64-A4-SE1-H128-I256"
LLAMA = "meta-llama/Llama-3.1-8B--L2-H256-I512"
OLMO = "allenai/OLMo-1B-hf--L2"            # OLMo tags carry no width (reference grammar): full-width layers

LAYOUTS = [
    (OLMOE, dict(pp=2, ep=2, tp=1, vpp=1, merged=False)),
    (OLMOE, dict(pp=2, ep=2, tp=1, vpp=2, merged=True)),
    (OLMOE, dict(pp=1, ep=4, tp=1, vpp=1, merged=True)),
    (DSV3, dict(pp=1, ep=2, tp=1, vpp=1, merged=True)),
    (DSV3, dict(pp=1, ep=2, tp=1, vpp=1, merged=False)),
    (LLAMA, dict(pp=1, ep=1, tp=2, vpp=1, merged=False)),
    (OLMO, dict(pp=2, ep=1, tp=2, vpp=1, merged=False)),
]


def _shard(model_choice, lay, rank, device="cpu"):
    pmap = ParallelDpPpEpTpMapper(data_parallelism=1, pipeline_parallelism=lay["pp"], expert_parallelism=lay["ep"],
                                  tensor_parallelism=lay["tp"], rank=rank, create_groups=False)
    kw = dict(pipeline_parallelism=lay["pp"], expert_parallelism=lay["ep"], tensor_parallelism=lay["tp"],
              virtual_pipeline_parallelism=lay["vpp"])
    if "OLMoE" in model_choice or "DeepSeek" in model_choice:
        kw.update(use_fast_moe=True, use_merged_mlp_in_fast_moe=lay["merged"])
    return build_model(model_choice, pmap, dtype=torch.bfloat16, device=device, **kw)


@pytest.mark.parametrize("model_choice,lay", LAYOUTS)
def test_generators_match_seeded_init_and_round_trip(tmp_path, model_choice, lay):
    sdir, pdir = str(tmp_path / "serial"), str(tmp_path / "parallel")
    # two workers split the serial tensors
    a = mg.generate_serial_model(model_choice, sdir, rank=0, world_size=2, verbose=False)
    b = mg.generate_serial_model(model_choice, sdir, rank=1, world_size=2, verbose=False)
    assert not set(a) & set(b)
    store = mg.serial_model_dir(sdir, model_choice)
    assert sorted(os.listdir(store)) == sorted(f"{n}.pt" for n in a + b)

    grid = lay["pp"] * lay["ep"] * lay["tp"]
    serial = {}
    for r in range(grid):
        path = mg.generate_parallel_model(model_choice, pipeline_parallelism=lay["pp"], expert_parallelism=lay["ep"],
                                          tensor_parallelism=lay["tp"], virtual_pipeline_parallelism=lay["vpp"],
                                          use_merged_mlp_in_fast_moe=lay["merged"], rank=r, serial_models_dir=sdir,
                                          parallel_models_dir=pdir, verbose=False)
        assert os.path.basename(path) == f"model_{r}.pth"
        sd = torch.load(path, map_location="cpu", weights_only=True)
        cfg, ref = _shard(model_choice, lay, r)
        init_weights(ref, cfg.initializer_range, seed=0)
        ref_sd = ref.state_dict()
        assert set(sd) == set(ref_sd)
        for k in sd:
            assert torch.equal(sd[k], ref_sd[k]), k
        ref.load_state_dict(sd, strict=True)
        model_io.scatter_shard(model_io.shard_plan(ref), sd, serial)

    assert set(serial) == set(a + b)
    for n, t in serial.items():
        want = model_io.load_serial_tensor(store, n).to(torch.bfloat16)
        assert torch.equal(t, want), n


def test_plan_on_meta_device_lists_every_global_expert_and_layer():
    names = dict(mg.serial_tensor_list(OLMOE)[1])
    assert "model.layers.3.mlp.experts.7.down_proj.weight" in names
    assert "model.layers.0.mlp.gate.weight" in names and "lm_head.weight" in names
    union = {}
    for r in range(4):
        _, m = _shard(OLMOE, dict(pp=2, ep=2, tp=1, vpp=2, merged=True), r, device="meta")
        union.update(model_io.serial_parameter_shapes([model_io.shard_plan(m)]))
    assert union == names


def test_seeded_tensor_depends_on_name_and_seed_only():
    a = model_io.seeded_serial_tensor("model.layers.1.self_attn.q_proj.weight", (8, 16), 0.02, seed=3)
    b = model_io.seeded_serial_tensor("model.layers.1.self_attn.q_proj.weight", (8, 16), 0.02, seed=3)
    c = model_io.seeded_serial_tensor("model.layers.2.self_attn.q_proj.weight", (8, 16), 0.02, seed=3)
    d = model_io.seeded_serial_tensor("model.layers.1.self_attn.q_proj.weight", (8, 16), 0.02, seed=4)
    assert torch.equal(a, b) and not torch.equal(a, c) and not torch.equal(a, d)
    assert torch.equal(model_io.seeded_serial_tensor("model.norm.weight", (16,), 0.02), torch.ones(16))
    assert torch.equal(model_io.seeded_serial_tensor("x.q_proj.bias", (16,), 0.02), torch.zeros(16))
