"""Checkpoint converters: sharded training checkpoint -> Hugging Face directory -> cached shards.

The Hugging Face implementation (``transformers``) is the oracle for the forward pass: logits of
the converted checkpoint loaded with ``AutoModelForCausalLM`` must match this framework's serial
model with the same weights.
"""
import os

import pytest
import torch

from optimus_lm_b200 import convert, model_io
from optimus_lm_b200.engine import init_weights

OLMOE = "allenai/OLMoE-1B-7B-0924--L2-SH0.0625-SA0.25-SE0.125-SC0.25-SI0.25"
LLAMA = "meta-llama/Llama-3.2-1B--L2-H256-I512"
OLMO = "allenai/OLMo-1B-hf--L2"            # OLMo tags carry no width (reference grammar): full-width layers
DSV3 = "deepseek-ai/DeepSeek-V3--L3-DL1-N16-K2-MI64-A4-SE1-H128-I256"   # MLA, sigmoid group-limited router, YaRN


def _write_checkpoint(tmp_path, model_choice, pp, ep, tp, vpp, merged, dtype=torch.float32):
    """Shards initialised in memory and saved in the training-checkpoint file format."""
    d = str(tmp_path / "ckpt")
    os.makedirs(d, exist_ok=True)
    grid = pp * ep * tp
    for mp in range(grid):
        cfg, model, _ = convert.meta_shard(model_choice, mp, pp, ep, tp, vpp, merged, device="cpu", dtype=dtype)
        init_weights(model, cfg.initializer_range, seed=7)
        name = "model_checkpoint.pth" if grid == 1 else f"model_checkpoint_shard-{mp}.pth"
        torch.save({"train_step_id": 1, "state_dict": model.state_dict()}, os.path.join(d, name))
    return d


def _serial_logits(model_choice, ids, dtype=torch.float32):
    cfg, model, _ = convert.meta_shard(model_choice, 0, device="cpu", dtype=dtype)
    init_weights(model, cfg.initializer_range, seed=7)
    model.eval()
    with torch.no_grad():
        out = model(ids)
    return out.logits if hasattr(out, "logits") else out["output"]


@pytest.mark.parametrize("model_choice,lay", [
    (OLMOE, dict(pp=2, ep=2, tp=1, vpp=1, merged=True)),
    (OLMOE, dict(pp=1, ep=2, tp=1, vpp=1, merged=False)),
    (LLAMA, dict(pp=1, ep=1, tp=2, vpp=1, merged=False)),
    (OLMO, dict(pp=2, ep=1, tp=1, vpp=1, merged=False)),
    (DSV3, dict(pp=1, ep=2, tp=1, vpp=1, merged=True)),
])
def test_om_checkpoint_to_hf_matches_transformers(tmp_path, model_choice, lay):
    transformers = pytest.importorskip("transformers")
    ckpt = _write_checkpoint(tmp_path, model_choice, **lay)
    hf_dir = str(tmp_path / "hf")
    convert.om_checkpoint_to_hf(model_choice, ckpt, hf_dir, pp=lay["pp"], ep=lay["ep"], tp=lay["tp"], vpp=lay["vpp"],
                                verbose=False)
    assert os.path.exists(os.path.join(hf_dir, "config.json"))
    hf = transformers.AutoModelForCausalLM.from_pretrained(hf_dir, dtype=torch.float32)
    hf.eval()
    torch.manual_seed(0)
    ids = torch.randint(2, 1000, (2, 24))
    with torch.no_grad():
        want = hf(ids).logits
    got = _serial_logits(model_choice, ids)
    assert got.shape == want.shape
    assert torch.allclose(got, want, atol=2e-4, rtol=1e-3), (got - want).abs().max()


def test_hf_to_omcached_round_trip(tmp_path):
    lay = dict(pp=2, ep=2, tp=1, vpp=1, merged=True)
    ckpt = _write_checkpoint(tmp_path, OLMOE, **lay)
    hf_dir = str(tmp_path / "hf")
    convert.om_checkpoint_to_hf(OLMOE, ckpt, hf_dir, pp=2, ep=2, verbose=False)
    paths = convert.hf_checkpoint_to_omcached(OLMOE, hf_dir, str(tmp_path / "parallel"), dtype=torch.float32,
                                              verbose=False, **lay)
    assert [os.path.basename(p) for p in paths] == [f"model_{i}.pth" for i in range(4)]
    for mp, p in enumerate(paths):
        a = torch.load(p, weights_only=True)
        b = torch.load(os.path.join(ckpt, f"model_checkpoint_shard-{mp}.pth"), weights_only=True)["state_dict"]
        assert set(a) == set(b)
        for k in a:
            assert torch.equal(a[k], b[k]), k
    # checkpoint shards -> cached shards is a re-save of the bare state dicts
    cached = convert.om_checkpoint_to_omcached(ckpt, str(tmp_path / "cached"), verbose=False)
    assert len(cached) == 4
    a = torch.load(cached[3], weights_only=True)
    assert torch.equal(a["model.norm.weight"], b["model.norm.weight"]) if "model.norm.weight" in a else True
    # and a cached directory converts to serial like a checkpoint does
    s1 = convert.om_checkpoint_to_serial(OLMOE, str(tmp_path / "cached"), pp=2, ep=2, cached=True)
    s2 = convert.om_checkpoint_to_serial(OLMOE, ckpt, pp=2, ep=2)
    assert set(s1) == set(s2) and all(torch.equal(s1[k], s2[k]) for k in s1)


def test_large_checkpoint_is_split_into_indexed_shards(tmp_path):
    serial = {f"model.layers.{i}.w": torch.full((64, 64), float(i)) for i in range(6)}
    convert.write_hf_checkpoint(serial, {"model_type": "x"}, str(tmp_path), max_shard_bytes=40000)
    reader = convert.HFCheckpointReader(str(tmp_path))
    assert len(set(reader.where.values())) == 3
    assert torch.equal(reader.get("model.layers.4.w"), serial["model.layers.4.w"])
