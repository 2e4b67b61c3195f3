"""Data preparation pipeline end to end on a toy corpus: URL files -> tokenize (two workers) ->
metadata -> shards, then read back through both dataset classes."""
import gzip
import json
import os

import numpy as np

from optimus_lm_b200 import data_prep
from optimus_lm_b200.datasets import PclDataPrallelDataset, PclShardedDataParallelDataset


class ToyTokenizer:
    """Bytes of the text as token ids; EOS = 0."""
    eos_token_id = 0

    def __call__(self, texts, add_special_tokens=False):
        if isinstance(texts, str):
            return {"input_ids": [b + 1 for b in texts.encode()]}
        return {"input_ids": [[b + 1 for b in t.encode()] for t in texts]}


def _corpus(root):
    layout = data_prep.DatasetLayout(str(root), "toy/mix", "allenai/OLMoE-1B-7B-0924--L2")
    urls = data_prep.expand_manifest({"alpha": [("a-", 0, 1, 4, ".json.gz")], "beta": [("", 7, 7, 3, ".jsonl")]},
                                     base_url="https://example.invalid/data/")
    assert data_prep.write_url_files(layout.root, urls) == 3
    rng = np.random.default_rng(0)
    docs = {}
    for path in layout.raw_paths():
        os.makedirs(os.path.dirname(path), exist_ok=True)
        texts = ["".join(chr(97 + int(c)) for c in rng.integers(0, 26, size=int(rng.integers(5, 400))))
                 for _ in range(int(rng.integers(300, 400)))]
        docs[path] = texts
        opener = gzip.open if path.endswith(".gz") else open
        with opener(path, "wt", encoding="utf-8") as fh:
            for t in texts:
                fh.write(json.dumps({"text": t, "id": 1}) + "\n")
    return layout, docs


def test_pipeline_end_to_end(tmp_path):
    layout, docs = _corpus(tmp_path)
    assert layout.tokenizer_name == "olmo"
    assert [os.path.basename(p) for p in layout.tokenized_paths()] == ["alpha_a-0000.npy", "alpha_a-0001.npy", "beta_007.npy"]
    tok = ToyTokenizer()
    logs = []
    a = data_prep.tokenize_dataset(layout, tok, 3, rank=0, world_size=2, log=logs.append)
    b = data_prep.tokenize_dataset(layout, tok, 3, rank=1, world_size=2, log=logs.append)
    assert len(a) == 2 and len(b) == 1
    # a second pass finds the completion markers and does nothing
    assert data_prep.tokenize_dataset(layout, tok, 3, log=logs.append) == []
    for raw, out in zip(layout.raw_paths(), layout.tokenized_paths()):
        want = []
        for t in docs[raw]:
            want += [c + 1 for c in t.encode()] + [0]
        got = np.load(out)
        assert got.dtype == np.int32 and got.tolist() == want

    C = 64
    counts = data_prep.generate_metadata(layout, 3, C, num_orders=2, log=logs.append)
    assert counts == [len(np.load(p)) // C for p in layout.tokenized_paths()]
    order = np.load(layout.shuffling_order_path(3, C, 1))
    assert sorted(order.tolist()) == list(range(sum(counts)))
    assert os.path.exists(layout.shuffling_order_path(3, C, 2))

    tokens_per_shard = 100 * C
    w0 = data_prep.generate_shards(layout, 3, C, tokens_per_shard, rank=0, world_size=2, log=logs.append)
    w1 = data_prep.generate_shards(layout, 3, C, tokens_per_shard, rank=1, world_size=2, log=logs.append)
    n_shards = -(-sum(counts) // 100)
    assert len(w0) + len(w1) == n_shards

    plain = PclDataPrallelDataset(layout.preprocessed, 3, C)
    sharded = PclShardedDataParallelDataset(layout.preprocessed, 3, C, num_tokens_per_shard=tokens_per_shard)
    assert plain.num_instances == sharded.num_instances == sum(counts)
    for i in list(range(0, sum(counts), 37)) + [sum(counts) - 1]:
        assert np.array_equal(plain[i], sharded[i]), i


def test_verify_download_reports_missing_and_mismatched(tmp_path):
    layout, docs = _corpus(tmp_path)
    paths = layout.raw_paths()
    sizes = {u: os.path.getsize(p) for u, p in zip(layout.urls(), paths)}
    assert data_prep.verify_download(layout.root, remote_size=sizes.get) == []
    os.remove(paths[0])
    sizes[layout.urls()[1]] += 1
    problems = data_prep.verify_download(layout.root, remote_size=sizes.get)
    assert len(problems) == 2 and problems[0].startswith("Missing file") and "size mismatch" in problems[1]


def test_builtin_manifest_expands_to_numbered_urls():
    urls = data_prep.expand_manifest(data_prep.OLMOE_MIX_0924)
    assert len(urls["dclm"]) == 1970 and urls["dclm"][3].endswith("/dclm/dclm-0003.json.zst")
    assert urls["open-web-math"][0].endswith("/open-web-math/041.jsonl.gz")
