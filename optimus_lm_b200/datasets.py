"""Token datasets for data-parallel pretraining.

On-disk layout and indexing of the reference (optimus/datasets.py:6-121):

``<dataset_dir>/tokenized_data/<category>_<file>.npy``   int32 token arrays, one per source file
``<dataset_dir>/../../urls.txt``                          source list that fixes the file order
``<dataset_dir>/num_instances_f{F}_c{C}.npy``             instances (= C-token windows) per file
``<dataset_dir>/shuffling_order_f{F}_c{C}_1.npy``         global permutation of all instances
``<dataset_dir>/sharded_data_f{F}_c{C}/shard_{i}.npy``    pre-shuffled fixed-size shards

Instance ``(base + i) * dp_size + dp_ind`` belongs to data-parallel rank ``dp_ind`` (EP ranks count
as data-parallel ranks: ``dp_size = DP*EP``, index ``dp_ind*EP + ep_ind``).  Resuming calls
``set_base_dp_idx(train_step * batch_size)``.

Differences: the file lookup is a binary search over the cumulative instance counts instead of
a linear scan, and ``SyntheticTokenDataset`` provides uniform-random tokens with the same
interface for benchmarks and tests (no files needed).
"""
from __future__ import annotations

import bisect
import os

import numpy as np
import torch
from torch.utils.data import Dataset

TOKENS_PER_SHARD = 50 * 256 * 12 * 1 * 4096  # 0.6B-token shards, as written by scripts/generate_shards.py


def tokenized_file_paths(dataset_dir: str):
    """File order = order of ``urls.txt``; ``.../<category>/<name>.<ext>`` -> ``<category>_<name>.npy``."""
    out = []
    with open(os.path.join(dataset_dir, "../../urls.txt")) as fh:
        for url in fh:
            parts = url.strip().split("/")
            if len(parts) < 2:
                continue
            out.append(os.path.join(dataset_dir, "tokenized_data", f"{parts[-2]}_{parts[-1].split('.')[0]}.npy"))
    return out


class _DpIndexed(Dataset):
    def __init__(self, context_size, dp_size, dp_ind):
        self.context_size, self.dp_size, self.dp_ind = context_size, dp_size, dp_ind
        self.base_dp_idx = 0
        self.num_instances = 0

    def set_base_dp_idx(self, base_dp_idx):
        self.base_dp_idx = base_dp_idx

    def __len__(self):
        return int(self.num_instances // self.dp_size)

    def _serial(self, dp_idx):
        return (self.base_dp_idx + dp_idx) * self.dp_size + self.dp_ind


class PclDataPrallelDataset(_DpIndexed):
    """Per-file token arrays + a global shuffling order (class name spelled as in the reference)."""

    def __init__(self, dataset_dir, num_data_files, context_size, dp_size=1, dp_ind=0):
        super().__init__(context_size, dp_size, dp_ind)
        self.tokenized_file_paths = tokenized_file_paths(dataset_dir)
        F = len(self.tokenized_file_paths) if num_data_files == -1 else num_data_files
        self.data_list = [None] * F
        self.num_instances_list = np.load(os.path.join(dataset_dir, f"num_instances_f{F}_c{context_size}.npy"))
        self.shuffling_order = np.load(os.path.join(dataset_dir, f"shuffling_order_f{F}_c{context_size}_1.npy"),
                                       mmap_mode="r")
        self.num_instances = int(np.sum(self.num_instances_list))
        self.cum_instances_list = [0] + [int(c) for c in np.cumsum(self.num_instances_list)]

    def __getitem__(self, dp_idx):
        idx = int(self.shuffling_order[self._serial(dp_idx)])
        f = bisect.bisect_right(self.cum_instances_list, idx) - 1
        local = idx - self.cum_instances_list[f]
        if self.data_list[f] is None:
            self.data_list[f] = np.load(self.tokenized_file_paths[f], mmap_mode="r")
        s = local * self.context_size
        return np.copy(self.data_list[f][s:s + self.context_size])


PclDataParallelDataset = PclDataPrallelDataset


class PclShardedDataParallelDataset(_DpIndexed):
    """Pre-shuffled shards of a fixed token count: O(1) index arithmetic."""

    def __init__(self, dataset_dir, num_data_files, context_size, dp_size=1, dp_ind=0,
                 num_tokens_per_shard=TOKENS_PER_SHARD):
        super().__init__(context_size, dp_size, dp_ind)
        assert num_tokens_per_shard % context_size == 0, "num_tokens_per_shard should be divisible by context_size"
        self.num_instances_per_shard = num_tokens_per_shard // context_size
        if num_data_files == -1:
            with open(os.path.join(dataset_dir, "../../urls.txt")) as fh:
                num_data_files = len(fh.readlines())
        shard_dir = os.path.join(dataset_dir, f"sharded_data_f{num_data_files}_c{context_size}")
        names = sorted((f for f in os.listdir(shard_dir) if f.endswith(".npy")),
                       key=lambda x: int(x.split("_")[1].split(".npy")[0]))
        ids = [int(f.split("_")[1].split(".npy")[0]) for f in names]
        assert ids and ids[0] == 0, "Shards should start from 0"
        assert ids[-1] == len(ids) - 1, "Shards should end at num_shards - 1"
        self.sharded_file_paths = [os.path.join(shard_dir, f) for f in names]
        self.num_instances_list = np.load(os.path.join(dataset_dir, f"num_instances_f{num_data_files}_c{context_size}.npy"))
        self.num_instances = int(np.sum(self.num_instances_list))
        self.data_list = [None] * len(self.sharded_file_paths)

    def __getitem__(self, dp_idx):
        idx = self._serial(dp_idx)
        f, local = divmod(idx, self.num_instances_per_shard)
        if self.data_list[f] is None:
            self.data_list[f] = np.load(self.sharded_file_paths[f], mmap_mode="r")
        s = local * self.context_size
        return np.copy(self.data_list[f][s:s + self.context_size])


class SyntheticTokenDataset(_DpIndexed):
    """Uniform-random token ids; instance ``i`` is a pure function of ``(seed, i)``, so any
    data-parallel layout reads the same global stream."""

    def __init__(self, vocab_size, context_size, num_instances=1 << 30, dp_size=1, dp_ind=0, seed=0):
        super().__init__(context_size, dp_size, dp_ind)
        self.vocab_size, self.seed = vocab_size, seed
        self.num_instances = num_instances

    def __getitem__(self, dp_idx):
        rng = np.random.Generator(np.random.Philox(key=self.seed, counter=[self._serial(dp_idx), 0, 0, 0]))
        return rng.integers(0, self.vocab_size, size=self.context_size, dtype=np.int32)


def write_synthetic_dataset_dir(root: str, vocab_size: int, context_size: int, num_files: int = 2,
                                instances_per_file: int = 64, seed: int = 0, tokenizer: str = "olmo",
                                name: str = "synthetic") -> str:
    """Write a tiny dataset in the reference's directory layout (for tests and for running other
    tools against the same files).  Returns the ``preprocessed/<tokenizer>`` directory."""
    base = os.path.join(root, name)
    ddir = os.path.join(base, "preprocessed", tokenizer)
    os.makedirs(os.path.join(ddir, "tokenized_data"), exist_ok=True)
    rng = np.random.default_rng(seed)
    with open(os.path.join(base, "urls.txt"), "w") as fh:
        for f in range(num_files):
            fh.write(f"https://example.invalid/data/cat{f % 2}/part{f:03d}.parquet\n")
    counts = []
    for f in range(num_files):
        n = instances_per_file + f  # uneven on purpose
        arr = rng.integers(0, vocab_size, size=n * context_size + 7, dtype=np.int32)
        np.save(os.path.join(ddir, "tokenized_data", f"cat{f % 2}_part{f:03d}.npy"), arr)
        counts.append(n)
    np.save(os.path.join(ddir, f"num_instances_f{num_files}_c{context_size}.npy"), np.array(counts, dtype=np.int64))
    np.random.seed(42)
    np.save(os.path.join(ddir, f"shuffling_order_f{num_files}_c{context_size}_1.npy"),
            np.random.permutation(int(sum(counts))).astype(np.int64))
    return ddir
