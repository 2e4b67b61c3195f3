"""Dataset preparation: URL lists -> downloaded files -> tokenized ``.npy`` -> instance counts and
shuffling orders -> pre-shuffled shards.

Directory layout (the one ``datasets.py`` reads; reference scripts/tokenize_data.py:94-99,
scripts/generate_metadata.py:29-41, scripts/generate_shards.py:32-38):

    <datasets_dir>/<dataset with / -> _>/urls.txt                      one URL per line, ``.../<category>/<file>``
    .../data/<category>/<file>                                         raw download
    .../preprocessed/<tokenizer>/tokenized_data/<category>_<stem>.npy  int32 token stream, EOS after each document
    .../preprocessed/<tokenizer>/num_instances_f<F>_c<C>.npy           instances (C tokens each) per file
    .../preprocessed/<tokenizer>/shuffling_order_f<F>_c<C>_<k>.npy     permutation of all instances
    .../preprocessed/<tokenizer>/sharded_data_f<F>_c<C>/shard_<i>.npy  instances in shuffled order

Every stage splits its files over ``world_size`` workers by index and marks finished outputs with a
``.completed`` file, so an interrupted run resumes where it stopped.  The functions take the
tokenizer as an argument (anything with ``__call__(text)["input_ids"]`` and ``eos_token_id``), so
they are testable without a tokenizer download.
"""
from __future__ import annotations

import gzip
import io
import json
import math
import os
import time
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np

MODEL_TOKENIZER_MAP = {
    "allenai/OLMoE-1B-7B-0924": "olmo",
    "allenai/OLMo-1B-hf": "olmo",
    "allenai/OLMo-7B-hf": "olmo",
    "meta-llama/Llama-3.1-8B": "llama",
    "meta-llama/Llama-3.2-1B": "llama",
    "deepseek-ai/DeepSeek-V3": "deepseek",
}

DEFAULT_TOKENS_PER_SHARD = 50 * 256 * 12 * 1 * 4096


def worker_identity():
    """(rank, world_size) from the launcher environment: torchrun, PALS/PMI, Open MPI, SLURM."""
    for r, w in (("RANK", "WORLD_SIZE"), ("PALS_RANKID", "PMI_SIZE"), ("PMI_RANK", "PMI_SIZE"),
                 ("OMPI_COMM_WORLD_RANK", "OMPI_COMM_WORLD_SIZE"), ("SLURM_PROCID", "SLURM_NTASKS")):
        if r in os.environ and w in os.environ:
            return int(os.environ[r]), int(os.environ[w])
    return 0, 1


class DatasetLayout:
    def __init__(self, datasets_dir: str, dataset_choice: str, model_choice: str):
        base_model = model_choice.split("--")[0]
        assert base_model in MODEL_TOKENIZER_MAP, \
            f"Model {model_choice} not supported. Supported models are {list(MODEL_TOKENIZER_MAP)}"
        self.tokenizer_name = MODEL_TOKENIZER_MAP[base_model]
        self.root = os.path.join(datasets_dir, dataset_choice.replace("/", "_"))
        self.urls_file = os.path.join(self.root, "urls.txt")
        self.data_dir = os.path.join(self.root, "data")
        self.preprocessed = os.path.join(self.root, "preprocessed", self.tokenizer_name)
        self.tokenized = os.path.join(self.preprocessed, "tokenized_data")

    def urls(self) -> List[str]:
        with open(self.urls_file) as fh:
            return [u.strip() for u in fh if u.strip()]

    @staticmethod
    def _cat_file(url):
        parts = url.split("/")
        return parts[-2], parts[-1]

    def raw_paths(self) -> List[str]:
        return [os.path.join(self.data_dir, *self._cat_file(u)) for u in self.urls()]

    def tokenized_paths(self) -> List[str]:
        out = []
        for u in self.urls():
            cat, name = self._cat_file(u)
            out.append(os.path.join(self.tokenized, f"{cat}_{name.split('.')[0]}.npy"))
        return out

    def num_instances_path(self, num_files, context_size):
        return os.path.join(self.preprocessed, f"num_instances_f{num_files}_c{context_size}.npy")

    def shuffling_order_path(self, num_files, context_size, order=1):
        return os.path.join(self.preprocessed, f"shuffling_order_f{num_files}_c{context_size}_{order}.npy")

    def sharded_dir(self, num_files, context_size):
        return os.path.join(self.preprocessed, f"sharded_data_f{num_files}_c{context_size}")


# ---------------------------------------------------------------- stage 0: URL lists

# File-name patterns of allenai/OLMoE-mix-0924: category -> [(prefix, first, last, zero-fill width, extension)].
# The ``starcoder`` category has one pattern per programming language; its list comes from a manifest
# file (``--manifest``, JSON of the same shape) or from the hub's file listing when a network is there.
OLMOE_MIX_0924 = {
    "algebraic-stack": [("algebraic-stack-train-", 0, 15, 4, ".json.gz")],
    "dclm": [("dclm-", 0, 1969, 4, ".json.zst")],
    "open-web-math": [("", 41, 53, 3, ".jsonl.gz"), ("open-web-math-train-", 0, 12, 4, ".json.gz")],
    "pes2o": [("pes2o-", 0, 25, 4, ".json.gz")],
    "wiki": [("wiki-", 0, 1, 4, ".json.gz")],
}
OLMOE_MIX_BASE_URL = "https://huggingface.co/datasets/allenai/OLMoE-mix-0924/resolve/main/data/"


def expand_manifest(manifest: Dict[str, Sequence], base_url: str = OLMOE_MIX_BASE_URL) -> Dict[str, List[str]]:
    out: Dict[str, List[str]] = {}
    for category, groups in manifest.items():
        urls = []
        for prefix, first, last, width, ext in groups:
            urls += [f"{base_url}{category}/{prefix}{str(i).zfill(width)}{ext}" for i in range(first, last + 1)]
        out[category] = urls
    return out


def urls_from_hub_listing(repo_id: str, subdir: str = "data") -> Dict[str, List[str]]:
    """Category -> URLs from the hub's file listing (needs network access and ``huggingface_hub``)."""
    from huggingface_hub import list_repo_files

    out: Dict[str, List[str]] = {}
    for f in sorted(list_repo_files(repo_id, repo_type="dataset")):
        parts = f.split("/")
        if len(parts) == 3 and parts[0] == subdir:
            out.setdefault(parts[1], []).append(f"https://huggingface.co/datasets/{repo_id}/resolve/main/{f}")
    return out


def write_url_files(dataset_path: str, urls_by_category: Dict[str, List[str]]) -> int:
    """``urls_<category>.txt`` per category and the concatenated ``urls.txt`` (reference
    scripts/generate_urls.py:152-170)."""
    os.makedirs(dataset_path, exist_ok=True)
    n = 0
    with open(os.path.join(dataset_path, "urls.txt"), "w") as all_fh:
        for category, urls in urls_by_category.items():
            with open(os.path.join(dataset_path, f"urls_{category}.txt"), "w") as fh:
                for u in urls:
                    fh.write(u + "\n")
                    all_fh.write(u + "\n")
                    n += 1
    return n


def verify_download(dataset_dir: str, start: int = 0, end: int = -1,
                    remote_size: Optional[Callable[[str], Optional[int]]] = None) -> List[str]:
    """Compare local file sizes with the servers' Content-Length (reference scripts/verify_download.py).
    Returns the list of problems found."""
    if remote_size is None:
        import requests

        def remote_size(url):
            r = requests.head(url, allow_redirects=True, timeout=5)
            return int(r.headers.get("Content-Length", 0)) if r.status_code == 200 else None

    with open(os.path.join(dataset_dir, "urls.txt")) as fh:
        urls = [u.strip() for u in fh if u.strip()]
    end = len(urls) if end == -1 else end
    assert end <= len(urls), f"file_end_id {end} exceeds number of URLs {len(urls)}"
    problems = []
    for url in urls[start:end]:
        cat, name = url.split("/")[-2:]
        path = os.path.join(dataset_dir, "data", cat, name)
        try:
            want = remote_size(url)
        except Exception as e:  # network errors are reported, not fatal
            problems.append(f"Error checking URL {url}: {e}")
            continue
        if want is None:
            problems.append(f"Failed to fetch size for {url}")
        elif not os.path.exists(path):
            problems.append(f"Missing file: {path}")
        elif os.path.getsize(path) != want:
            problems.append(f"File size mismatch for {path}: local size = {os.path.getsize(path)}, remote size = {want}")
    return problems


# ---------------------------------------------------------------- stage 1: tokenize


def read_documents(file_path: str, text_key: str = "text") -> Iterator[str]:
    """Documents of a ``.zst`` / ``.gz`` / plain JSON-lines file or of a ``.parquet`` table."""
    ext = os.path.splitext(file_path)[1].lower()
    if ext == ".parquet":
        import pyarrow.parquet as pq

        pf = pq.ParquetFile(file_path)
        for batch in pf.iter_batches(columns=[text_key]):
            for t in batch.column(0):
                yield t.as_py()
        return
    if ext == ".zst":
        import zstandard as zstd  # optional dependency, only needed for .zst inputs

        raw = open(file_path, "rb")
        stream = io.TextIOWrapper(zstd.ZstdDecompressor().stream_reader(raw), encoding="utf-8")
    elif ext == ".gz":
        raw = None
        stream = gzip.open(file_path, "rt", encoding="utf-8")
    elif ext in (".jsonl", ".json"):
        raw = None
        stream = open(file_path, "rt", encoding="utf-8")
    else:
        raise ValueError(f"Unsupported file extension: {ext}")
    try:
        for line in stream:
            line = line.rstrip("\n")
            if line:
                yield json.loads(line)[text_key]
    finally:
        stream.close()
        if raw is not None:
            raw.close()


def tokenize_file(file_path: str, out_path: str, tokenizer, *, batch_docs: int = 256, verbose: bool = False,
                  log=print) -> int:
    """One raw file -> int32 token stream (document tokens + EOS, concatenated).  Documents are
    tokenized in batches (fast tokenizers parallelise over a batch) and appended to chunked int32
    arrays, not to a Python list.  Returns the number of tokens written."""
    chunks: List[np.ndarray] = []
    eos = tokenizer.eos_token_id
    total, docs, t0 = 0, 0, time.time()

    def flush(batch):
        nonlocal total
        enc = tokenizer(batch, add_special_tokens=False)["input_ids"]
        for ids in enc:
            arr = np.empty(len(ids) + 1, dtype=np.int32)
            arr[:-1] = ids
            arr[-1] = eos
            chunks.append(arr)
            total += arr.size

    batch: List[str] = []
    for doc in read_documents(file_path):
        batch.append(doc)
        docs += 1
        if len(batch) == batch_docs:
            flush(batch)
            batch = []
            if verbose and docs % (batch_docs * 8) == 0:
                log(f"Documents processed : {docs}, Tokens processed {total}, Time elapsed {time.time() - t0:.2f} seconds")
    if batch:
        flush(batch)
    out = np.concatenate(chunks) if chunks else np.zeros(0, dtype=np.int32)
    tmp = out_path + ".tmp.npy"
    np.save(tmp, out)
    os.replace(tmp, out_path)
    return int(total)


def tokenize_dataset(layout: DatasetLayout, tokenizer, num_files: int, *, rank=0, world_size=1, verbose=False,
                     log=print) -> List[str]:
    raw, tok = layout.raw_paths(), layout.tokenized_paths()
    assert num_files <= len(raw), f"Only {len(raw)} files are present"
    os.makedirs(layout.tokenized, exist_ok=True)
    done = []
    for i in range(num_files):
        if i % world_size != rank:
            continue
        marker = tok[i].replace(".npy", ".completed")
        if os.path.exists(marker):
            log(f"Rank {rank} : File {raw[i]} already tokenized. Skipping.")
            continue
        log(f"Rank {rank} : Processing file {raw[i]}")
        n = tokenize_file(raw[i], tok[i], tokenizer, verbose=verbose, log=lambda m: log(f"Rank {rank} : {m}"))
        log(f"Rank {rank} : Saved file {tok[i]}. Number of file tokens {n}")
        with open(marker, "w") as fh:
            fh.write("1")
        done.append(tok[i])
    return done


# ---------------------------------------------------------------- stage 2: metadata


def generate_metadata(layout: DatasetLayout, num_files: int, context_size: int, num_orders: int = 1,
                      seed: int = 42, log=print):
    """Instances per file and ``num_orders`` global shuffling orders (reference
    scripts/generate_metadata.py:45-71: ``np.random.seed(42)`` then one permutation per order)."""
    tok = layout.tokenized_paths()
    assert num_files <= len(tok), f"Only {len(tok)} files are present"
    counts = []
    for i in range(num_files):
        counts.append(int(np.load(tok[i], mmap_mode="r").shape[0]) // context_size)
    total = int(sum(counts))
    log(f"Number of training instances : {total}")
    log(f"Number of training tokens    : {(total * context_size) * 1e-9:.1f} B tokens")
    np.random.seed(seed)
    for k in range(num_orders):
        order = np.random.permutation(np.arange(total))
        np.save(layout.shuffling_order_path(num_files, context_size, k + 1), order)
    np.save(layout.num_instances_path(num_files, context_size), np.array(counts))
    return counts


# ---------------------------------------------------------------- stage 3: shards


def generate_shards(layout: DatasetLayout, num_files: int, context_size: int,
                    tokens_per_shard: int = DEFAULT_TOKENS_PER_SHARD, *, rank=0, world_size=1, order: int = 1,
                    log=print) -> List[str]:
    """Materialise the shuffled instance order as ``shard_<i>.npy`` files of
    ``tokens_per_shard // context_size`` instances each (reference scripts/generate_shards.py:41-139).
    Instances of a shard are copied file by file with one fancy-indexed gather per source file (the
    memory-mapped source is then read in ascending order) instead of one copy per instance."""
    tok = layout.tokenized_paths()
    assert num_files <= len(tok), f"Only {len(tok)} files are present"
    out_dir = layout.sharded_dir(num_files, context_size)
    os.makedirs(out_dir, exist_ok=True)
    per_shard = tokens_per_shard // context_size
    assert per_shard > 0, "tokens_per_shard is smaller than one instance"
    order_arr = np.load(layout.shuffling_order_path(num_files, context_size, order))
    counts = np.load(layout.num_instances_path(num_files, context_size))
    total = int(counts.sum())
    cum = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    num_shards = math.ceil(total / per_shard)
    if rank == 0:
        log(f"Number of data files          : {num_files}")
        log(f"Context size                  : {context_size}")
        log(f"Number of training tokens     : {(total * context_size) * 1e-9:.1f} B")
        log(f"Number of shards              : {num_shards}")
        log(f"Number of instances per shard : {per_shard}")
    mmaps: Dict[int, np.ndarray] = {}
    written = []
    for s in range(num_shards):
        if s % world_size != rank:
            continue
        path = os.path.join(out_dir, f"shard_{s}.npy")
        marker = path.replace(".npy", ".completed")
        if os.path.exists(marker):
            log(f"Rank {rank} : Shard {s} already generated. Skipping.")
            continue
        lo, hi = s * per_shard, min(total, (s + 1) * per_shard)
        ids = order_arr[lo:hi].astype(np.int64)
        file_of = np.searchsorted(cum, ids, side="right") - 1
        shard = np.zeros((hi - lo, context_size), dtype=np.int32)
        for f in np.unique(file_of):
            sel = np.nonzero(file_of == f)[0]
            local = ids[sel] - cum[f]
            asc = np.argsort(local, kind="stable")
            if f not in mmaps:
                mmaps[int(f)] = np.load(tok[int(f)], mmap_mode="r")
            src = mmaps[int(f)][: counts[f] * context_size].reshape(counts[f], context_size)
            shard[sel[asc]] = src[local[asc]]
        tmp = path + ".tmp.npy"
        np.save(tmp, shard.reshape(-1))
        os.replace(tmp, path)
        with open(marker, "w") as fh:
            fh.write("1")
        log(f"Rank {rank} : Saved shard file {s}")
        written.append(path)
    return written
