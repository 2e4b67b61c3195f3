"""Write the shuffled instances as shard_<i>.npy files (split over the launched workers).  Role of the reference's scripts/generate_shards.py (same flags and file layout);
the work is done by optimus_lm_b200/data_prep.py.  Run under torchrun / mpirun to split the files over ranks.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200 import data_prep  # noqa: E402

if __name__ == "__main__":
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--datasets_dir", type=str, default="datasets/")
    p.add_argument("--model_choice", type=str, default="allenai/OLMoE-1B-7B-0924")
    p.add_argument("--dataset_choice", type=str, default="allenai/OLMoE-mix-0924")
    p.add_argument("--num_files", type=int, required=True)
    p.add_argument("--context_size", type=int, default=2048)
    p.add_argument("--tokens_per_shard", type=int, default=data_prep.DEFAULT_TOKENS_PER_SHARD)
    a = p.parse_args()
    rank, world = data_prep.worker_identity()
    layout = data_prep.DatasetLayout(a.datasets_dir, a.dataset_choice, a.model_choice)
    data_prep.generate_shards(layout, a.num_files, a.context_size, a.tokens_per_shard, rank=rank, world_size=world)
