"""Tokenize the first --num_files raw files of a dataset into int32 .npy token streams.  Role of the reference's scripts/tokenize_data.py (same flags and file layout);
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
    p.add_argument("--verbose", action="store_true")
    a = p.parse_args()
    rank, world = data_prep.worker_identity()
    layout = data_prep.DatasetLayout(a.datasets_dir, a.dataset_choice, a.model_choice)
    from transformers import AutoTokenizer
    tokenizer = AutoTokenizer.from_pretrained(a.model_choice.split("--")[0])
    data_prep.tokenize_dataset(layout, tokenizer, a.num_files, rank=rank, world_size=world, verbose=a.verbose)
