"""Count the instances of every tokenized file and draw the global shuffling orders.  Role of the reference's scripts/generate_metadata.py (same flags and file layout);
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
    p.add_argument("--num_orders", type=int, default=1)
    a = p.parse_args()
    rank, world = data_prep.worker_identity()
    layout = data_prep.DatasetLayout(a.datasets_dir, a.dataset_choice, a.model_choice)
    data_prep.generate_metadata(layout, a.num_files, a.context_size, a.num_orders)
