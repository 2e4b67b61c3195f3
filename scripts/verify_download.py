"""Check every downloaded file against the size its server reports.  Role of the reference's
scripts/verify_download.py.

    python scripts/verify_download.py --dataset_dir datasets/allenai_OLMoE-mix-0924 [--file_start_id 0 --file_end_id -1]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200 import data_prep  # noqa: E402

if __name__ == "__main__":
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--dataset_dir", type=str, required=True)
    p.add_argument("--file_start_id", type=int, default=0)
    p.add_argument("--file_end_id", type=int, default=-1)
    a = p.parse_args()
    for line in data_prep.verify_download(a.dataset_dir, a.file_start_id, a.file_end_id):
        print(line)
