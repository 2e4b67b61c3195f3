"""Training checkpoint shards -> cached model shards: ``model_checkpoint_shard-<i>.pth`` (a dict with
``state_dict``) is re-saved as ``model_<i>.pth`` (the bare state dict), so that a new experiment can
start from a checkpoint's weights with ``--use_om_cached_model``.  Role of the reference's
scripts/convert_omcp_to_omcached.py, with the directories as arguments.

    python scripts/convert_omcp_to_omcached.py --om_checkpoint_dir <exp>/checkpoints/step61500-tokens1548B \
        --om_cached_dir parallel_models/allenai__OLMoE-1B-7B-0924_pp4-ep12-tp1-vpp1
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200.convert import om_checkpoint_to_omcached  # noqa: E402

if __name__ == "__main__":
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--om_checkpoint_dir", type=str, required=True)
    p.add_argument("--om_cached_dir", type=str, required=True)
    a = p.parse_args()
    print(f"OM model checkpoint dir : {a.om_checkpoint_dir}")
    print(f"OM model cached dir     : {a.om_cached_dir}")
    om_checkpoint_to_omcached(a.om_checkpoint_dir, a.om_cached_dir)
