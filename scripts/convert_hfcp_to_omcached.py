"""Hugging Face checkpoint directory -> cached model shards (``model_<mp_ind>.pth``) of a parallel
layout, the files ``dist_train.py --use_om_cached_model`` loads.  Role of the reference's
scripts/convert_hfcp_to_omcached.py (Llama, PP only); any family and PP/EP/TP/VPP layout here.

    python scripts/convert_hfcp_to_omcached.py --model_choice meta-llama/Llama-3.1-8B \
        --hf_checkpoint_dir <dir> --pipeline_parallelism 2
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200.convert import add_layout_arguments, hf_checkpoint_to_omcached  # noqa: E402
from optimus_lm_b200.model_generation import worker_identity  # noqa: E402

if __name__ == "__main__":
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--model_choice", type=str, default="meta-llama/Llama-3.1-8B")
    p.add_argument("--hf_checkpoint_dir", type=str, required=True)
    p.add_argument("--parallel_models_dir", type=str, default="./parallel_models")
    p.add_argument("--use_merged_mlp_in_fast_moe", action="store_true")
    add_layout_arguments(p)
    a = p.parse_args()
    rank, world = worker_identity()
    grid = a.pipeline_parallelism * a.expert_parallelism * a.tensor_parallelism
    hf_checkpoint_to_omcached(a.model_choice, a.hf_checkpoint_dir, a.parallel_models_dir, pp=a.pipeline_parallelism,
                              ep=a.expert_parallelism, tp=a.tensor_parallelism, vpp=a.virtual_pipeline_parallelism,
                              merged=a.use_merged_mlp_in_fast_moe, ranks=range(rank, grid, world))
