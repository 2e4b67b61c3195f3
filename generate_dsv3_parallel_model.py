"""Command-line entry: writes the sharded model_<mp_ind>.pth files of ``--model_choice`` (default deepseek-ai/DeepSeek-V3--N264-L96).

Same role and flags as the reference's generate_dsv3_parallel_model.py; the work is done by
optimus_lm_b200/model_generation.py.  Run directly for one worker, or under torchrun / mpirun to
split the tensors (serial) or the shards (parallel) over the ranks.
"""
from optimus_lm_b200.model_generation import parallel_main

if __name__ == "__main__":
    parallel_main("deepseek-ai/DeepSeek-V3--N264-L96")
