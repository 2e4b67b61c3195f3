"""Command-line entry: writes the per-tensor serial store of ``--model_choice`` (default allenai/OLMoE-1B-7B-0924).

Same role and flags as the reference's generate_serial_model.py; the work is done by
optimus_lm_b200/model_generation.py.  Run directly for one worker, or under torchrun / mpirun to
split the tensors (serial) or the shards (parallel) over the ranks.
"""
from optimus_lm_b200.model_generation import serial_main

if __name__ == "__main__":
    serial_main("allenai/OLMoE-1B-7B-0924")
