"""OLMoE training checkpoint (single file or EP shards, merged or per-expert experts) -> Hugging Face
directory.  Role of the reference's evals/convert_olmoe_om_checkpoint_to_hf.py; the layout is a
command-line argument instead of a constant in the file.

    python evals/convert_olmoe_om_checkpoint_to_hf.py --model_choice allenai/OLMoE-1B-7B-0924--SE1.125 \
        --om_checkpoint_dir <exp>/checkpoints/main --expert_parallelism 12
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200.convert import om_to_hf_main  # noqa: E402

if __name__ == "__main__":
    om_to_hf_main("allenai/OLMoE-1B-7B-0924", "olmoe")
