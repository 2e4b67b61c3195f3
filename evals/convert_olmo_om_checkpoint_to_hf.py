"""OLMo (dense) training checkpoint -> Hugging Face directory.  Role of the reference's
evals/convert_olmo_om_checkpoint_to_hf.py; PP / TP sharded checkpoints are merged as well.

    python evals/convert_olmo_om_checkpoint_to_hf.py --model_choice allenai/OLMo-1B-hf \
        --om_checkpoint_dir <exp>/checkpoints/main
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200.convert import om_to_hf_main  # noqa: E402

if __name__ == "__main__":
    om_to_hf_main("allenai/OLMo-1B-hf", "olmo")
