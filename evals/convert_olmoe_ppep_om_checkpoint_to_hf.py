"""OLMoE training checkpoint written by a PP x EP (x VPP) run -> Hugging Face directory.  Role of the
reference's evals/convert_olmoe_ppep_om_checkpoint_to_hf.py, whose layout (PP 4 x EP 12) is the
default here and can be changed on the command line.

    python evals/convert_olmoe_ppep_om_checkpoint_to_hf.py \
        --model_choice allenai/OLMoE-1B-7B-0924--SA3-SH1.5-SE2.25-SC0.5-SI2-L36 \
        --om_checkpoint_dir <exp>/checkpoints/main --pipeline_parallelism 4 --expert_parallelism 12
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200.convert import om_to_hf_main  # noqa: E402

if __name__ == "__main__":
    om_to_hf_main("allenai/OLMoE-1B-7B-0924", "olmoe", pp=4, ep=12)
