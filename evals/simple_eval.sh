#!/bin/bash
# Evaluate one Hugging Face checkpoint directory with the lm_eval harness on GPU 0.
# Usage: bash evals/simple_eval.sh [checkpoint_dir] [output_dir]
ckpt=${1:-checkpoint_hf}
python -m lm_eval --model hf --model_args "pretrained=$ckpt,dtype=bfloat16" \
    --tasks arc_easy,arc_challenge,hellaswag,piqa,boolq,sciq,winogrande,openbookqa,mmlu \
    --device cuda:0 --batch_size 32 --output_path "${2:-results}"
