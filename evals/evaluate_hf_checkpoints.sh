#!/bin/bash
# Run the lm_eval harness on every converted checkpoint of an experiment; checkpoints are dealt
# round-robin to RANK / WORLD_SIZE workers (one GPU each).  Needs the lm_eval package.
# Usage: [RANK=0 WORLD_SIZE=1] bash evals/evaluate_hf_checkpoints.sh <exp_dir> [tasks]
set -euo pipefail
if [ $# -lt 1 ]; then
    echo "Usage: bash $0 <exp_dir> [tasks]"
    exit 1
fi
exp_dir=$1
tasks=${2:-arc_easy,arc_challenge,hellaswag,piqa,boolq,sciq,winogrande,openbookqa,mmlu}
rank=${RANK:-0}; world_size=${WORLD_SIZE:-1}
i=0
for cp in $(ls "$exp_dir/hf_checkpoints" | grep -E "^(step|main)" | sort -V); do
    mine=$(( i % world_size == rank )); i=$(( i + 1 ))
    [ "$mine" -eq 1 ] || continue
    out="$exp_dir/results/$cp"
    if [ -d "$out" ]; then
        echo "Checkpoint $cp already processed. Skipping."
        continue
    fi
    echo "Processing Checkpoint $cp (Rank : $rank)"
    python -m lm_eval --model hf --model_args "pretrained=$exp_dir/hf_checkpoints/$cp,dtype=bfloat16" \
        --tasks "$tasks" --device "cuda:$(( rank % 8 ))" --batch_size 32 --output_path "$out"
done
