#!/bin/bash
# Convert every completed checkpoint of an experiment to Hugging Face format (skips finished ones).
# Usage: bash evals/generate_hf_checkpoints.sh <exp_dir> <model_choice> [pp] [ep] [tp] [vpp]
set -euo pipefail
if [ $# -lt 2 ]; then
    echo "Usage: bash $0 <exp_dir> <model_choice> [pp] [ep] [tp] [vpp]"
    exit 1
fi
exp_dir=$1; model_choice=$2; pp=${3:-1}; ep=${4:-1}; tp=${5:-1}; vpp=${6:-1}
here="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
case "$model_choice" in
    *OLMoE*) script=convert_olmoe_ppep_om_checkpoint_to_hf.py ;;
    *)       script=convert_olmo_om_checkpoint_to_hf.py ;;
esac
mkdir -p "$exp_dir/hf_checkpoints"
for checkpoint in $(ls "$exp_dir/checkpoints" | grep -E "^(step|main)" | sort -V); do
    src="$exp_dir/checkpoints/$checkpoint"; dst="$exp_dir/hf_checkpoints/$checkpoint"
    if [ ! -f "$src/completed" ]; then
        echo "Checkpoint $checkpoint is not fully saved yet. Skipping."
    elif [ -f "$dst/completed" ]; then
        echo "Checkpoint $checkpoint already converted. Skipping."
    else
        echo "Processing $checkpoint"
        python "$here/$script" --model_choice "$model_choice" --om_checkpoint_dir "$src" --hf_checkpoint_dir "$dst" \
            --pipeline_parallelism "$pp" --expert_parallelism "$ep" --tensor_parallelism "$tp" --virtual_pipeline_parallelism "$vpp"
        touch "$dst/completed"
    fi
done
