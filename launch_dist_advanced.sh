#!/bin/bash
# Usage: bash launch_dist_advanced.sh <gpus_per_node> <num_nodes> <script.py> [args...]
# As launch_dist.sh, but first screens the allocation: nodes that do not answer a ping and nodes that
# an earlier run of this job reported in launch_info/<job>/failed_soft_nodes.txt are left out, and the
# job starts on the first <num_nodes> healthy nodes (fails if there are fewer).
if [ $# -lt 3 ]; then
    echo "Usage: bash $0 <gpus_per_node> <num_nodes> <script.py> [args...]"
    exit 1
fi
ppn=$1
num_nodes=$2
shift 2
cd "$(dirname "${BASH_SOURCE[0]}")" || exit 1
exec python -m optimus_lm_b200.launcher --gpus_per_node "$ppn" --num_nodes "$num_nodes" --health_check -- "$@"
