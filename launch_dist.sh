#!/bin/bash
# Usage: [HOSTFILE_PATH=nodes.txt] bash launch_dist.sh <gpus_per_node> <num_nodes> <script.py> [args...]
# One process per GPU via torch.distributed.run on every node (see optimus_lm_b200/launcher.py).
if [ $# -lt 3 ]; then
    echo "Usage: bash $0 <gpus_per_node> <num_nodes> <script.py> [args...]"
    exit 1
fi
ppn=$1
num_nodes=$2
shift 2
cd "$(dirname "${BASH_SOURCE[0]}")" || exit 1
exec python -m optimus_lm_b200.launcher --gpus_per_node "$ppn" --num_nodes "$num_nodes" -- "$@"
