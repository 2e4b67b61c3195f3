#!/bin/bash
# Create the working folders on a (large, shared) storage directory and link them into the repository root.
if [ $# -ne 1 ]; then
    echo "Usage: bash $0 <storage_dir>"
    exit 1
fi
storage=$1
for d in cached_models pretrain_parallel_models serial_models parallel_models job_logs launch_info datasets; do
    mkdir -p "$storage/$d"
    ln -sfn "$storage/$d" "$d"
done
