#!/bin/bash
# Download every file of <dataset_dir>/urls_<category>.txt into <dataset_dir>/data/<category>/ with
# resumable parallel transfers.  Usage: bash scripts/download.sh <dataset_dir> [parallel_downloads]
set -euo pipefail
if [ $# -lt 1 ]; then
    echo "Usage: bash $0 <dataset_dir> [parallel_downloads]"
    exit 1
fi
dataset_dir=$1
parallel=${2:-8}
mkdir -p "$dataset_dir/data"
for list in "$dataset_dir"/urls_*.txt; do
    category=$(basename "$list" .txt)
    category=${category#urls_}
    echo "Downloading $category"
    mkdir -p "$dataset_dir/data/$category"
    xargs -a "$list" -n 1 -P "$parallel" wget -c -q -P "$dataset_dir/data/$category"
done
echo "Dataset download completed."
