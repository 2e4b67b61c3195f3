#!/bin/bash
# Build the CUDA extension (sm_100a) and the stand-alone C library in-tree.
set -e
cd "$(dirname "${BASH_SOURCE[0]}")"
MAX_JOBS=${MAX_JOBS:-8} python setup.py build_ext --inplace
python -c "import optimus_lm_b200.ops._ext as e; print('extension:', e.extension().__file__)"
