#!/bin/bash
# Experiment driver.  Environment variables select the model, layout, optimizer and debug switches
# (the list and its defaults are in optimus_lm_b200/experiment.py); they are folded into the
# experiment name and the dist_train.py command line, which is then launched NUM_REPEATS times.
#   NUM_NODES=1 GPUS_PER_NODE=8 EP=8 USE_FAST_MOE=1 USE_MERGED_MLP_IN_FAST_MOE=1 \
#   USE_OM_PGSHARDED_OPTIMIZER=1 BATCH_SIZE=4 CONTEXT_SIZE=4096 SYNTHETIC_DATA=1 SYNTHETIC_INIT=1 bash run_experiment.sh
cd "$(dirname "${BASH_SOURCE[0]}")" || exit 1
exec python -m optimus_lm_b200.experiment "$@"
