"""Experiment driver: environment variables -> experiment name + ``dist_train.py`` command line ->
launch, optionally repeated.

The reference drives experiments with ``run_experiment.sh`` (reference run_experiment.sh:6-501): some
80 environment variables select the model, the parallel layout, the optimizer and the debugging
switches, are folded into a canonical experiment name (which the loss-comparison and plotting tools
parse again) and into the argument list of ``dist_train.py``.  The same contract is implemented
here as testable Python; ``run_experiment.sh`` at the repository root is a two-line wrapper.

    NUM_NODES=1 GPUS_PER_NODE=8 EP=8 USE_FAST_MOE=1 USE_MERGED_MLP_IN_FAST_MOE=1 USE_OM_PGSHARDED_OPTIMIZER=1 \
        BATCH_SIZE=4 CONTEXT_SIZE=4096 bash run_experiment.sh

Differences: ``GPUS_PER_NODE`` defaults to 8; launching goes through ``launcher.py`` (torchrun on one
node, ``torchrun``-per-node over ssh/srun on several); ``SYNTHETIC_DATA`` / ``SYNTHETIC_INIT`` /
``TRAIN_STEPS`` expose the file-free mode of ``dist_train.py``; ``DRY_RUN=1`` prints the command only.
"""
from __future__ import annotations

import os
import shlex
import subprocess
import sys
import time
from dataclasses import dataclass, field
from typing import Dict, List, Mapping, Optional, Tuple

SUPPORTED_DATASETS = {
    "allenai/dolma": "dolma",
    "allenai/OLMoE-mix-0924": "olmoemix0924",
    "HuggingFaceFW/fineweb-edu": "finewebedu",
    "Salesforce/wikitext": "wikitext",
}

# variable -> default.  "null" means "leave dist_train.py's default".
DEFAULTS: Dict[str, str] = dict(
    FINAL="0", USE_ADVANCED_LAUNCHER="0", NUM_REPEATS="1", HOSTFILE_PATH="",
    MODEL_CHOICE="allenai/OLMoE-1B-7B-0924", DTYPE="bf16", USE_HF_MODEL="0", ENABLE_SAC="0", SAC_LEVEL="0",
    USE_FAST_MOE="0", USE_MERGED_MLP_IN_FAST_MOE="0", USE_TRITON_PATH_FOR_GEMM_IN_FAST_MOE="0",
    USE_TRITON_PATH_FOR_NONGEMM_IN_FAST_MOE="0", FORCE_UNIFORM_ROUTING="0", USE_LOCAL_ROUTER_AUX_LOSS="0",
    DISABLE_MODEL_CACHING="0", USE_OM_CACHED_MODEL="0", INIT_MODEL_DIR="null", USE_BROADCAST_FOR_MODEL_INIT="1",
    USE_ALLREDUCE_IN_BROADCAST_MODEL_INIT="0",
    PP="1", EP="1", TP="1", VPP="1", USE_SP_IN_TP="0", PP_SCHEME="gpipe", REUSE_BUFFERS_IN_1F1B="1", USE_PP_FIRST="0",
    BATCH_SIZE="1", MICRO_BATCH_SIZE="1", NUM_NODES="1", GPUS_PER_NODE="8",
    DATASET_CHOICE="allenai/OLMoE-mix-0924", NUM_DATA_FILES="-1", TOKENIZER="olmo", USE_SHARDED_DATASET="0",
    CONTEXT_SIZE="2048", GRAD_ACC_STEPS="1",
    USE_PT_OPTIMIZER="0", USE_OM_OPTIMIZER="0", USE_OM_SHARDED_OPTIMIZER="0", USE_OM_SUBSHARDED_OPTIMIZER="0",
    USE_OM_PGSHARDED_OPTIMIZER="0", USE_OM_PGSUBSHARDED_OPTIMIZER="0", OPT_USE_ALLREDUCE_FOR_GRAD_ACC="0",
    OPT_USE_ALLREDUCE_FOR_PARAM_GATHER="0", OPT_USE_CHUNKED_ALLREDUCE="0", OPT_USE_FP32_FOR_GRAD_ACC="0",
    DISABLE_DELAYED_GRAD_CLIPPING="0", USE_ONE_STEP_GRAD_CLIPPING="0",
    LR="null", MIN_LR="null", WARMUP_STEPS="null", LR_TRAIN_STEPS="null", LR_SCHEDULE="null", WEIGHT_DECAY="null",
    ENABLE_CHECKPOINTING="1", DISABLE_COLD_CHECKPOINTING="0", DP_STAGGERED_CHECKPOINTING="0",
    DISABLE_OPTIMIZER_STATE_CHECKPOINTING="0", CHECKPOINT_STEPS="1000", DEBUG="0", PAPER="0", PROFILE="0",
    PROFILE_MODULES="0", LOG_MEMORY_USAGE="0", DUMP_WEIGHT_GRADIENTS="0", ENABLE_BAD_GRAD_CHECK="0",
    SKIP_OPTIMIZER_STEP="0", SKIP_OPTIMIZER_STEP_WEIGHT_UPDATE="0", SKIP_BACKWARD_PASS="0", LOG_ALL_RANKS="0",
    ENABLE_PP_DEBUG="0", VERBOSE="0", EXIT_STEPS="-1", ENABLE_TB_LOGGING="0", USE_LATEST_TRAINER="0",
    STORAGE_DIR=".", SYNTHETIC_DATA="0", SYNTHETIC_INIT="0", TRAIN_STEPS="null", DRY_RUN="0",
)

_OPTIMIZER_SWITCHES = ("USE_PT_OPTIMIZER", "USE_OM_OPTIMIZER", "USE_OM_SHARDED_OPTIMIZER", "USE_OM_PGSHARDED_OPTIMIZER",
                       "USE_OM_SUBSHARDED_OPTIMIZER", "USE_OM_PGSUBSHARDED_OPTIMIZER")


class ExperimentError(ValueError):
    pass


@dataclass
class Experiment:
    env: Dict[str, str]
    name: str = ""
    args: List[str] = field(default_factory=list)
    exp_dir: str = ""
    num_gpus: int = 1
    dp: int = 1
    global_batch_size: int = 1

    def flag(self, key) -> bool:
        return int(self.env[key]) == 1

    def num(self, key) -> int:
        return int(self.env[key])


def resolve_env(environ: Optional[Mapping[str, str]] = None) -> Dict[str, str]:
    environ = os.environ if environ is None else environ
    env = {k: str(environ.get(k, d)) for k, d in DEFAULTS.items()}
    if not env["HOSTFILE_PATH"]:
        env["HOSTFILE_PATH"] = environ.get("PBS_NODEFILE", "")
    env["JOB_ID"] = str(environ.get("PBS_JOBID", environ.get("SLURM_JOB_ID", "0")))
    return env


def build_experiment(environ: Optional[Mapping[str, str]] = None) -> Experiment:
    """Validate the variables and derive the experiment name, directory and argument list."""
    x = Experiment(env=resolve_env(environ))
    e, flag, num = x.env, x.flag, x.num
    if e["DATASET_CHOICE"] not in SUPPORTED_DATASETS:
        raise ExperimentError(f"Unsupported dataset choice. Supported datasets are: {' '.join(SUPPORTED_DATASETS)}")
    if sum(num(k) for k in _OPTIMIZER_SWITCHES) != 1:
        raise ExperimentError("Exactly one of " + ", ".join(_OPTIMIZER_SWITCHES) + " must be set to 1.")
    for dim in ("PP", "EP", "TP"):
        if num(dim) != 1 and flag("USE_HF_MODEL"):
            raise ExperimentError(f"{dim} can only be used with USE_HF_MODEL set to 0.")
    pp, ep, tp, vpp = num("PP"), num("EP"), num("TP"), num("VPP")
    x.num_gpus = num("NUM_NODES") * num("GPUS_PER_NODE")
    if x.num_gpus % (pp * ep * tp) != 0:
        raise ExperimentError(f"NUM_NODES*GPUS_PER_NODE = {x.num_gpus} is not a multiple of PP*EP*TP = {pp * ep * tp}")
    x.dp = x.num_gpus // (pp * ep * tp)
    x.global_batch_size = x.dp * ep * num("BATCH_SIZE")

    model_key = e["MODEL_CHOICE"].split("/")[1] if "/" in e["MODEL_CHOICE"] else e["MODEL_CHOICE"]
    dataset_key = e["DATASET_CHOICE"].replace("/", "_")
    storage = e["STORAGE_DIR"]
    dataset_dir = f"{storage}/datasets/{dataset_key}/preprocessed/{e['TOKENIZER']}/"
    a: List[str] = ["--model_choice", e["MODEL_CHOICE"], "--dataset_dir", dataset_dir, "--dtype", e["DTYPE"],
                    "--batch_size", e["BATCH_SIZE"], "--context_size", e["CONTEXT_SIZE"],
                    "--opt_grad_acc_steps", e["GRAD_ACC_STEPS"],
                    "--data_parallelism", str(x.dp), "--pipeline_parallelism", str(pp), "--expert_parallelism", str(ep),
                    "--tensor_parallelism", str(tp), "--virtual_pipeline_parallelism", str(vpp)]
    for key, opt in (("LR", "--lr"), ("MIN_LR", "--min_lr"), ("WARMUP_STEPS", "--warmup_steps"),
                     ("LR_SCHEDULE", "--lr_schedule"), ("WEIGHT_DECAY", "--weight_decay"),
                     ("LR_TRAIN_STEPS", "--lr_train_steps"), ("TRAIN_STEPS", "--train_steps")):
        if e[key] != "null":
            a += [opt, e[key]]

    name = model_key + "_" + SUPPORTED_DATASETS[e["DATASET_CHOICE"]]
    if flag("USE_HF_MODEL"):
        a.append("--use_hf_model")
        name += "_hf"
    else:
        name += "_om"
        if flag("USE_OM_CACHED_MODEL"):
            a += ["--use_om_cached_model", "--om_cached_models_dir", f"{storage}/parallel_models"]
            name += "_omcached"
        if e["INIT_MODEL_DIR"] != "null":
            a += ["--init_model_dir", e["INIT_MODEL_DIR"]]
            name += "_finetune"
        if "OLMoE" in e["MODEL_CHOICE"]:
            if flag("USE_LOCAL_ROUTER_AUX_LOSS"):
                a.append("--use_local_router_aux_loss")
                name += "_lral"
            else:
                name += "_gral"
            if flag("FORCE_UNIFORM_ROUTING"):
                a.append("--force_uniform_routing")
                name += "_fur"
            if flag("USE_FAST_MOE"):
                a.append("--use_fast_moe")
                name += "_fastmoe"
                for key, opt, tag in (("USE_MERGED_MLP_IN_FAST_MOE", "--use_merged_mlp_in_fast_moe", "-mmlp"),
                                      ("USE_TRITON_PATH_FOR_GEMM_IN_FAST_MOE", "--use_triton_path_for_gemm_in_fast_moe", "-tritongemm"),
                                      ("USE_TRITON_PATH_FOR_NONGEMM_IN_FAST_MOE", "--use_triton_path_for_nongemm_in_fast_moe", "-tritonnongemm")):
                    if flag(key):
                        a.append(opt)
                        name += tag
        if "DeepSeek" in e["MODEL_CHOICE"] and flag("FORCE_UNIFORM_ROUTING"):
            a.append("--force_uniform_routing")
            name += "_fur"
        if flag("ENABLE_SAC"):
            a += ["--use_activation_checkpointing", "--activation_checkpointing_level", e["SAC_LEVEL"]]
            name += f"_ac{e['SAC_LEVEL']}"

    name += f"_{e['DTYPE']}_n{e['NUM_NODES']}xg{e['GPUS_PER_NODE']}"
    name += f"_gbs{x.global_batch_size}-bs{e['BATCH_SIZE']}-cs{e['CONTEXT_SIZE']}-gas{e['GRAD_ACC_STEPS']}"
    name += f"_dp{x.dp}-pp{pp}-ep{ep}-tp{tp}"
    if vpp != 1:
        name += f"-vpp{vpp}"
    if tp != 1 and flag("USE_SP_IN_TP"):
        a.append("--use_sequence_parallelism_in_tp")
        name += "_sp1"
    if pp != 1:
        a += ["--pp_scheme", e["PP_SCHEME"], "--micro_batch_size", e["MICRO_BATCH_SIZE"]]
        name += f"-ps{e['PP_SCHEME']}-mbs{e['MICRO_BATCH_SIZE']}"
        if e["PP_SCHEME"] == "1f1b":
            if flag("REUSE_BUFFERS_IN_1F1B"):
                a.append("--reuse_buffers_in_1f1b")
            name += f"-rb{e['REUSE_BUFFERS_IN_1F1B']}"
        if flag("USE_PP_FIRST"):
            a.append("--use_pp_first")
            name += "-ppfirst"

    if flag("USE_PT_OPTIMIZER"):
        a.append("--opt_use_pt_optimizer")
        name += "_ptopt-ddp"
    else:
        for key, opt, tag in (("USE_OM_OPTIMIZER", None, "_omopt-ddp"),
                              ("USE_OM_SHARDED_OPTIMIZER", "--opt_use_sharded_optimizer", "_omopt-shard"),
                              ("USE_OM_SUBSHARDED_OPTIMIZER", "--opt_use_subsharded_optimizer", "_omopt-subshard"),
                              ("USE_OM_PGSHARDED_OPTIMIZER", "--opt_use_pgsharded_optimizer", "_omopt-pgshard"),
                              ("USE_OM_PGSUBSHARDED_OPTIMIZER", "--opt_use_pgsubsharded_optimizer", "_omopt-pgsubshard"),
                              ("OPT_USE_FP32_FOR_GRAD_ACC", "--opt_use_fp32_for_grad_acc", "-gafp32"),
                              ("OPT_USE_ALLREDUCE_FOR_GRAD_ACC", "--opt_use_allreduce_for_grad_acc", "-gaar"),
                              ("OPT_USE_ALLREDUCE_FOR_PARAM_GATHER", "--opt_use_allreduce_for_param_gather", "-pgar"),
                              ("OPT_USE_CHUNKED_ALLREDUCE", "--opt_use_chunked_allreduce", "-arch")):
            if flag(key):
                if opt:
                    a.append(opt)
                name += tag
    for key, opt, tag in (("DISABLE_DELAYED_GRAD_CLIPPING", "--opt_disable_delayed_grad_clipping", "-gcfromstart"),
                          ("USE_ONE_STEP_GRAD_CLIPPING", "--opt_use_one_step_grad_clipping", "-onestepgc"),
                          ("SKIP_OPTIMIZER_STEP", "--skip_optimizer_step", "_skipoptstep"),
                          ("SKIP_OPTIMIZER_STEP_WEIGHT_UPDATE", "--skip_optimizer_step_weight_update", "_skipoptstepwupdate"),
                          ("LOG_MEMORY_USAGE", "--log_memory_usage", ""),
                          ("DUMP_WEIGHT_GRADIENTS", "--dump_weight_gradients", ""),
                          ("SKIP_BACKWARD_PASS", "--skip_backward_pass", "_skipbwd"),
                          ("DISABLE_MODEL_CACHING", "--disable_model_caching", ""),
                          ("PROFILE", "--profile", "_profile"),
                          ("PROFILE_MODULES", "--profile_modules", "_profilemods")):
        if flag(key):
            a.append(opt)
            name += tag
    if flag("FINAL"):
        name += "_final"
    elif flag("DEBUG"):
        name += "_debug"
    elif flag("PAPER"):
        name += "_paper"
    else:
        name += "_temp"

    if num("NUM_DATA_FILES") != -1:
        a += ["--num_data_files", e["NUM_DATA_FILES"]]
    for key, opt in (("USE_SHARDED_DATASET", "--use_sharded_dataset"), ("VERBOSE", "--verbose"),
                     ("ENABLE_TB_LOGGING", "--enable_tb_logging"), ("ENABLE_BAD_GRAD_CHECK", "--enable_bad_grad_check"),
                     ("LOG_ALL_RANKS", "--log_all_ranks"), ("ENABLE_PP_DEBUG", "--enable_pp_debug"),
                     ("SYNTHETIC_DATA", "--synthetic_data"), ("SYNTHETIC_INIT", "--synthetic_init")):
        if flag(key):
            a.append(opt)
    if flag("ENABLE_CHECKPOINTING"):
        a += ["--enable_checkpointing", "--checkpoint_steps", e["CHECKPOINT_STEPS"]]
        for key, opt in (("DISABLE_OPTIMIZER_STATE_CHECKPOINTING", "--disable_optimizer_state_checkpointing"),
                         ("DISABLE_COLD_CHECKPOINTING", "--disable_cold_checkpointing"),
                         ("DP_STAGGERED_CHECKPOINTING", "--dp_staggered_checkpointing")):
            if flag(key):
                a.append(opt)
    if num("EXIT_STEPS") != -1:
        a += ["--exit_steps", e["EXIT_STEPS"]]
    for key, opt in (("USE_BROADCAST_FOR_MODEL_INIT", "--use_broadcast_for_model_init"),
                     ("USE_ALLREDUCE_IN_BROADCAST_MODEL_INIT", "--use_allreduce_in_broadcast_model_init"),
                     ("USE_LATEST_TRAINER", "--use_latest_trainer")):
        if flag(key):
            a.append(opt)
    x.name = name
    x.exp_dir = f"{storage}/pretrain_parallel_models/{name}"
    a += ["--exp_dir", x.exp_dir, "--cached_models_dir", f"{storage}/cached_models"]
    x.args = a
    return x


def launch_command(x: Experiment, repo_root: str) -> List[str]:
    """Full process command line: launcher prefix (when more than one GPU) + ``dist_train.py`` + args."""
    train = [sys.executable, os.path.join(repo_root, "dist_train.py")] + x.args
    if x.num_gpus <= 1:
        return train
    launcher = [sys.executable, "-m", "optimus_lm_b200.launcher", "--gpus_per_node", x.env["GPUS_PER_NODE"],
                "--num_nodes", x.env["NUM_NODES"]]
    if x.env["HOSTFILE_PATH"]:
        launcher += ["--hostfile", x.env["HOSTFILE_PATH"]]
    if x.flag("USE_ADVANCED_LAUNCHER"):
        launcher.append("--health_check")
    return launcher + ["--"] + train[1:]


def run(environ: Optional[Mapping[str, str]] = None, repo_root: Optional[str] = None) -> int:
    repo_root = repo_root or os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        x = build_experiment(environ)
    except ExperimentError as err:
        print(f"Error: {err}")
        return 1
    storage = x.env["STORAGE_DIR"]
    cmd = launch_command(x, repo_root)
    if x.flag("DRY_RUN"):
        print(" ".join(shlex.quote(c) for c in cmd))
        return 0
    for d in (f"{storage}/cached_models", x.exp_dir, f"{x.exp_dir}/checkpoints/checkpoint1",
              f"{x.exp_dir}/checkpoints/checkpoint2"):
        os.makedirs(d, exist_ok=True)
    rc = 0
    for i in range(x.num("NUM_REPEATS")):
        if i > 0:
            time.sleep(60)  # let the file system and the fabric settle between repeats
        log_path = os.path.join(x.exp_dir, f"log_{x.env['JOB_ID']}_{time.strftime('%Y%m%d_%H%M%S')}.txt")
        print(" ".join(shlex.quote(c) for c in cmd) + f" | tee {log_path}", flush=True)
        with open(log_path, "w") as log:
            proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=repo_root)
            for line in proc.stdout:
                sys.stdout.write(line)
                sys.stdout.flush()
                log.write(line)
                log.flush()
            rc = proc.wait()
    return rc


if __name__ == "__main__":
    sys.exit(run())
