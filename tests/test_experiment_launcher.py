"""Experiment naming / argument rules and the launcher's node health screen (host-side only)."""
import os

import pytest

from optimus_lm_b200 import experiment, launcher


def test_experiment_name_and_arguments_follow_the_naming_contract():
    x = experiment.build_experiment(dict(
        MODEL_CHOICE="allenai/OLMoE-1B-7B-0924--SE1.125", NUM_NODES="2", GPUS_PER_NODE="8", PP="2", EP="4",
        PP_SCHEME="1f1b", MICRO_BATCH_SIZE="1", BATCH_SIZE="8", CONTEXT_SIZE="4096", USE_FAST_MOE="1",
        USE_MERGED_MLP_IN_FAST_MOE="1", USE_OM_CACHED_MODEL="1", USE_OM_PGSHARDED_OPTIMIZER="1",
        OPT_USE_ALLREDUCE_FOR_PARAM_GATHER="1", ENABLE_SAC="1", SAC_LEVEL="1", FINAL="1", LR="4e-4", EXIT_STEPS="32"))
    assert x.dp == 2 and x.global_batch_size == 2 * 4 * 8
    assert x.name == ("OLMoE-1B-7B-0924--SE1.125_olmoemix0924_om_omcached_gral_fastmoe-mmlp_ac1_bf16_n2xg8"
                      "_gbs64-bs8-cs4096-gas1_dp2-pp2-ep4-tp1-ps1f1b-mbs1-rb1_omopt-pgshard-pgar_final")
    a = x.args
    assert a[a.index("--data_parallelism") + 1] == "2" and a[a.index("--expert_parallelism") + 1] == "4"
    for opt in ("--use_fast_moe", "--use_merged_mlp_in_fast_moe", "--use_om_cached_model", "--opt_use_pgsharded_optimizer",
                "--opt_use_allreduce_for_param_gather", "--reuse_buffers_in_1f1b", "--enable_checkpointing",
                "--use_broadcast_for_model_init", "--use_activation_checkpointing"):
        assert opt in a, opt
    assert a[a.index("--lr") + 1] == "4e-4" and a[a.index("--exit_steps") + 1] == "32"
    assert a[a.index("--exp_dir") + 1] == "./pretrain_parallel_models/" + x.name
    assert "--min_lr" not in a and "--use_pp_first" not in a


def test_experiment_accepts_every_flag_dist_train_knows():
    """Every option the experiment driver can emit must be an option of dist_train.py."""
    import dist_train
    parser_opts = set()
    for act in dist_train.build_parser()._actions:
        parser_opts.update(act.option_strings)
    env = {k: "1" for k, v in experiment.DEFAULTS.items() if v == "0"}
    for k in experiment._OPTIMIZER_SWITCHES:
        env[k] = "0"
    env.update(USE_HF_MODEL="0", USE_OM_SHARDED_OPTIMIZER="1", PP="2", TP="2", GPUS_PER_NODE="8", PP_SCHEME="1f1b",
               LR="1e-3", MIN_LR="1e-4", WARMUP_STEPS="10", LR_TRAIN_STEPS="100", LR_SCHEDULE="linear",
               WEIGHT_DECAY="0.1", TRAIN_STEPS="5", INIT_MODEL_DIR="/x", NUM_DATA_FILES="3", EXIT_STEPS="4",
               NUM_REPEATS="1")
    x = experiment.build_experiment(env)
    emitted = {t for t in x.args if t.startswith("--")}
    assert emitted <= parser_opts, emitted - parser_opts


def test_experiment_validation_errors():
    with pytest.raises(experiment.ExperimentError, match="Exactly one"):
        experiment.build_experiment({})
    with pytest.raises(experiment.ExperimentError, match="Unsupported dataset"):
        experiment.build_experiment(dict(USE_OM_OPTIMIZER="1", DATASET_CHOICE="x/y"))
    with pytest.raises(experiment.ExperimentError, match="EP can only"):
        experiment.build_experiment(dict(USE_PT_OPTIMIZER="1", USE_HF_MODEL="1", EP="2"))
    assert experiment.run(dict(DRY_RUN="1")) == 1


def test_dry_run_prints_launcher_command(capsys):
    assert experiment.run(dict(DRY_RUN="1", USE_OM_OPTIMIZER="1", GPUS_PER_NODE="2", USE_ADVANCED_LAUNCHER="1")) == 0
    out = capsys.readouterr().out
    assert "optimus_lm_b200.launcher" in out and "--health_check" in out and "dist_train.py" in out
    assert experiment.run(dict(DRY_RUN="1", USE_OM_OPTIMIZER="1", GPUS_PER_NODE="1")) == 0
    assert "launcher" not in capsys.readouterr().out


def test_select_nodes_drops_hard_and_soft_failures():
    nodes = [f"n{i}" for i in range(6)]
    logs = []
    got = launcher.select_nodes(nodes, 3, probe=lambda n: n != "n1", soft_failed=["n2", "zz"], log=logs.append)
    assert got == ["n0", "n3", "n4"]
    assert "Number of hard failed nodes : 1" in logs and "Failed soft nodes : n2" in logs
    with pytest.raises(RuntimeError, match="Required: 5, Available: 4"):
        launcher.select_nodes(nodes, 5, probe=lambda n: n != "n1", soft_failed=["n2"], log=logs.append)


def test_launcher_multi_node_commands_and_soft_failure_file(tmp_path, monkeypatch):
    hostfile = tmp_path / "hosts"
    hostfile.write_text("a slots=8\nb\nb\nc\n# comment\nd\n")
    assert launcher.read_hostfile(str(hostfile)) == ["a", "b", "c", "d"]
    monkeypatch.setenv("OPTIMUS_LAUNCH_INFO_DIR", str(tmp_path / "li"))
    monkeypatch.setenv("PBS_JOBID", "123.head")
    monkeypatch.delenv("SLURM_JOB_ID", raising=False)
    info = launcher.launch_info_dir()
    assert info.endswith("li/123")
    os.makedirs(info)
    with open(os.path.join(info, "failed_soft_nodes.txt"), "w") as fh:
        fh.write("a\n")
    started = []

    class P:
        def wait(self):
            return 0

    rc = launcher.main(["--gpus_per_node", "8", "--num_nodes", "2", "--hostfile", str(hostfile), "--health_check",
                        "--", "dist_train.py", "--x", "1"], probe=lambda n: n != "b",
                       spawn=lambda c: started.append(c) or P())
    assert rc == 0 and len(started) == 2
    assert started[0][:4] == ["ssh", "-o", "BatchMode=yes", "c"] and started[1][3] == "d"
    assert "--node-rank=1" in started[1][-1] and "--master-addr c" in started[1][-1] and "--nnodes=2" in started[0][-1]
    assert open(os.path.join(info, "hostfile")).read() == "c\nd\n"
    # too few healthy nodes
    rc = launcher.main(["--num_nodes", "3", "--hostfile", str(hostfile), "--health_check", "--", "x.py"],
                       probe=lambda n: n != "b", spawn=lambda c: P())
    assert rc == 1


def test_single_node_command_uses_loopback_rendezvous():
    cmds = launcher.node_commands(["127.0.0.1"], ["dist_train.py", "--a"], 4, 29511, "local", "/tmp")
    assert len(cmds) == 1 and "--nproc-per-node=4" in cmds[0] and cmds[0][-2:] == ["dist_train.py", "--a"]
    assert cmds[0][cmds[0].index("--master-addr") + 1] == "127.0.0.1"


def test_gpu_health_report_parses_read_only_query():
    fake = "0, 0, Not Active, Not Active\n1, 3, Not Active, Not Active\n2, 0, Active, Not Active\n3, [N/A], Not Active, Not Active\n"
    got = launcher.gpu_health_report(lambda: fake)
    assert got == ["GPU 1: 3 uncorrected ECC errors", "GPU 2: hardware slowdown active"]
