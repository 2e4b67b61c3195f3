"""Compare training runs from their logs: per-run summary, run-vs-first-run deviations and eight charts.

Same job and config format as the reference's compare_losses.py / compare_config.json:

    python compare_losses.py --config_path compare_config.json        # experiments named in the config
    python compare_losses.py                                          # every ./logs/*.txt as its own run

``exp_info_list`` in the config holds ``[experiment_dir_name, optional label]`` entries (looked up under
``pretrain_parallel_models[_archive]/``); with one entry each log file of that experiment is its own
curve, with none the ``*_temp`` experiments are listed.  Charts are PNG with matplotlib, SVG without.
"""
import argparse
import json
import os
import sys

from optimus_lm_b200 import log_analysis as la


def main(argv=None):
    p = argparse.ArgumentParser(description="Plot training loss and other metrics.")
    p.add_argument("--num_logs", type=int, default=None, help="Number of log files to consider from the last")
    p.add_argument("--min_loss", type=float, default=None)
    p.add_argument("--max_loss", type=float, default=None)
    p.add_argument("--start_step", type=int, default=None)
    p.add_argument("--end_step", type=int, default=None)
    p.add_argument("--start_tokens", type=float, default=None, help="in billions")
    p.add_argument("--end_tokens", type=float, default=None, help="in billions")
    p.add_argument("--skip_label", type=int, default=None)
    p.add_argument("--label_inside_plot", type=int, default=None)
    p.add_argument("--plot_dir", type=str, default=".")
    p.add_argument("--logs_dir", type=str, default="./logs")
    p.add_argument("--exp_dump_dir", type=str, default=".")
    p.add_argument("--config_path", type=str, default=None)
    p.add_argument("--analysis_choice", type=int, default=None)
    a = p.parse_args(argv)

    if a.config_path is not None:
        with open(a.config_path) as fh:
            cfg_all = json.load(fh)
        choice = cfg_all["analysis_choice"] if a.analysis_choice is None else a.analysis_choice
        cfg = cfg_all[f"analysis{choice}"]
        for key in ("min_loss", "max_loss", "start_step", "end_step", "start_tokens", "end_tokens", "num_logs"):
            if getattr(a, key) is None:
                setattr(a, key, cfg.get(key))
        a.skip_label = cfg.get("skip_label", False) if a.skip_label is None else a.skip_label == 1
        a.plot_dir = cfg.get("plot_dir", a.plot_dir)
        exp_info_list = cfg.get(f"exp_info_list{cfg.get('exp_group_id', '')}") or []
        if not exp_info_list:
            d = os.path.join(a.exp_dump_dir, "pretrain_parallel_models")
            temps = sorted((f for f in os.listdir(d) if f.endswith("_temp") and os.path.isdir(os.path.join(d, f))),
                           key=lambda f: os.path.getmtime(os.path.join(d, f))) if os.path.isdir(d) else []
            print("No experiments in the config. Temporary experiments found:")
            print(",\n".join(f'["{t}"]' for t in temps))
            return 0
        if len(exp_info_list) > 1:
            groups = [la.experiment_logs(e[0], a.exp_dump_dir) for e in exp_info_list]
            labels = [(e[1] if len(e) > 1 and e[1] is not None else e[0]) for e in exp_info_list]
            if a.num_logs is not None:
                groups = [g[-a.num_logs:] for g in groups]
        else:
            logs = la.experiment_logs(exp_info_list[0][0], a.exp_dump_dir)
            if a.num_logs is not None:
                logs = logs[-a.num_logs:]
            groups = [[f] for f in logs]
            labels = [os.path.basename(f)[:-4].replace("log_", "") for f in logs]
    else:
        logs = sorted(os.path.join(a.logs_dir, f) for f in os.listdir(a.logs_dir) if f.endswith(".txt"))
        if a.num_logs is not None:
            logs = logs[-a.num_logs:]
        groups = [[f] for f in logs]
        labels = [os.path.basename(f)[:-4].replace("log_", "") for f in logs]
        a.skip_label = bool(a.skip_label)

    runs = [la.filter_series(la.merge_logs(g), a.start_step, a.end_step, a.start_tokens, a.end_tokens) for g in groups]
    for label, run in zip(labels, runs):
        print(f"{label}: {la.summarize(run)}")
    for label, run in zip(labels[1:], runs[1:]):
        print(f"{labels[0]} vs {label}: {la.compare_series(runs[0], run)}")
    for path in la.plot_all(runs, labels, a.plot_dir, "training", a.min_loss, a.max_loss, bool(a.skip_label)):
        print("Plot saved at", path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
