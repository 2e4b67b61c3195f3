"""Accuracy-vs-training-tokens curves (one chart per benchmark + the average) for one or more runs.

    python evals/generate_plots.py --results_roots <exp>/results <other>/results --labels mine baseline
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200.eval_results import plot_curves  # noqa: E402

if __name__ == "__main__":
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--results_roots", nargs="+", required=True, help="directories holding step<N>-tokens<T>B/ results")
    p.add_argument("--labels", nargs="+", default=None)
    p.add_argument("--plot_dir", type=str, default="plots")
    a = p.parse_args()
    for f in plot_curves(a.results_roots, a.labels or a.results_roots, a.plot_dir):
        print("Plot saved at", f)
