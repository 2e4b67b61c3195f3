"""Print the benchmark table (LaTeX rows) of one or more evaluation result directories.

    python evals/gather_eval_results.py --results_dir_list results/step10000-tokens63B results/main
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from optimus_lm_b200.eval_results import latex_table  # noqa: E402

if __name__ == "__main__":
    p = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    p.add_argument("--results_dir_list", nargs="+", type=str, default=["results/checkpoint_hf"])
    print(latex_table(p.parse_args().results_dir_list))
