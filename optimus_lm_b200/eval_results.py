"""Collecting downstream-evaluation results (JSON files written by the ``lm_eval`` harness) into a
LaTeX-ready table and accuracy-vs-training-tokens curves.

Reference: evals/gather_eval_results.py (table of nine benchmarks + average over result directories)
and evals/generate_plots.py (per-benchmark and average accuracy against the ``step<N>-tokens<T>B``
checkpoint names).  Paths are arguments here; charts use the same writer as the loss comparison.
"""
from __future__ import annotations

import json
import os
import re
from collections import OrderedDict
from typing import Dict, List, Optional, Sequence

BENCHMARK_METRIC = OrderedDict([
    ("arc_easy", "acc_norm,none"), ("arc_challenge", "acc_norm,none"), ("hellaswag", "acc_norm,none"),
    ("piqa", "acc_norm,none"), ("boolq", "acc,none"), ("sciq", "acc,none"), ("winogrande", "acc,none"),
    ("openbookqa", "acc_norm,none"), ("mmlu", "acc,none"),
])
DEFAULT_TASKS = ",".join(BENCHMARK_METRIC)


def find_result_json(results_dir: str) -> str:
    """The newest ``*.json`` under ``results_dir`` (the harness nests one directory per model path)."""
    found = []
    for root, _, files in os.walk(results_dir):
        found += [os.path.join(root, f) for f in files if f.endswith(".json")]
    assert found, f"no JSON result file under {results_dir}"
    return max(found, key=os.path.getmtime)


def load_scores(results_dir: str) -> Dict[str, Optional[float]]:
    with open(find_result_json(results_dir)) as fh:
        res = json.load(fh)["results"]
    return {b: (res[b].get(m) if b in res else None) for b, m in BENCHMARK_METRIC.items()}


def average(scores: Dict[str, Optional[float]]) -> float:
    vals = [v for v in scores.values() if v is not None]
    return sum(vals) / len(vals) if vals else 0.0


def latex_table(results_dirs: Sequence[str]) -> str:
    cols = [load_scores(d) for d in results_dirs]
    lines = []
    for b in BENCHMARK_METRIC:
        cells = " & ".join("  -  " if c[b] is None else f"{c[b] * 100:.1f} " for c in cols)
        lines.append(f"{b:20s} & {cells}\\\\ \\hline")
    lines.append(f"{'Average':20s} & " + " & ".join(f"{average(c) * 100:.1f} " for c in cols) + "\\\\")
    return "\n".join(lines)


_CKPT_RE = re.compile(r"^step(\d+)-tokens(\d+)B$")


def checkpoint_curve(results_root: str) -> "OrderedDict[str, Dict[str, Optional[float]]]":
    """``step<N>-tokens<T>B`` sub-directories of ``results_root`` in step order -> scores."""
    names = sorted((n for n in os.listdir(results_root) if _CKPT_RE.match(n)),
                   key=lambda n: int(_CKPT_RE.match(n).group(1)))
    return OrderedDict((n, load_scores(os.path.join(results_root, n))) for n in names)


def plot_curves(results_roots: Sequence[str], labels: Sequence[str], plot_dir: str = "plots") -> List[str]:
    from . import log_analysis as la

    chart, ext = (la._mpl_chart, "png") if la.have_matplotlib() else (la._svg_chart, "svg")
    os.makedirs(plot_dir, exist_ok=True)
    curves = [checkpoint_curve(r) for r in results_roots]
    xs = [[int(_CKPT_RE.match(n).group(2)) for n in c] for c in curves]
    written = []
    for b in list(BENCHMARK_METRIC) + ["average_benchmark"]:
        series = []
        for c, x in zip(curves, xs):
            y = [(average(s) if b == "average_benchmark" else (s[b] or 0.0)) for s in c.values()]
            series.append((x, y))
        path = os.path.join(plot_dir, f"{b}_results.{ext}")
        if chart(series, list(labels), path, "Training Tokens (B)", "Accuracy"):
            written.append(path)
    return written
