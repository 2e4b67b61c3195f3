"""Training-log analysis: parse the step lines ``dist_train.py`` prints, filter, summarise, compare
runs numerically and plot.

The reference's ``compare_losses.py`` parses the same line format (compare_losses.py:31-74) and
draws eight charts per comparison (loss vs step / tokens / wall time, gradient norm vs step / tokens,
LR, tokens/s/GPU, TFLOP/s; compare_losses.py:130-400).  Added here: ``compare_series`` - the largest
loss / grad-norm deviation between two runs over their common steps, which is how a parallel layout
is checked against a serial run - and a chart writer that needs no plotting library (SVG), used when
``matplotlib`` is not installed.
"""
from __future__ import annotations

import math
import os
import re
from typing import Dict, List, Optional, Sequence

KEYS = ["step_id", "loss_value", "grad_norm", "lr", "step_time", "tokens_processed", "tokens_per_sec", "time_stamp",
        "tflops", "world_size"]

_NUM = r"([+-]?(?:\d+\.?\d*|\.\d+)(?:[eE][+-]?\d+)?|nan|inf)"
_STEP_RE = re.compile(r"Step\s*(\d+).*?Loss\s*:\s*" + _NUM + r".*?Grad norm\s*:\s*" + _NUM + r".*?LR\s*:\s*" + _NUM +
                      r".*?Time\s*:\s*" + _NUM + r".*?Tokens Processed\s*:\s*(\d+).*?Tokens/sec\s*:\s*(\d+)")
_WORLD_RE = re.compile(r"(?:PMI_SIZE|WORLD_SIZE|World size)\s*[=:]\s*(\d+)")
_TS_RE = re.compile(r"Timestamp\s*:\s*" + _NUM)
_TF_RE = re.compile(r"Tflops\s*:\s*" + _NUM)


def parse_log(path: str) -> Dict[str, list]:
    """Step series of one log file, sorted by step id."""
    rows = []
    world = 1
    with open(path, "r", errors="replace") as fh:
        for line in fh:
            w = _WORLD_RE.search(line)
            if w:
                world = int(w.group(1))
            m = _STEP_RE.search(line)
            if not m:
                continue
            ts = _TS_RE.search(line)
            tf = _TF_RE.search(line)
            rows.append((int(m.group(1)), float(m.group(2)), float(m.group(3)), float(m.group(4)), float(m.group(5)),
                         int(m.group(6)), int(m.group(7)), float(ts.group(1)) if ts else None,
                         float(tf.group(1)) if tf else 0.0, world))
    rows.sort(key=lambda r: r[0])
    return {k: [r[i] for r in rows] for i, k in enumerate(KEYS)}


def merge_logs(paths: Sequence[str]) -> Dict[str, list]:
    """Concatenate the series of the logs of one experiment (a run resumed several times); when a step
    appears in more than one log the latest file wins."""
    by_step = {}
    for p in paths:
        d = parse_log(p)
        for i, s in enumerate(d["step_id"]):
            by_step[s] = tuple(d[k][i] for k in KEYS)
    rows = [by_step[s] for s in sorted(by_step)]
    return {k: [r[i] for r in rows] for i, k in enumerate(KEYS)}


def filter_series(d: Dict[str, list], start_step=None, end_step=None, start_tokens=None, end_tokens=None):
    """Keep steps in [start_step, end_step] and token counts (in billions) in [start_tokens, end_tokens]."""
    keep = []
    for i, s in enumerate(d["step_id"]):
        tb = d["tokens_processed"][i] * 1e-9
        if (start_step is not None and s < start_step) or (end_step is not None and s > end_step):
            continue
        if (start_tokens is not None and tb < start_tokens) or (end_tokens is not None and tb > end_tokens):
            continue
        keep.append(i)
    return {k: [v[i] for i in keep] for k, v in d.items()}


def summarize(d: Dict[str, list]) -> Dict[str, float]:
    n = len(d["step_id"])
    if n == 0:
        return {"steps": 0}
    out = {"steps": n, "first_step": d["step_id"][0], "last_step": d["step_id"][-1], "last_loss": d["loss_value"][-1],
           "last_grad_norm": d["grad_norm"][-1], "tokens_processed": d["tokens_processed"][-1]}
    if n > 1:
        tf = d["tflops"][1:]
        out["avg_tflops"] = sum(tf) / len(tf)
        t0, t1 = d["time_stamp"][0], d["time_stamp"][-1]
        if t0 is not None and t1 is not None and t1 > t0:
            tokens = d["tokens_processed"][-1] - d["tokens_processed"][0]
            out["wall_time_s"] = t1 - t0
            out["tokens_per_sec_per_gpu"] = (tokens / (t1 - t0)) / max(1, d["world_size"][0])
    return out


def compare_series(a: Dict[str, list], b: Dict[str, list]) -> Dict[str, float]:
    """Largest absolute and relative deviation of loss and gradient norm over the steps both runs have."""
    ia = {s: i for i, s in enumerate(a["step_id"])}
    common = [s for s in b["step_id"] if s in ia]
    out = {"common_steps": len(common)}
    ib = {s: i for i, s in enumerate(b["step_id"])}
    for key in ("loss_value", "grad_norm"):
        mx, mr = 0.0, 0.0
        for s in common:
            x, y = a[key][ia[s]], b[key][ib[s]]
            if math.isnan(x) or math.isnan(y):
                mx = mr = float("nan")
                break
            mx = max(mx, abs(x - y))
            mr = max(mr, abs(x - y) / max(abs(x), 1e-12))
        out[f"max_abs_diff_{key}"] = mx
        out[f"max_rel_diff_{key}"] = mr
    return out


# ---------------------------------------------------------------- charts

_COLORS = ["#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#bcbd22", "#17becf"]


def _svg_chart(series, labels, path, xlabel, ylabel, logy=False, ymin=None, ymax=None, hlines=(), points=False):
    W, H, L, R, T, B = 900, 520, 70, 20, 20, 50 + 16 * len(labels)
    xs = [x for s in series for x in s[0]]
    ys = [y for s in series for y in s[1] if (not logy or y > 0)]
    if not xs or not ys:
        return False
    tr = (lambda v: math.log10(v)) if logy else (lambda v: v)
    x0, x1 = min(xs), max(xs)
    y0 = tr(ymin) if ymin is not None else min(tr(y) for y in ys)
    y1 = tr(ymax) if ymax is not None else max(tr(y) for y in ys)
    if x1 == x0:
        x1 = x0 + 1
    if y1 == y0:
        y1 = y0 + 1
    px = lambda x: L + (x - x0) / (x1 - x0) * (W - L - R)
    py = lambda y: T + (1 - (tr(y) - y0) / (y1 - y0)) * (H - T - B)
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{W}" height="{H}" font-family="sans-serif" font-size="12">',
           f'<rect width="{W}" height="{H}" fill="white"/>',
           f'<rect x="{L}" y="{T}" width="{W - L - R}" height="{H - T - B}" fill="none" stroke="black"/>']
    for i in range(6):
        gx = x0 + (x1 - x0) * i / 5
        gy = y0 + (y1 - y0) * i / 5
        yy = T + (1 - i / 5) * (H - T - B)
        out.append(f'<line x1="{px(gx):.1f}" y1="{T}" x2="{px(gx):.1f}" y2="{H - B}" stroke="#ddd"/>')
        out.append(f'<line x1="{L}" y1="{yy:.1f}" x2="{W - R}" y2="{yy:.1f}" stroke="#ddd"/>')
        out.append(f'<text x="{px(gx):.1f}" y="{H - B + 15}" text-anchor="middle">{gx:.4g}</text>')
        lab = 10 ** gy if logy else gy
        out.append(f'<text x="{L - 5}" y="{yy + 4:.1f}" text-anchor="end">{lab:.4g}</text>')
    out.append(f'<text x="{(L + W - R) / 2}" y="{H - B + 32}" text-anchor="middle">{xlabel}</text>')
    out.append(f'<text x="14" y="{(T + H - B) / 2}" text-anchor="middle" transform="rotate(-90 14 {(T + H - B) / 2})">{ylabel}</text>')
    for k, ((sx, sy), label) in enumerate(zip(series, labels)):
        c = _COLORS[k % len(_COLORS)]
        pts = [(px(x), py(y)) for x, y in zip(sx, sy) if (not logy or y > 0) and y0 <= tr(y) <= y1]
        if points:
            out += [f'<circle cx="{a:.1f}" cy="{b:.1f}" r="2" fill="{c}"/>' for a, b in pts]
        elif pts:
            out.append(f'<polyline fill="none" stroke="{c}" stroke-width="1.5" points="' +
                       " ".join(f"{a:.1f},{b:.1f}" for a, b in pts) + '"/>')
        ly = H - B + 48 + 16 * k
        out.append(f'<rect x="{L}" y="{ly - 9}" width="12" height="4" fill="{c}"/><text x="{L + 18}" y="{ly}">{label}</text>')
    for h in hlines:
        if y0 <= tr(h) <= y1:
            out.append(f'<line x1="{L}" y1="{py(h):.1f}" x2="{W - R}" y2="{py(h):.1f}" stroke="red" stroke-dasharray="5,4"/>')
    out.append("</svg>")
    with open(path, "w") as fh:
        fh.write("\n".join(out))
    return True


def _mpl_chart(series, labels, path, xlabel, ylabel, logy=False, ymin=None, ymax=None, hlines=(), points=False):
    import matplotlib
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    for (sx, sy), label in zip(series, labels):
        if sx:
            plt.plot(sx, sy, "." if points else "-", label=label)
    plt.grid()
    if logy:
        plt.yscale("log")
    if ymax is not None:
        plt.ylim(top=ymax)
    if ymin is not None:
        plt.ylim(bottom=ymin)
    for h in hlines:
        plt.axhline(y=h, color="red", linestyle="--")
    plt.xlabel(xlabel)
    plt.ylabel(ylabel)
    if any(labels):
        plt.legend(loc="upper left", bbox_to_anchor=(0, -0.15), borderaxespad=0.0, ncol=max(math.ceil(len(series) / 12), 1))
    plt.savefig(path, bbox_inches="tight")
    plt.clf()
    return True


def have_matplotlib() -> bool:
    try:
        import matplotlib  # noqa: F401
        return True
    except ImportError:
        return False


def plot_all(runs: Sequence[Dict[str, list]], labels: Sequence[str], plot_dir: str = ".", plot_name: str = "training",
             min_loss=None, max_loss=None, skip_label=False) -> List[str]:
    """The eight comparison charts; returns the files written (``.png`` with matplotlib, else ``.svg``)."""
    os.makedirs(plot_dir, exist_ok=True)
    chart, ext = (_mpl_chart, "png") if have_matplotlib() else (_svg_chart, "svg")
    labels = ["" for _ in labels] if skip_label else list(labels)
    written = []

    def emit(suffix, xkey, ykey, xlabel, ylabel, **kw):
        xform = kw.pop("xform", lambda v: v)
        series = [([xform(x) for x in r[xkey]], list(r[ykey])) for r in runs]
        labs = kw.pop("labels", labels)
        path = os.path.join(plot_dir, f"{plot_name}_{suffix}.{ext}")
        if chart(series, labs, path, xlabel, ylabel, **kw):
            written.append(path)

    emit("loss-step", "step_id", "loss_value", "Train step id", "Loss", ymin=min_loss, ymax=max_loss)
    emit("loss-tokens", "tokens_processed", "loss_value", "Training Tokens (B)", "Loss", ymin=min_loss, ymax=max_loss,
         xform=lambda v: v / 1e9)
    if all(r["time_stamp"] and None not in r["time_stamp"] for r in runs if r["step_id"]):
        t0 = min(min(r["time_stamp"]) for r in runs if r["step_id"])
        hrs = [f"{l} ({(r['time_stamp'][-1] - r['time_stamp'][0]) / 3600:.2f} hr)" if l else l
               for l, r in zip(labels, runs) if r["step_id"]]
        nonempty = [r for r in runs if r["step_id"]]
        path = os.path.join(plot_dir, f"{plot_name}_loss-time.{ext}")
        if chart([([(t - t0) / 3600 for t in r["time_stamp"]], r["loss_value"]) for r in nonempty], hrs, path,
                 "Wall clock Time (hr)", "Loss", ymin=min_loss, ymax=max_loss):
            written.append(path)
    emit("gradnorm", "step_id", "grad_norm", "Step id", "Grad norm", logy=True)
    emit("gradnorm-tokens", "tokens_processed", "grad_norm", "Tokens processed", "Grad norm", logy=True)
    emit("lr", "step_id", "lr", "Step id", "LR", ymin=0)
    summ = [summarize(r) for r in runs]
    emit("tps", "step_id", "tokens_per_sec", "Step id", "Tokens/sec/GPU", points=True,
         labels=[f"{l} (Avg: {int(s.get('tokens_per_sec_per_gpu', -1))})" for l, s in zip(labels, summ)],
         hlines=[s["tokens_per_sec_per_gpu"] for s in summ if "tokens_per_sec_per_gpu" in s])
    emit("tflops", "step_id", "tflops", "Step id", "Tflops", points=True,
         labels=[f"{l} (Avg: {s.get('avg_tflops', 0):5.2f})" for l, s in zip(labels, summ)],
         hlines=[s["avg_tflops"] for s in summ if "avg_tflops" in s])
    return written


def experiment_logs(exp_name: str, exp_dump_dir: str = ".") -> List[str]:
    """Sorted ``*.txt`` logs of an experiment, looked up in the archive directory first."""
    for sub in ("pretrain_parallel_models_archive", "pretrain_parallel_models"):
        d = os.path.join(exp_dump_dir, sub, exp_name)
        if os.path.isdir(d):
            return sorted(os.path.join(d, f) for f in os.listdir(d) if f.endswith(".txt"))
    return []
