"""Evaluation-result table and curves from harness-style JSON files."""
import json
import os

from optimus_lm_b200 import eval_results as er


def _result(dirpath, base):
    os.makedirs(os.path.join(dirpath, "nested__model__path"), exist_ok=True)
    res = {b: {m: base + 0.01 * i, "alias": b} for i, (b, m) in enumerate(er.BENCHMARK_METRIC.items())}
    with open(os.path.join(dirpath, "nested__model__path", "results_2025.json"), "w") as fh:
        json.dump({"results": res}, fh)


def test_table_and_curves(tmp_path):
    root = tmp_path / "results"
    for step, tok, base in ((1000, 6, 0.30), (20000, 126, 0.50), (5000, 31, 0.40)):
        _result(str(root / f"step{step}-tokens{tok}B"), base)
    _result(str(root / "main"), 0.55)
    table = er.latex_table([str(root / "step1000-tokens6B"), str(root / "main")])
    rows = table.splitlines()
    assert rows[0].startswith("arc_easy") and "30.0  & 55.0" in rows[0] and rows[-1].startswith("Average")
    assert "34.0  & 59.0" in rows[-1]
    curve = er.checkpoint_curve(str(root))
    assert list(curve) == ["step1000-tokens6B", "step5000-tokens31B", "step20000-tokens126B"]
    files = er.plot_curves([str(root)], ["run"], str(tmp_path / "plots"))
    assert len(files) == 10 and all(os.path.getsize(f) > 300 for f in files)
