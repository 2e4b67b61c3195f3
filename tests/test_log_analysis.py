"""Log parsing, run comparison and chart writing against a log written in the driver's line format."""
import json
import os

import compare_losses
from optimus_lm_b200 import log_analysis as la

LINE = ("Step {s:4d} / 100, Loss : {loss:9.6f}, Grad norm : {gn:.6f}, LR : {lr:.8f}, Time : 0.2500 sec, DL time : 0.0010 sec, "
        "Tokens Processed : {tok}, Tokens/sec : 65536, Timestamp : {ts}, Tflops : 410.25, ETA : 0.01 hr, "
        "Local Loss : {loss:9.6f}, Local Grad norm :  1.000000, Rank : 0 (0,0,0,0)\n")


def _write(path, n, bias=0.0, start=0):
    with open(path, "w") as fh:
        fh.write("WORLD_SIZE = 8\nsome unrelated line\n")
        for s in range(start, start + n):
            fh.write(LINE.format(s=s, loss=11.0 - 0.01 * s + bias, gn=2.0 + 0.1 * s, lr=4e-5 + 1e-7 * s,
                                 tok=(s + 1) * 131072, ts=1700000000.0 + 0.25 * s))


def test_parse_filter_summarize_compare(tmp_path):
    a, b = str(tmp_path / "log_1_a.txt"), str(tmp_path / "log_2_b.txt")
    _write(a, 20)
    _write(b, 20, bias=0.002)
    da, db = la.parse_log(a), la.parse_log(b)
    assert da["step_id"] == list(range(20)) and da["world_size"][0] == 8
    assert abs(da["loss_value"][3] - 10.97) < 1e-9 and da["tokens_per_sec"][0] == 65536 and da["tflops"][0] == 410.25
    f = la.filter_series(da, start_step=5, end_step=9)
    assert f["step_id"] == [5, 6, 7, 8, 9]
    s = la.summarize(da)
    assert s["steps"] == 20 and abs(s["tokens_per_sec_per_gpu"] - (19 * 131072 / (19 * 0.25)) / 8) < 1e-6
    c = la.compare_series(da, db)
    assert c["common_steps"] == 20 and abs(c["max_abs_diff_loss_value"] - 0.002) < 1e-9 and c["max_abs_diff_grad_norm"] == 0
    # a resumed run: second log continues (and overlaps) the first
    r = str(tmp_path / "log_3_resume.txt")
    _write(r, 10, start=15)
    m = la.merge_logs([a, r])
    assert m["step_id"] == list(range(25))


def test_compare_losses_cli_writes_charts(tmp_path, capsys):
    exp = tmp_path / "pretrain_parallel_models"
    for name, bias in (("runA_temp", 0.0), ("runB_temp", 0.5)):
        os.makedirs(exp / name)
        _write(str(exp / name / "log_0_20250101_000000.txt"), 12, bias=bias)
    cfg = {"analysis_choice": 0, "analysis0": {"exp_info_list": [["runA_temp", "A"], ["runB_temp"]],
                                               "plot_dir": str(tmp_path / "plots"), "max_loss": 12.0}}
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(cfg))
    assert compare_losses.main(["--config_path", str(cfg_path), "--exp_dump_dir", str(tmp_path)]) == 0
    out = capsys.readouterr().out
    assert "A vs runB_temp" in out and "'max_abs_diff_loss_value': 0.5" in out
    plots = sorted(os.listdir(tmp_path / "plots"))
    assert len(plots) == 8 and any(p.startswith("training_loss-step.") for p in plots)
    assert os.path.getsize(tmp_path / "plots" / plots[0]) > 500
    # empty experiment list: the temporary experiments are listed
    cfg["analysis0"]["exp_info_list"] = []
    cfg_path.write_text(json.dumps(cfg))
    assert compare_losses.main(["--config_path", str(cfg_path), "--exp_dump_dir", str(tmp_path)]) == 0
    assert '["runA_temp"]' in capsys.readouterr().out
