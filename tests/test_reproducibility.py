"""The fidelity studies: stage logic on synthetic rows, the pure parts of the diagnostics, and the drivers end to end on the
CPU backend."""
import importlib.util
import json
import os
import sys
import xml.dom.minidom

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
THR = os.path.join(ROOT, "reproducibility", "throughput_fidelity")
sys.path.insert(0, THR)
sys.path.insert(0, os.path.join(THR, "diagnostics"))

from stages.analyze import analyze, regime                     # noqa: E402
from stages.common import append_jsonl, geomean, quantile, read_jsonl, stage   # noqa: E402
from stages.make_plots import make_plots                        # noqa: E402
from stages.report import report_html, report_md                # noqa: E402
from stages.select_cells import select_cells                    # noqa: E402
from stages.sweep import sweep                                  # noqa: E402


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def rows(n_geo=2, budgets=(20, 40, 60, 80, 100)):
    pred, meas = [], []
    for g in range(n_geo):
        for b in budgets:
            i = len(pred)
            link = max(0.0, 95.0 - b)                                   # small budgets are link-bound
            pred.append({"opt": "adamw", "seq": 1024 * (g + 1), "t_round": 16384, "rounds": 2, "budget": b, "s_step": 10.0 / (1 + b / 50),
                         "link_pct": link, "recomp_pct": 20.0 if b == 40 else 0.0})
            ratio = 1.0 + (0.3 if b == 20 else 0.02 * g)
            meas.append({"cell": i, "opt": "adamw", "seq": 1024 * (g + 1), "t_round": 16384, "rounds": 2, "budget": b, "pred_s": pred[-1]["s_step"],
                         "meas_s": pred[-1]["s_step"] * ratio, "ratio": ratio, "tok_s": 32768 / (pred[-1]["s_step"] * ratio), "recomp_pct": pred[-1]["recomp_pct"],
                         "replay_gap_pct": 25.0 if b == 20 else 1.0, "overflows": 3 if b == 20 and g == 0 else 0,
                         "clocks": {"sm_mhz": 1300, "reasons": ["sw_power_cap"] + (["hw_slowdown"] if b == 20 and g == 1 else [])}})
    pred.append({"opt": "adamw", "seq": 8192, "t_round": 16384, "rounds": 2, "budget": 5, "note": "INFEASIBLE"})
    return pred, meas


def test_selection_covers_every_geometry_and_both_ends_of_the_budget_axis():
    pred, _ = rows()
    assert select_cells(pred, 50) == list(range(10))                        # fewer feasible cells than the target: all of them
    pick = select_cells(pred, 6)
    assert len(pick) == 6 and 10 not in pick                                # the infeasible cell is never picked
    for g in range(2):
        mine = [i for i in pick if pred[i]["seq"] == 1024 * (g + 1)]
        budgets = [pred[i]["budget"] for i in mine]
        assert len(mine) == 3 and min(budgets) == 20 and max(budgets) == 100        # lowest and highest budget of every geometry


def test_analysis_splits_by_axis_and_names_causes():
    pred, meas = rows()
    meas.append({"cell": 3, "opt": "adamw", "budget": 80, "seq": 1024, "error": "RuntimeError: boom"})
    a = analyze(pred, meas)
    assert a["cells"] == 10 and a["failed"] == 1 and a["worst"]["ratio"] == pytest.approx(1.3)
    assert a["within_10pct"] == pytest.approx(0.8) and 1.0 < a["geomean_ratio"] < 1.1
    assert set(a["by_axis"]["budget_third"]) == {"low", "mid", "high"} and a["by_axis"]["budget_third"]["low"]["geomean_ratio"] > a["by_axis"]["budget_third"]["high"]["geomean_ratio"]
    assert set(a["by_axis"]["regime"]) == {"link-bound", "recompute-heavy", "compute-bound"}
    off = {o["cell"]: o["why"] for o in a["off_by_more_than_10pct"]}
    assert set(off) == {0, 5}
    assert "scheduling loss 25.0 %" in off[0] and "task pricing +5.0 %" in off[0] and "3 allocator overflows" in off[0]
    assert "device throttled: sw_power_cap, hw_slowdown" in off[5]
    assert regime({"link_pct": 80}) == "link-bound" and regime({"recomp_pct": 30}) == "recompute-heavy" and regime({}) == "compute-bound"
    assert analyze(pred, [meas[-1]]) == {"cells": 0, "failed": 1, "errors": ["RuntimeError: boom"]}


def test_plots_are_well_formed_svg_and_the_report_carries_them():
    pred, meas = rows()
    plots = make_plots(meas)
    assert set(plots) == {"pred_vs_meas.svg", "ratio_by_budget.svg", "throughput_by_budget.svg"}
    for name, svg in plots.items():
        doc = xml.dom.minidom.parseString(svg)                              # parses: every tag closed, every attribute quoted
        assert doc.documentElement.tagName == "svg" and len(doc.getElementsByTagName("circle")) == 10, name
    md = report_md("llama3_8b", {"device": "B200", "torch": "2", "python": "3", "copy_gbs": 6000.0}, pred, meas, analyze(pred, meas))
    assert "geometric mean measured / predicted" in md and "By budget third:" in md and "Cells off by more than 10 %" in md and "1 predicted cells had no plan" in md
    page = report_html(md, plots)
    assert page.count("<svg") == 3 and page.count("<table>") == page.count("</table>") >= 3
    assert make_plots([{"error": "x"}]) == {}


def test_stage_files_resume_and_a_killed_sweep_keeps_its_rows(tmp_path, capsys):
    out = str(tmp_path)
    calls = []
    assert stage(out, "s", False, lambda: calls.append(1) or {"v": 1}) == {"v": 1}
    assert stage(out, "s", True, lambda: calls.append(1) or {"v": 2}) == {"v": 1} and len(calls) == 1       # kept, not recomputed
    assert stage(out, "s", False, lambda: {"v": 3}) == {"v": 3}
    path = os.path.join(out, "m.jsonl")
    append_jsonl(path, {"a": 1})
    with open(path, "a") as f:
        f.write('{"a": 2')                                                   # a line cut short by a kill
    assert read_jsonl(path) == [{"a": 1}]
    assert geomean([1, 4]) == pytest.approx(2.0) and quantile([1, 2, 3, 4, 5], 0.5) == 3 and quantile([1, 2], 0.5) == 1.5

    class Cfg:
        seq_len = 128
    measured = []

    def one(fam, cfg, budget):
        measured.append(budget)
        if budget == 2:
            raise RuntimeError("no room")
        return {"ratio": 1.0 + budget / 100, "budget": budget}
    cells = [("adamw", ("f", Cfg(), b)) for b in (1, 2, 3)]
    got = sweep(out, cells, [0, 1, 2], one, resume=False)
    assert [("ratio" in r, "error" in r) for r in got] == [(True, False), (False, True), (True, False)]
    again = sweep(out, cells, [0, 1, 2], one, resume=True)                   # only the failed cell is measured again
    assert measured == [1, 2, 3, 2] and [r["cell"] for r in again] == [0, 1, 2]


def test_diagnostics_pure_parts(tmp_path):
    import pcie_calib
    import throttle_probe
    from task_cost_audit import kind_of
    f = pcie_calib.fit([(n, 15e-6 + n / 48e9) for n in (1 << 20, 1 << 24, 1 << 28)])
    assert f["gbs"] == pytest.approx(48.0, rel=1e-6) and f["latency_us"] == pytest.approx(15.0, rel=1e-3)
    assert pcie_calib.main(["--device", "cpu"]) == 0
    csv = tmp_path / "clocks.csv"
    head = "index, clocks.sm [MHz], clocks.max.sm [MHz], power.draw [W], clocks_event_reasons.active, clocks_event_reasons.hw_slowdown, " \
           "clocks_event_reasons.hw_thermal_slowdown, clocks_event_reasons.sw_thermal_slowdown, clocks_event_reasons.sw_power_cap\n"
    csv.write_text(head + "0, 1305 MHz, 1965 MHz, 990 W, 0x4, Not Active, Not Active, Not Active, Active\n" * 3)
    v = throttle_probe.from_csv(str(csv))
    assert v["ok"] and v["sm_mhz_median"] == 1305 and v["reasons"] == ["sw_power_cap"]
    csv.write_text(head + "0, 1305 MHz, 1965 MHz, 990 W, 0x8, Active, Not Active, Not Active, Not Active\n")
    assert not throttle_probe.from_csv(str(csv))["ok"]
    assert not throttle_probe.verdict([900, 905], 1965, set())["ok"] and throttle_probe.verdict([1900], 1965, set())["ok"]
    assert kind_of("block_bwd_0_1_12") == "block_bwd" and kind_of("optimizer_head_0") == "optimizer_head" and kind_of("head_loss_0_1") == "head_loss"


def test_overlap_report_accounts_for_every_microsecond():
    from trace_overlap import overlap_report
    from dataflow_b200.runtime.trace import Interval

    class T:
        intervals = [Interval("a", "compute", 0, 10), Interval("b", "compute", 15, 25), Interval("x", "from_slow", 5, 18),
                     Interval("y", "to_slow", 8, 12), Interval("z", "to_slow", 26, 30)]

        def by_track(self, tr):
            return [i for i in self.intervals if i.track == tr]
    r = overlap_report(T())
    assert r["span_us"] == 30
    assert r["compute_and_copy_pct"] + r["compute_only_pct"] + r["copy_only_pct"] + r["nothing_pct"] == pytest.approx(100.0)
    assert r["compute_busy_pct"] == pytest.approx(100 * 20 / 30) and r["nothing_pct"] == pytest.approx(100 * 1 / 30)       # only [25, 26) is empty
    assert r["lanes"]["from_slow"]["hidden_under_compute_pct"] == pytest.approx(100 * 8 / 13)                               # [5,10) and [15,18)
    assert r["lanes"]["to_slow"]["hidden_under_compute_pct"] == pytest.approx(100 * 2 / 8) and r["both_directions_pct"] == pytest.approx(100 * 4 / 30)


def test_the_study_driver_runs_staged_and_resumes(tmp_path, capsys):
    thr = load(os.path.join(THR, "run_experiment.py"), "run_experiment")
    out = tmp_path / "thr"
    args = ["--preset", "llama3:tiny", "--device", "cpu", "--budgets", "0.02,1", "--steps", "4", "--out", str(out)]
    assert thr.main(args) == 0
    for name in ("env_probe.json", "predict.json", "select.json", "measure.jsonl", "analyze.json", "report.md", "report.html", "pred_vs_meas.svg"):
        assert (out / name).exists(), name
    assert "measured / predicted" in (out / "report.md").read_text()
    assert json.loads((out / "analyze.json").read_text())["cells"] == 2
    capsys.readouterr()
    assert thr.main(args + ["--resume"]) == 0
    text = capsys.readouterr().out
    assert "[predict] kept" in text and text.count("[measure] cell") == 2 and "kept" in text.split("[measure]")[1]


def test_a_cell_is_traced_and_analysed_and_dispatch_cost_is_measured(tmp_path, capsys):
    cell = load(os.path.join(THR, "trace_cell.py"), "trace_cell")
    assert cell.main(["--preset", "llama3:tiny", "--budget", "0.02", "--device", "cpu", "--steps", "2", "--out", str(tmp_path), "--name", "c"]) == 0
    ana = json.loads((tmp_path / "c.analysis.json").read_text())
    assert ana["ratio"] > 0 and ana["task_costs"]["kinds"][0]["share_of_mispricing_pct"] > 0 and "idle_pct" in ana["gaps"]
    o = ana["overlap"]
    assert o["compute_and_copy_pct"] + o["compute_only_pct"] + o["copy_only_pct"] + o["nothing_pct"] == pytest.approx(100.0)
    measured = json.loads((tmp_path / "c.measured.json").read_text())
    assert measured["trace"]["intervals"] and measured["measured_makespan_us"] == ana["measured_makespan_us"]
    assert json.loads((tmp_path / "c.chrome.json").read_text())["traceEvents"][0]["ph"] == "X"
    disp = load(os.path.join(THR, "dispatch_cost.py"), "dispatch_cost")
    capsys.readouterr()
    assert disp.main(["--device", "fake", "--tasks", "60", "--reps", "2"]) == 0
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["us_per_task"] > 0 and res["us_per_task_with_round_trip"] > res["us_per_task"] * 0.8


def test_the_accuracy_driver_reports_curves_and_weights(tmp_path):
    acc = load(os.path.join(ROOT, "reproducibility", "accuracy_fidelity", "run_accuracy.py"), "run_accuracy")
    out = tmp_path / "acc"
    assert acc.main(["--preset", "llama3:tiny", "--device", "cpu", "--steps", "2", "--budgets", "0.02", "--out", str(out)]) == 0
    md = (out / "report.md").read_text()
    assert "final weights: max rel. L2 to the twin" in md and "| 0.02 |" in md
    curves = json.loads((out / "curves.json").read_text())
    assert set(curves) == {"twin", "unconstrained", "0.02 GiB"} and curves["0.02 GiB"] == curves["unconstrained"]
    assert xml.dom.minidom.parseString((out / "curves.svg").read_text()).getElementsByTagName("polyline").length == 3
