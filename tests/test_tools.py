"""Smoke runs of the command-line tools on the CPU (each through its ``main``)."""
import importlib.util
import json
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tool(rel):
    sys.path.insert(0, os.path.join(ROOT, "tools"))
    spec = importlib.util.spec_from_file_location("tool_" + rel.replace("/", "_").replace(".py", ""), os.path.join(ROOT, "tools", rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_predict_step_grid_and_infeasible_rows(capsys, tmp_path):
    out = tmp_path / "rows.json"
    assert tool("bench/predict_step.py").main(["--preset", "llama3:tiny", "--budget", "0.0001,0.02,1", "--top", "2", "--json", str(out)]) == 0
    rows = json.loads(out.read_text())
    assert "INFEASIBLE" in rows[0]["note"] and rows[1]["tok_s"] > 0 and rows[2]["fast_gib"] <= 1
    assert rows[1]["link_gb"] > 0 and rows[1]["link_pct"] > 0            # the tight budget streams through the host link
    assert "most expensive tasks" in capsys.readouterr().out


def test_export_then_trace_program(tmp_path, capsys):
    assert tool("export/export_program.py").main(["--preset", "llama3:tiny", "--fast-gib", "0.02", "--recompute", "--out", str(tmp_path)]) == 0
    for ext in ("program", "annotated", "webapp", "summary"):
        assert (tmp_path / f"llama3-tiny.{ext}.json").exists()
    assert tool("export/trace_program.py").main(["--program", str(tmp_path / "llama3-tiny.annotated.json"), "--kinds", "offload", "--intervals"]) == 0
    assert "outcome SUCCESS" in capsys.readouterr().out


def test_engine_gate_on_the_virtual_backend_matches_the_simulator(tmp_path):
    assert tool("verify/engine_gate.py").main(["--config", "mini", "--fast-gib", "0.05", "--backend", "fake", "--out", str(tmp_path)]) == 0
    s = json.loads((tmp_path / "engine_gate-mini.summary.json").read_text())
    assert s["peak_equal"] and abs(s["gap_pct"]) < 1e-6


def test_dispatch_floor_and_gap_census(capsys):
    assert tool("bench/dispatch_floor.py").main(["--backend", "fake", "--tasks", "200", "--repeat", "2"]) == 0
    assert "us/task" in capsys.readouterr().out
    assert tool("bench/gap_census.py").main(["--preset", "llama3:tiny", "--device", "cpu", "--steps", "2"]) == 0
    assert "compute intervals" in capsys.readouterr().out


def test_planners_match_the_exact_oracle_on_tiny_chains(capsys):
    assert tool("bench/pressurefit_exact_oracle.py").main(["--chains", "4", "--tasks", "6", "--tolerance", "0.05"]) == 0
    assert "worst excess" in capsys.readouterr().out
    # the span planners against the same exhaustive optimum: accounting and growth land within a few per cent of it, the
    # constructive one within 15 %
    assert tool("bench/pressurefit_exact_oracle.py").main(["--chains", "4", "--tasks", "6", "--tolerance", "0.05", "--policies", "max_reduce,min_grow"]) == 0
    assert tool("bench/pressurefit_exact_oracle.py").main(["--chains", "4", "--tasks", "6", "--tolerance", "0.15", "--policies", "roundtrip"]) == 0


def test_verify_family_audit_and_listing(capsys):
    vf = tool("verify/verify_family.py")
    assert vf.main(["--list"]) == 0
    assert "llama3" in capsys.readouterr().out
    assert vf.main(["--family", "llama3", "--audit-only"]) == 0
    assert vf.audit("no_such_family")


def test_pressure_correctness_is_exact_on_the_host_backend():
    assert tool("verify/pressure_correctness.py").main(["--budgets", "0.02", "--steps", "2"]) == 0


def test_fetch_dataset_writes_shards_the_source_reads(tmp_path):
    (tmp_path / "a.txt").write_text("first document\n\nsecond document, longer\n\nthird\n")
    out = tmp_path / "ds"
    assert tool("train/fetch_dataset.py").main(["--inputs", str(tmp_path / "*.txt"), "--out", str(out), "--split-paragraphs", "--val-fraction", "0.34"]) == 0
    meta = json.loads((out / "corpus.meta.json").read_text())
    assert meta["tokens"]["documents"] == 3 and meta["shards"] == {"train": 1, "val": 1}
    from dataflow_b200.data.sources.shards import read_shard
    ids = read_shard(str(out / "corpus_train_000000.bin"))
    assert bytes(int(x) for x in ids if x < 256).startswith(b"first document")


def test_doc_tools(capsys, tmp_path):
    assert tool("gen_model_docs/list_models.py").main([]) == 0
    assert "llama3_8b" in capsys.readouterr().out
    assert tool("gen_model_docs/list_kernels.py").main(["--kernel-set", "eager"]) == 0
    assert tool("gen_model_docs/gen_model_docs.py").main(["--out", str(tmp_path)]) == 0
    assert (tmp_path / "index.md").exists() and "w_qkv" in (tmp_path / "llama3.md").read_text()


def test_reproducibility_drivers_run_staged_and_resume(tmp_path, capsys):
    spec = importlib.util.spec_from_file_location("run_accuracy", os.path.join(ROOT, "reproducibility", "accuracy_fidelity", "run_accuracy.py"))
    acc = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(acc)
    args = ["--preset", "llama3:tiny", "--device", "cpu", "--steps", "2", "--budgets", "0.02", "--out", str(tmp_path / "acc")]
    assert acc.main(args) == 0
    assert "budget GiB" in (tmp_path / "acc" / "report.md").read_text()
    assert acc.main(args + ["--resume"]) == 0
    assert "kept" in capsys.readouterr().out
    spec = importlib.util.spec_from_file_location("run_experiment", os.path.join(ROOT, "reproducibility", "throughput_fidelity", "run_experiment.py"))
    thr = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(thr)
    assert thr.main(["--preset", "llama3:tiny", "--device", "cpu", "--budgets", "0.02", "--steps", "4", "--out", str(tmp_path / "thr")]) == 0
    assert "measured / predicted" in (tmp_path / "thr" / "report.md").read_text()


def test_eval_checkpoint_reads_solo_and_sharded_checkpoints_alike(tmp_path, capsys):
    """The same training run as one process and as two FSDP ranks: both checkpoints load into the twin (weights only) and
    give the same held-out loss."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, os.path.join(root, "tools", "train", "train.py"), "train", "--preset", "llama3:tiny", "--steps", "2", "--device", "cpu",
            "--dtype-policy", "bf16_master", "--checkpoint-every", "2"]
    for name, extra in (("solo", ["--ga-rounds", "4"]), ("fsdp", ["--gpus", "2", "--parallel", "fsdp", "--ga-rounds", "2"])):
        r = subprocess.run(base + extra + ["--checkpoint-dir", str(tmp_path / name)], capture_output=True, text=True, timeout=600, cwd=root)
        assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2500:]
    got = {}
    for name in ("solo", "fsdp"):
        assert tool("train/eval_checkpoint.py").main(["--checkpoint", str(tmp_path / name / "step_000002"), "--preset", "llama3:tiny", "--steps", "2"]) == 0
        got[name] = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert got["solo"]["tokens"] == got["fsdp"]["tokens"] > 0 and got["solo"]["checkpoint"] == 2
    assert got["fsdp"]["loss"] == pytest.approx(got["solo"]["loss"], rel=2e-3) and 1.0 < got["solo"]["loss"] < 8.0


def test_planner_quality_gate_quick_corpus_holds_its_baseline(capsys):
    """The quick corpus of the planner quality gate (12 scenarios of the workload library, every registered policy): no plan
    over its cap, and the training entry's planner (the better of Lookahead and PressureFit) is no worse than recorded."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tools", "bench", "planner_quality_gate.py")
    spec = importlib.util.spec_from_file_location("planner_quality_gate", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.main(["--quick", "--check"]) == 0
    out = capsys.readouterr().out
    assert "12 scenarios" in out and "REGRESSION" not in out


def test_pretrain_report_tables_figures_and_band(tmp_path, capsys):
    import math
    import re
    import xml.dom.minidom
    rep = tool("train/pretrain_report.py")

    def run(name, wobble, n=40, nan_at=None):
        losses = [6 * math.exp(-i / 25) + 1 + wobble * ((i * 7919) % 13) / 13 for i in range(n)]
        if nan_at is not None:
            losses[nan_at] = float("nan")
        p = tmp_path / name
        p.write_text(json.dumps({"losses": losses, "step_wall_s": [0.5 + (3.0 if i == 0 else 0.0) + 0.001 * (i % 5) for i in range(n)],
                                 "tokens_per_step": 4096, "meta": {"preset": "tiny", "world": 2, "policy": "lookahead:cost_aware"}}))
        return str(p)
    a, b, c = run("a.json", 0.01), run("b.json", 0.012), run("c.json", 0.9)
    (tmp_path / "ev.jsonl").write_text(json.dumps({"checkpoint": 20, "loss": 3.9}) + "\nnot json\n")
    page = tmp_path / "r.html"
    assert rep.main([a, b, "--html", str(page), "--band", "0.05", "--evals", str(tmp_path / "ev.jsonl")]) == 0
    out = capsys.readouterr().out
    assert "band 5.0 %" in out and "inside" in out and "a.json" in out
    text = page.read_text()
    svgs = re.findall(r"<svg.*?</svg>", text, flags=re.S)
    assert len(svgs) == 3
    for s in svgs:
        xml.dom.minidom.parseString(s)
    assert "slowest steps: step 1" in text and "lookahead:cost_aware" in text and "<circle" in svgs[0]       # the warm-up step, the held-out point
    assert rep.main([a, c, "--band", "0.05"]) == 1 and "outside from step" in capsys.readouterr().out            # a curve that leaves the band fails
    r = rep.load_run(run("n.json", 0.0, nan_at=5), 3)
    assert r["non_finite"] == 1 and r["tok_s"] == pytest.approx(4096 / r["s_step_p50"])
    assert rep.band_report({"losses": []}, {"losses": [1.0]}, 0.1) == {"steps": 0}
