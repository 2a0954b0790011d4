"""Flags of `tools/train/train.py train` that shape a run without changing its numbers: the profile window and its trace
files, the pinned-memory budget, the backend choice, the reference's `--tp-mlp` spelling."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRAIN = os.path.join(ROOT, "tools", "train", "train.py")


def _run(*args, timeout=600):
    return subprocess.run([sys.executable, TRAIN, "train", "--preset", "llama3:tiny", "--device", "cpu", "--dtype-policy", "fp32", *args],
                          capture_output=True, text=True, timeout=timeout, cwd=ROOT)


def test_profile_window_writes_one_trace_per_step_and_leaves_losses_alone(tmp_path):
    plain, win = tmp_path / "plain.json", tmp_path / "win.json"
    prof = tmp_path / "prof"
    assert _run("--steps", "4", "--out", str(plain)).returncode == 0
    r = _run("--steps", "4", "--out", str(win), "--prof-dir", str(prof), "--profile-start-before-step", "2",
             "--profile-stop-after-step", "3")
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    a, b = json.loads(plain.read_text()), json.loads(win.read_text())
    # two processes: the host BLAS may split its sums differently when the machine is loaded, hence approx
    assert a["losses"] == pytest.approx(b["losses"], rel=1e-5)
    files = sorted(os.listdir(prof))
    assert files == ["step_000002.rank0.json", "step_000003.rank0.json"]
    assert [os.path.basename(p) for p in b["meta"]["traces"]] == files
    t = json.loads((prof / files[0]).read_text())
    assert t["step"] == 2 and t["measured_makespan_us"] > 0 and t["summary"]["by_key_ms"]
    names = {iv["name"] for iv in t["trace"]["intervals"]} if "intervals" in t["trace"] else set(map(str, t["trace"]))
    assert names


def test_backing_budget_refuses_a_run_that_needs_more_pinned_memory(tmp_path):
    r = _run("--steps", "1", "--backing-budget", "0.0001")
    assert r.returncode != 0 and "--backing-budget" in (r.stderr + r.stdout)
    assert _run("--steps", "1", "--backing-budget", "4").returncode == 0


def test_backend_and_tp_mlp_spellings(tmp_path):
    out = tmp_path / "tp.json"
    r = _run("--steps", "2", "--gpus", "2", "--tp-mlp", "--backend", "nccl", "--out", str(out))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    res = json.loads(out.read_text())
    assert res["meta"]["world"] == 2 and res["meta"]["family"] == "tp_mlp"
    assert _run("--steps", "1", "--backend", "smoke-signals").returncode != 0


def test_profile_window_object_brackets_exactly_its_steps():
    from dataflow_b200.run.profiling import ProfileWindow
    assert not ProfileWindow(None, 0, 0)
    w = ProfileWindow(None, 3, 0)                       # a stop of 0 means a one-step window

    class T:
        device = None
    for s in range(1, 6):
        w.before(s, T)
        seen = w.active
        w.after(s, T)
        assert seen == (s == 3)
    assert not w.active


def test_topology_group_names_world_and_devices(tmp_path):
    sys.path.insert(0, os.path.join(ROOT, "tools", "train"))
    try:
        import train as cli
    finally:
        sys.path.pop(0)
    topo = tmp_path / "box.toml"
    topo.write_text('[hosts.box]\ndevices = [0, 1, 2, 3]\n[groups.pair]\nmembers = ["box:2", "box:3"]\nbackend = "nccl"\n'
                    '[groups.all]\nmembers = ["box:0", "box:1", "box:2", "box:3"]\n')
    assert cli.ranks_from_topology(str(topo), "pair") == (2, [2, 3], "nccl")
    assert cli.ranks_from_topology(str(topo), "all")[0] == 4
    far = tmp_path / "far.toml"
    far.write_text('[hosts.box]\ndevices = [0]\n[hosts.far]\naddress = "me@far"\ndevices = [0]\n[groups.g]\nmembers = ["box:0", "far:0"]\n')
    with pytest.raises(SystemExit, match="one box"):
        cli.ranks_from_topology(str(far), None)
    out = tmp_path / "r.json"
    r = _run("--steps", "2", "--topology", str(topo), "--group", "pair", "--parallel", "co", "--out", str(out))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    assert json.loads(out.read_text())["meta"]["world"] == 2


def test_checkpoint_redundancy_limits_who_writes_replicas_and_resume_still_works(tmp_path):
    base = ["--steps", "4", "--gpus", "2", "--parallel", "co", "--ga-rounds", "1", "--checkpoint-dir"]
    sizes = {}
    for red in (None, 1):
        ck = tmp_path / f"ck{red}"
        extra = ["--checkpoint-redundancy", str(red)] if red else []
        a = _run(*base, str(ck), "--checkpoint-every", "2", "--out", str(tmp_path / f"a{red}.json"), *extra)
        assert a.returncode == 0, a.stdout[-1500:] + a.stderr[-2500:]
        rec = json.loads((ck / "step_000002" / "checkpoint_record.json").read_text())
        assert rec["scheme"]["replica_copies"] == (red or 2)
        copies = [len(v) for k, v in rec["slices"].items() if k.startswith("W_")]
        assert copies and set(copies) == {red or 2}
        sizes[red] = sum(os.path.getsize(os.path.join(d, f)) for d, _, fs in os.walk(ck / "step_000002" / "rank1") for f in fs)
        b = _run(*base, str(ck), "--resume", str(ck / "step_000002"), "--out", str(tmp_path / f"b{red}.json"))
        assert b.returncode == 0, b.stdout[-1500:] + b.stderr[-2500:]
        assert json.loads((tmp_path / f"a{red}.json").read_text())["losses"] == json.loads((tmp_path / f"b{red}.json").read_text())["losses"]
    assert sizes[1] < 0.2 * sizes[None]                 # rank 1 wrote (almost) nothing


def test_warm_profiles_prices_the_tasks_and_stops(tmp_path):
    out = tmp_path / "never.json"
    r = _run("--steps", "3", "--warm-profiles", "--out", str(out))
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    assert "--warm-profiles stops here" in r.stdout and "no steps ran" in r.stdout and "step     1" not in r.stdout


def test_task_profiles_soak_first_and_cache_under_their_own_key(tmp_path, monkeypatch):
    """``soak_seconds`` runs unsampled steps until the time is up before the steps that count (a power-capped device settles
    below its first burst); a soaked or contended measurement never overwrites the plain one in the cache."""
    import dataclasses
    import time
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import Trainer
    from dataflow_b200.run.profiling import PcieContender, profile_program
    monkeypatch.setenv("DATAFLOW_PROFILE_CACHE", str(tmp_path))
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32")
    tr = Trainer("llama3", cfg, budget_gib=None, device=None, hyper={"lr": 1e-3}, seed=0)
    try:
        plain = profile_program(tr)
        t0 = time.perf_counter()
        soaked = profile_program(tr, soak_seconds=0.5)
        assert time.perf_counter() - t0 >= 1.5                     # three cuts, half a second of settling each
        assert set(soaked) == set(plain) and all(v > 0 for v in soaked.values())
        names = sorted(p.name for p in tmp_path.iterdir())
        assert len(names) == 2 and any("-soak0.5" in n for n in names)
        with PcieContender(None) as c:                             # no device: nothing to contend with
            assert c.copies == 0
    finally:
        tr.close()


def test_user_mistakes_end_in_one_line_not_a_traceback(capsys):
    """An unknown preset, optimizer or data scheme, a flag below its minimum, a budget nothing fits: exit code 2 and one line
    that says what to fix."""
    import importlib.util
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("train_tool", os.path.join(root, "tools", "train", "train.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    base = ["train", "--steps", "1", "--device", "cpu"]
    for extra, needle in ((["--preset", "nope"], "unknown preset 'nope'"),
                          (["--preset", "llama3:tiny", "--data", "nosuch:thing"], "unknown data scheme 'nosuch'"),
                          (["--preset", "llama3:tiny", "--fast-budget", "0.0001"], "fits the budget"),
                          (["--preset", "llama3:tiny", "--resume", "/nonexistent/dir"], "no complete checkpoint")):
        assert tool.main(base + extra) == 2
        err = capsys.readouterr().err
        assert needle in err and "Traceback" not in err, err
    for extra, needle in ((["--preset", "llama3:tiny", "--opt", "lion"], "unknown optimizer"), (["--preset", "llama3:tiny", "--batch", "0"], "must be at least 1"),
                          (["--preset", "llama3:tiny", "--ga-rounds", "0"], "must be at least 1")):
        with pytest.raises(SystemExit) as e:
            tool.main(base + extra)
        assert e.value.code == 2 and needle in capsys.readouterr().err
