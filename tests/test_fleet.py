"""Fleet mode: a conductor process drives one ``dataflowd`` daemon per rank over unix sockets; the daemons link into a peer
group and train in lock step.  Run here with two CPU daemons on the peer plane's host lane (no GPU, no NCCL): the loss curve
must be the one the process launcher (``torch.distributed.run``, gloo) produces for the same job, and the daemons must be
gone afterwards."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRAIN = os.path.join(ROOT, "tools", "train", "train.py")


def train(tmp_path, name, *extra):
    out = tmp_path / f"{name}.json"
    cmd = [sys.executable, TRAIN, "train", "--preset", "llama3:tiny", "--steps", "3", "--device", "cpu", "--gpus", "2",
           "--opt-shard", "co", "--dtype-policy", "fp32", "--out", str(out), *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=str(tmp_path), env=dict(os.environ, PYTHONPATH=ROOT))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return json.loads(out.read_text()), r.stdout


def test_two_daemons_train_the_same_curve_as_two_processes(tmp_path):
    fleet, log = train(tmp_path, "fleet", "--launcher", "fleet")
    assert "peer group dp ready" in log and "hostmem lane" in log
    proc, _ = train(tmp_path, "proc")
    assert len(fleet["losses"]) == 3
    assert fleet["losses"] == pytest.approx(proc["losses"], rel=1e-6)
    assert fleet["meta"]["launcher"] == "fleet" and fleet["meta"]["world"] == 2
    # no daemon of the run is left behind: their pidfiles name processes that have exited
    import glob
    import re
    m = re.search(r"socket (\S+)/dataflowd\.", log)
    assert m, log[-500:]
    for pidfile in glob.glob(os.path.join(m.group(1), "*.pid")):
        pid = int(open(pidfile).read().split()[0])
        assert not os.path.exists(f"/proc/{pid}") or open(f"/proc/{pid}/stat").read().split()[2] == "Z"


def test_fleet_mode_refuses_sharded_modes_by_name(tmp_path):
    cmd = [sys.executable, TRAIN, "train", "--preset", "llama3:tiny", "--steps", "1", "--device", "cpu", "--gpus", "2",
           "--opt-shard", "fsdp", "--launcher", "fleet", "--out", str(tmp_path / "x.json")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(tmp_path), env=dict(os.environ, PYTHONPATH=ROOT))
    assert r.returncode != 0 and "fleet mode runs replicas" in (r.stdout + r.stderr)


def test_timeline_wrap_and_profile_window(tmp_path):
    """The daemon launcher's profiler wrap is the capture-by-API command line, and a fleet run with a profile window opens and
    closes it through every daemon's ``profiler_control`` (no timeline profiler on this machine: NVTX ranges only)."""
    from dataflow_b200.distributed import daemons
    cmd = daemons.timeline_command("/opt/nsys/bin/nsys", "/tmp/out/timeline_rank0")
    assert cmd[:2] == ["/opt/nsys/bin/nsys", "profile"] and "--capture-range=cudaProfilerApi" in cmd and "--capture-range-end=stop" in cmd
    assert cmd[cmd.index("-o") + 1] == "/tmp/out/timeline_rank0"
    from dataflow_b200.run.conductor import RunSpec
    from dataflow_b200.run.fleet import run_fleet
    lines = []
    spec = RunSpec(preset="llama3:tiny", steps=3, device=None, world=2, parallel="co", launcher="fleet", overrides={"dtype_policy": "fp32"},
                   prof_dir=str(tmp_path / "prof"), profile_start_before_step=2, profile_stop_after_step=2)
    res = run_fleet(spec, log=lines.append)
    assert len(res.losses) == 3
    assert any("profile window steps 2..2" in l for l in lines)


def test_mixed_fleets_are_refused():
    from dataflow_b200 import code_revision
    from dataflow_b200.run.fleet import check_fleet_versions
    rev = code_revision()
    assert len(rev) == 16 and rev == code_revision()
    ok = {"rank0": {"code_rev": rev, "env": "torch 2 cuda 12"}, "rank1": {"code_rev": rev, "env": "torch 2 cuda 12"}}
    check_fleet_versions(ok, rev, "torch 2 cuda 12")
    with pytest.raises(RuntimeError, match="rank1 runs code deadbeef"):
        check_fleet_versions({**ok, "rank1": {"code_rev": "deadbeef", "env": "torch 2 cuda 12"}}, rev, "torch 2 cuda 12")
    with pytest.raises(RuntimeError, match="environment skew"):
        check_fleet_versions({**ok, "rank1": {"code_rev": rev, "env": "torch 3 cuda 13"}}, rev, "torch 2 cuda 12")
