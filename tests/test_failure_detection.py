"""Failure detection without faulting a GPU: failures are made on the host (a rank raises or leaves between steps) and the
surviving ranks must notice within the process-group timeout and end with an error instead of hanging; on a device, a
kernel whose wait can never be satisfied must return a status and leave the context usable."""
import os
import subprocess
import sys
import time

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("kind", ["raise", "exit"])
def test_a_rank_that_fails_between_steps_ends_the_job_quickly(kind, tmp_path):
    env = dict(os.environ, DATAFLOW_FAULT_PLAN=f"rank=1,step=2,kind={kind}", DATAFLOW_PG_TIMEOUT_S="8", PYTHONPATH=ROOT)
    cmd = [sys.executable, os.path.join(ROOT, "tools", "train", "train.py"), "train", "--preset", "llama3:tiny", "--steps", "6", "--device", "cpu",
           "--gpus", "2", "--parallel", "co", "--dtype-policy", "fp32", "--out", str(tmp_path / "r.json")]
    t0 = time.time()
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT, env=env)
    took = time.time() - t0
    assert r.returncode != 0                                      # the job does not pretend to have succeeded
    assert not (tmp_path / "r.json").exists()
    assert took < 120                                             # and does not wait out a 30-minute default
    text = r.stdout + r.stderr
    assert "step     2" in text and "step     6" not in text
    if kind == "raise":
        assert "fault plan: rank 1 fails after step 2" in text


def test_a_failed_job_restarts_from_its_newest_checkpoint_and_finishes_the_same_curve(tmp_path):
    """`--max-restarts 1`: rank 1 dies after step 3 (once); the conductor relaunches the job from the checkpoint of step 2
    and the finished curve is the one an undisturbed run produces."""
    import json
    base = [sys.executable, os.path.join(ROOT, "tools", "train", "train.py"), "train", "--preset", "llama3:tiny", "--steps", "5", "--device", "cpu",
            "--gpus", "2", "--parallel", "co", "--dtype-policy", "fp32", "--checkpoint-every", "2"]
    calm = subprocess.run(base + ["--checkpoint-dir", str(tmp_path / "ck0"), "--out", str(tmp_path / "calm.json")], capture_output=True,
                          text=True, timeout=600, cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT))
    assert calm.returncode == 0, calm.stderr[-2000:]
    env = dict(os.environ, DATAFLOW_FAULT_PLAN=f"rank=1,step=3,kind=exit,once={tmp_path / 'fired'}", DATAFLOW_PG_TIMEOUT_S="8", PYTHONPATH=ROOT)
    r = subprocess.run(base + ["--checkpoint-dir", str(tmp_path / "ck1"), "--out", str(tmp_path / "hit.json"), "--max-restarts", "1"],
                       capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    assert (tmp_path / "fired").exists() and "restart 1 of 1" in r.stdout and "resumed from" in r.stdout
    hit, ref = json.loads((tmp_path / "hit.json").read_text()), json.loads((tmp_path / "calm.json").read_text())
    assert hit["meta"].get("restarts") == 1 and len(hit["losses"]) == 5
    assert hit["losses"] == pytest.approx(ref["losses"], rel=1e-5)
    # without the allowance the same fault ends the job
    os.remove(tmp_path / "fired")
    r2 = subprocess.run(base + ["--checkpoint-dir", str(tmp_path / "ck2"), "--out", str(tmp_path / "dead.json")], capture_output=True,
                        text=True, timeout=600, cwd=ROOT, env=env)
    assert r2.returncode != 0 and not (tmp_path / "dead.json").exists()


def test_only_host_side_failures_are_restarted(tmp_path, monkeypatch):
    """A rank's failure marker says whether the failure came from Python code, from a peer that timed out or from the device;
    the conductor relaunches for the first two and stops on the third."""
    import json
    from dataflow_b200.parallel.zero import CommTimeout
    from dataflow_b200.run import conductor
    from dataflow_b200.run.rank_main import failure_kind, failure_marker
    assert failure_kind(RuntimeError("fault plan: rank 1 fails after step 2")) == "host"
    assert failure_kind(CommTimeout("fused communication kernel gave up: phase 1, peer/rank 3")) == "timeout"
    assert failure_kind(RuntimeError("CUDA error: an illegal memory access was encountered")) == "device"
    assert failure_kind(RuntimeError("gemm_bf16: kernel gave up (error word 17)")) == "device"
    assert failure_kind(RuntimeError("[Rank 0] Watchdog caught collective operation timeout")) == "timeout"
    out = str(tmp_path / "r.json")
    calls = []

    class P:
        returncode = 1

    def fake_run(cmd, env=None):
        calls.append(cmd)
        with open(failure_marker(out, 1), "w") as f:
            json.dump({"kind": "device", "message": "CUDA error: an illegal memory access was encountered"}, f)
        return P()

    monkeypatch.setattr(conductor.subprocess, "run", fake_run)
    spec = conductor.RunSpec(preset="llama3:tiny", world=2, steps=2, out=out, max_restarts=3, checkpoint_dir=str(tmp_path / "ck"))
    with pytest.raises(RuntimeError, match="device error and is not restarted"):
        conductor.run(spec, log=lambda *_: None)
    assert len(calls) == 1


@pytest.mark.gpu
def test_a_device_wait_that_cannot_be_satisfied_returns_a_status_and_the_context_stays_usable():
    """The expert-parallel combine kernel of rank 0 of a 2-rank group whose peer never publishes its rows: the bounded wait
    gives up, the error word names the phase and the peer, and the next kernel on the same context runs normally."""
    import torch
    from dataflow_b200.ops import native
    n = native()
    dev = torch.device("cuda", 0)
    T, K, d, e_local = 64, 2, 128, 4
    rows = [torch.zeros(256, d, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    words = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]           # ready word at +0, ack counter at +16 ints
    ids = torch.full((T, K), e_local, dtype=torch.int32, device=dev)                     # every slot belongs to the (silent) peer
    rows_local = torch.zeros(T, K, dtype=torch.int32, device=dev)
    out = torch.empty(T, d, dtype=torch.bfloat16, device=dev)
    err = torch.zeros(1, dtype=torch.int32, device=dev)
    done = torch.zeros(1, dtype=torch.int32, device=dev)
    t0 = time.time()
    n.ep_combine([r.data_ptr() for r in rows], [], None, None, ids, rows_local, out, None, e_local, 0,
                 [w.data_ptr() for w in words], [w.data_ptr() + 64 for w in words], 1, 0.25, err, done)
    torch.cuda.synchronize()
    took = time.time() - t0
    code = int(err.item())
    assert code != 0 and (code >> 8) in (51, 52)                  # gave up waiting for the peer's rows / for its acknowledgement
    assert took < 5.0
    assert int(words[0][0]) == 1                                  # this rank had published its own rows
    # the context is alive: an ordinary kernel and a copy work
    x = torch.randn(1024, 1024, device=dev, dtype=torch.bfloat16)
    y = torch.empty_like(x)
    n.gemm_bf16(x, False, x, True, y, None, None)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all()
