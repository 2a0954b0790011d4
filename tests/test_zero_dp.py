"""ZeRO data parallelism: CPU ranks over gloo exercise the host logic (lowering, slicing, init,
collective lane); on GPUs the fused peer-memory kernels are compared against the collective lane."""
import dataclasses
import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def launch(mode, world, device_kind, tmp_path, lane=None, port=29611):
    out = tmp_path / f"{mode}_{device_kind}_{lane}.json"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    if lane:
        env["DATAFLOW_DP_LANE"] = lane
    else:
        env.pop("DATAFLOW_DP_LANE", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_worker_zero.py"),
           mode, str(out), device_kind]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads(out.read_text())


def solo_reference_losses():
    """Single process, both ranks' data in one step: the math ZeRO must reproduce."""
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    fam = resolve_family("llama3")
    base = dataclasses.replace(fam.presets["tiny"](), dtype_policy="bf16_master")
    cfg = dataclasses.replace(base, grad_accum_rounds=base.grad_accum_rounds * 2)
    tr = Trainer("llama3", cfg, budget_gib=None, device=None, hyper={"lr": 2e-3, "weight_decay": 0.1}, seed=5, recompute=False)
    losses = []
    for s in range(4):
        data = []
        for rank in range(2):
            data += synthetic_rounds(base, base.grad_accum_rounds, tr.T, 64, 100 + rank, s)
        losses.append(tr.step(data))
    tr.close()
    return losses


@pytest.mark.parametrize("mode", ["zero3", "zero1", "fsdp"])
def test_zero_on_cpu_ranks_matches_single_process(mode, tmp_path):
    got = launch(mode, 2, "cpu", tmp_path, port={"zero3": 29611, "zero1": 29613, "fsdp": 29615}[mode])
    ref = solo_reference_losses()
    for a, b in zip(got["losses"], ref):
        assert a == pytest.approx(b, rel=2e-3)
    assert got["losses"][-1] < got["losses"][0]


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("mode", ["zero3", "zero1", "fsdp"])
def test_fused_p2p_kernels_match_collective_lane(mode, tmp_path):
    p2p = launch(mode, 2, "cuda", tmp_path, lane="p2p", port=29621)
    col = launch(mode, 2, "cuda", tmp_path, lane="collective", port=29623)
    for a, b in zip(p2p["losses"], col["losses"]):
        assert a == pytest.approx(b, rel=2e-3)
    assert p2p["w0_abs"] == pytest.approx(col["w0_abs"], rel=1e-4)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_published_buffers_outside_the_slab_go_through_the_staging_tail(tmp_path, monkeypatch):
    """A gradient or parameter slice that overflowed the engine slab is not mapped by the peers: the group copies it
    into the staging behind the slab first.  Forced here for every publish; results must not change."""
    col = launch("fsdp", 2, "cuda", tmp_path, lane="collective", port=29627)
    monkeypatch.setenv("ZERO_TEST_FORCE_STAGE", "1")
    p2p = launch("fsdp", 2, "cuda", tmp_path, lane="p2p", port=29625)
    for a, b in zip(p2p["losses"], col["losses"]):
        assert a == pytest.approx(b, rel=2e-3)
    assert p2p["w0_abs"] == pytest.approx(col["w0_abs"], rel=1e-4)


def test_sharded_modes_refuse_fp32_parameter_policies():
    """The sharded lanes slice packed objects as bf16 elements: an fp32 parameter policy is refused by name, not mis-read."""
    import dataclasses
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.parallel.zero import zero_lower_kwargs
    from dataflow_b200.run.driver import Trainer
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32")
    with pytest.raises(ValueError, match="needs bf16 parameters"):
        Trainer("llama3", cfg, budget_gib=None, device=None, lower_kwargs=zero_lower_kwargs("fsdp", 0, 2), init=False)
