"""Expert parallelism: the fused dispatch / combine kernels and their collective-lane oracle against a dense fp32
layer over all experts and all ranks' tokens."""
import json
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def launch(world, device_kind, tmp_path, lane=None, port=29711):
    out = tmp_path / f"ep_{device_kind}_{lane}.json"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    if lane:
        env["DATAFLOW_EP_LANE"] = lane
    else:
        env.pop("DATAFLOW_EP_LANE", None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dist_worker_ep.py"), str(out), device_kind]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return json.loads(out.read_text())


def test_plan_tables_are_consistent_single_rank():
    from dataflow_b200.parallel.ep import EpGroup
    g = EpGroup(0, 1, None, tokens=40, d_model=16, n_experts=4, top_k=2)
    gen = torch.Generator().manual_seed(0)
    ids = torch.stack([torch.randperm(4, generator=gen)[:2] for _ in range(40)]).to(torch.int32)
    w = torch.rand(40, 2, generator=gen)
    plan = g.plan(ids, w)
    table = plan._table
    assert int(plan.dropped) == 0 and (table >= 0).all()
    # every slot's row holds its token, lies in its expert's padded range, and carries its weight
    rows = table.reshape(-1).long()
    assert len(set(rows.tolist())) == 80
    assert (plan.row_src[rows] == torch.arange(40).repeat_interleave(2)).all()
    e = ids.reshape(-1).long()
    assert ((rows >= plan.offsets_pad[e]) & (rows < plan.offsets_pad[e + 1])).all()
    assert torch.allclose(plan.row_w[rows], w.reshape(-1))
    assert (plan.row_w[plan.row_src < 0] == 0).all()
    assert plan.counts.sum() == 80


def test_capacity_drops_slots_past_the_dispatched_matrix():
    from dataflow_b200.parallel.ep import EpGroup
    g = EpGroup(0, 2, None, tokens=300, d_model=16, n_experts=2, top_k=1, capacity_factor=1.0)
    assert g.C == 768                             # 300 slots rounded up to tiles + one padding tile per local expert
    # one process plays the whole group (the gather is the identity): 1000 slots, all routed to this rank's expert
    g.world, g.T, g.slots_global = 1, 1000, 1000
    plan = g.plan(torch.zeros(1000, 1, dtype=torch.int32), torch.ones(1000, 1))
    assert int(plan.dropped) == 1000 - 768
    assert int((plan._table >= 0).sum()) == 768
    assert int(plan.offsets_pad[-1]) == 768 and (plan.tile_expert == 0).all()
    # a step that dropped slots fails at its end, with the count, unless drops are allowed; the counter restarts every step
    with pytest.raises(RuntimeError, match="dropped 232 token slots"):
        g.check()
    g.check()
    g.allow_drops = True
    g.plan(torch.zeros(1000, 1, dtype=torch.int32), torch.ones(1000, 1))
    g.check()
    assert g.dropped_total == 2 * 232


def test_ep_collective_lane_on_cpu_ranks_matches_dense_oracle(tmp_path):
    got = launch(2, "cpu", tmp_path, port=29713)
    assert got["dropped"] == 0
    for k, v in got["max_rel"].items():
        assert v < 2e-2, (k, v)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("lane", ["p2p", "collective"])
def test_ep_fused_kernels_match_dense_oracle(lane, tmp_path):
    got = launch(2, "cuda", tmp_path, lane=lane, port=29715 if lane == "p2p" else 29717)
    assert got["dropped"] == 0
    for k, v in got["max_rel"].items():
        assert v < 2e-2, (k, v)


def launch_family(world, device_kind, tmp_path, lane=None, port=29731, budget=None, family="olmoe"):
    out = tmp_path / f"epfam_{family}_{device_kind}_{lane}_{budget}.json"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", EP_TEST_FAMILY=family)
    env.pop("DATAFLOW_EP_LANE", None)
    env.pop("EP_TEST_BUDGET", None)
    if lane:
        env["DATAFLOW_EP_LANE"] = lane
    if budget:
        env["EP_TEST_BUDGET"] = str(budget)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "dist_worker_epfam.py"), str(out), device_kind]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if r.returncode:
        at = r.stderr.find("Traceback")
        raise AssertionError(r.stderr[at:at + 3000] if at >= 0 else r.stdout[-1500:] + r.stderr[-1500:])
    return json.loads(out.read_text())


def solo_olmoe_losses(family="olmoe"):
    """One process, all experts, both ranks' data in one step (twice the rounds): the math the EP run must reproduce."""
    import dataclasses
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    fam = resolve_family(family)
    base = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32")
    cfg = dataclasses.replace(base, grad_accum_rounds=base.grad_accum_rounds * 2)
    tr = Trainer(family, cfg, budget_gib=None, device=None, hyper={"lr": 2e-3, "weight_decay": 0.1}, seed=5, leeway_bytes=0)
    losses = []
    try:
        for s in range(3):
            data = []
            for rank in range(2):
                data += synthetic_rounds(base, base.grad_accum_rounds, tr.T, 64, 100 + rank, s)
            losses.append(tr.step(data))
    finally:
        tr.close()
    return losses


def test_olmoe_with_experts_split_over_two_cpu_ranks_matches_one_process(tmp_path):
    got = launch_family(2, "cpu", tmp_path, port=29733)
    ref = solo_olmoe_losses()
    for a, b in zip(got["losses"], ref):
        assert a == pytest.approx(b, rel=1e-3)
    assert got["losses"][-1] < got["losses"][0]


@pytest.mark.parametrize("family,port", [("dsv3", 29741), ("glm52", 29743), ("qwen35moe", 29745)])
def test_reference_form_families_with_experts_split_over_two_cpu_ranks_match_one_process(family, port, tmp_path):
    """Multi-head latent attention families (autograd lane): the routed experts go through the expert-parallel exchange
    as an autograd function; replicated fields' gradients are summed over the group."""
    got = launch_family(2, "cpu", tmp_path, port=port, family=family)
    ref = solo_olmoe_losses(family)
    for a, b in zip(got["losses"], ref):
        assert a == pytest.approx(b, rel=1e-3)
    assert got["losses"][-1] < got["losses"][0]


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_olmoe_expert_parallel_fused_lane_trains_like_the_collective_lane(tmp_path):
    p2p = launch_family(2, "cuda", tmp_path, lane="p2p", port=29735)
    col = launch_family(2, "cuda", tmp_path, lane="collective", port=29737)
    for a, b in zip(p2p["losses"], col["losses"]):
        assert a == pytest.approx(b, rel=2e-2)
    assert p2p["losses"][-1] < p2p["losses"][0]
