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
