"""Fused tensor-parallel kernels (all-gather -> GEMM, GEMM -> reduce-scatter) against library collectives around
fp32 matmuls, on 2 GPUs.  NVLS stays off: the kernels use plain peer loads / stores only."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_fused_tp_kernels_match_collectives(tmp_path):
    out = tmp_path / "tp.json"
    env = {**os.environ, "NCCL_NVLS_ENABLE": "0"}
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29641", os.path.join(HERE, "dist_worker_tp.py"), str(out)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    got = json.load(open(out))
    for rank in got["ranks"]:
        assert rank["ag_rel"] < 1e-2, rank
        assert rank["rs_rel"] < 1e-2, rank


def test_collective_lane_matches_single_process_math_on_cpu(tmp_path):
    """The baseline lane of TpGroup on gloo ranks: column-parallel then row-parallel linear == the unsharded MLP."""
    worker = tmp_path / "w.py"
    worker.write_text(
        "import os, sys, json, torch, torch.distributed as dist\n"
        f"sys.path.insert(0, {os.path.dirname(HERE)!r})\n"
        "from dataflow_b200.parallel.tp import TpGroup\n"
        "dist.init_process_group('gloo')\n"
        "r, w = dist.get_rank(), dist.get_world_size()\n"
        "g = torch.Generator().manual_seed(0)\n"
        "X = torch.randn(8 * w, 16, generator=g); W1 = torch.randn(16, 12 * w, generator=g); W2 = torch.randn(12 * w, 16, generator=g)\n"
        "grp = TpGroup(r, w, None, max_rows=8, max_k=16, max_n=16)\n"
        "h = grp.ag_gemm(X[r * 8:(r + 1) * 8].contiguous(), W1[:, r * 12:(r + 1) * 12].contiguous())\n"
        "y = grp.gemm_rs(h, W2[r * 12:(r + 1) * 12].contiguous())\n"
        "ref = (X @ W1 @ W2)[r * 8:(r + 1) * 8]\n"
        "ok = torch.allclose(y, ref, rtol=1e-4, atol=1e-4)\n"
        "allr = [None] * w; dist.all_gather_object(allr, bool(ok))\n"
        "if r == 0: json.dump(allr, open(sys.argv[1], 'w'))\n"
        "dist.destroy_process_group()\n")
    out = tmp_path / "o.json"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29643", str(worker), str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-3000:]
    assert json.load(open(out)) == [True, True]
