"""tp_mlp family: tensor + sequence parallel llama blocks against the single-process llama3 engine from the same seed."""
import dataclasses
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def launch(world, device_kind, tmp_path, lane=None, port=29811, budget=None):
    out = tmp_path / f"tpfam_{device_kind}_{lane}_{budget}.json"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    env.pop("DATAFLOW_TP_LANE", None)
    env.pop("TP_TEST_BUDGET", None)
    if lane:
        env["DATAFLOW_TP_LANE"] = lane
    if budget:
        env["TP_TEST_BUDGET"] = str(budget)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "dist_worker_tpfam.py"), str(out), device_kind]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    if r.returncode:
        at = r.stderr.find("Traceback")
        raise AssertionError(r.stderr[at:at + 3000] if at >= 0 else r.stdout[-1500:] + r.stderr[-1500:])
    return json.loads(out.read_text())


def solo_losses(policy="fp32", **over):
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy=policy, **over)
    tr = Trainer("llama3", cfg, budget_gib=None, device=None, hyper={"lr": 2e-3, "weight_decay": 0.1}, seed=3, leeway_bytes=0)
    try:
        return [tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, s)) for s in range(3)]
    finally:
        tr.close()


def test_family_structure_and_sharded_sizes():
    from dataflow_b200.models.families import resolve_family, validate_family
    assert validate_family("tp_mlp") == []
    fam = resolve_family("tp_mlp")
    cfg = fam.presets["tiny"]()
    d = fam.derive_dims(cfg)
    assert (d.tp, d.hq, d.hkv, d.F, d.T, d.Ts) == (2, 2, 1, 256, 256, 128)
    full = resolve_family("llama3")
    lay_l, lay_f = fam.family_layouts(d), full.family_layouts(full.derive_dims(cfg))
    assert lay_l.block_w.size_bytes < 0.55 * lay_f.block_w.size_bytes
    prog = fam.lower(cfg)
    assert prog.object_sizes()["y_0_0_0"] == d.Ts * d.d * 2 and prog.metadata["tp"] == 2
    assert all(t.comm_groups.get("tp") == "tp" for t in prog.tasks if t.compute_block_key == "block_fwd")


def test_slices_reassemble_the_full_model():
    import torch
    from dataflow_b200.models.llama3.model import derive_dims
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.models.tp_mlp import slice_for_rank
    cfg = resolve_family("tp_mlp").presets["tiny"]()
    df = derive_dims(cfg)
    w13 = torch.arange(df.d * 2 * df.F, dtype=torch.float32).view(df.d, 2 * df.F)
    parts = [slice_for_rank("w13", w13, df, r, 2) for r in range(2)]
    fl = df.F // 2
    assert torch.equal(torch.cat([parts[0][:, :fl], parts[1][:, :fl]], 1), w13[:, :df.F])
    assert torch.equal(torch.cat([parts[0][:, fl:], parts[1][:, fl:]], 1), w13[:, df.F:])
    wqkv = torch.arange(df.d * df.qkv_dim, dtype=torch.float32).view(df.d, df.qkv_dim)
    p0 = slice_for_rank("w_qkv", wqkv, df, 0, 2)
    assert p0.shape[1] == df.qkv_dim // 2 and torch.equal(p0[:, :df.q_dim // 2], wqkv[:, :df.q_dim // 2])
    assert torch.equal(slice_for_rank("wo", wqkv[:, :df.q_dim].t().contiguous(), df, 1, 2), wqkv[:, df.q_dim // 2:df.q_dim].t())


def test_two_cpu_ranks_match_the_single_process_model(tmp_path):
    got = launch(2, "cpu", tmp_path, port=29813)
    ref = solo_losses()
    for a, b in zip(got["losses"], ref):
        assert a == pytest.approx(b, rel=5e-4)
    assert got["losses"][-1] < got["losses"][0]


def test_recompute_under_a_tight_budget_does_not_change_the_losses(tmp_path):
    free = launch(2, "cpu", tmp_path, port=29815)
    tight = launch(2, "cpu", tmp_path, port=29817, budget=0.012)
    assert tight["losses"] == pytest.approx(free["losses"], rel=1e-6)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
def test_fused_kernels_train_like_the_collective_lane(tmp_path):
    p2p = launch(2, "cuda", tmp_path, lane="p2p", port=29819)
    col = launch(2, "cuda", tmp_path, lane="collective", port=29821)
    for a, b in zip(p2p["losses"], col["losses"]):
        assert a == pytest.approx(b, rel=2e-2)
    assert p2p["losses"][-1] < p2p["losses"][0]


def test_vocab_parallel_head_matches_the_replicated_head(tmp_path):
    """`--vocab-parallel`: every rank holds half of the output projection's columns and exchanges softmax statistics; the
    curve is the replicated head's (and one process's), and the head objects are half the size."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, os.path.join(root, "tools", "train", "train.py"), "train", "--preset", "llama3:tiny", "--steps", "4", "--device", "cpu",
            "--dtype-policy", "fp32"]

    def run(extra, name):
        out = tmp_path / f"{name}.json"
        r = subprocess.run(base + extra + ["--out", str(out)], capture_output=True, text=True, timeout=900, cwd=root)
        assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2500:]
        return json.loads(out.read_text())["losses"]

    solo = run([], "solo")
    rep = run(["--gpus", "2", "--parallel", "tp"], "rep")
    vp = run(["--gpus", "2", "--parallel", "tp", "--vocab-parallel"], "vp")
    assert vp == pytest.approx(rep, rel=2e-4) and vp == pytest.approx(solo, rel=5e-4)
    assert vp[-1] < vp[0]
    import dataclasses
    from dataflow_b200.models.families import resolve_family
    fam = resolve_family("tp_mlp")
    cfg = fam.presets["tiny"]()
    full = fam.lower(cfg).object_sizes()
    half = fam.lower(dataclasses.replace(cfg, vocab_parallel=True)).object_sizes()
    assert half["W_head"] < 0.51 * full["W_head"] + 4096 and half["O_head"] < 0.51 * full["O_head"] + 4096
    assert half["W_embed"] == full["W_embed"]
