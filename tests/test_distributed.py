"""Schemes, shard plans, responsibilities / source policy, topology, group annotation, and the daemon tools."""
import os
import subprocess
import sys
import time

import pytest

from dataflow_b200.distributed import (ParallelismScheme, SchemeError, annotate_groups, compile_source_policy, expert_shards,
                                       load_topology, local_topology, responsibility_map, rs_eligible, scheme_from_flags,
                                       tp_attn_shards, tp_mlp_shards, zero_slices)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_scheme_grid_and_validation():
    s = scheme_from_flags(8, tp=4)                       # dp2 x tp4
    assert [a.kind for a in s.axes] == ["dp", "tp"] and s.world == 8
    assert s.coords(5) == {"dp": 1, "tp": 1}
    assert s.group_members("tp", 5) == [4, 5, 6, 7] and s.group_members("dp", 5) == [1, 5]
    assert ParallelismScheme.from_dict(s.to_dict()) == s
    w = ParallelismScheme.data_parallel(rank_rounds=[6, 2], responsibility="zero1rs").validate(2)
    assert w.rounds_of(0, 4) == 6 and w.rounds_of(1, 4) == 2
    with pytest.raises(SchemeError, match="responsibility"):
        ParallelismScheme.data_parallel(2, responsibility="zero9").validate()
    with pytest.raises(SchemeError, match="covers 4 ranks"):
        scheme_from_flags(4).validate(8)
    with pytest.raises(SchemeError, match="does not divide"):
        scheme_from_flags(6, tp=4)
    with pytest.raises(SchemeError, match="tp and ep"):
        scheme_from_flags(8, tp=2, ep=2)


def test_tp_and_ep_shard_plans_cover_everything_once():
    mlp = tp_mlp_shards(64, 256, 4)
    assert mlp.equal_shards and mlp.local_shape(1, "w13") == (64, 128) and mlp.local_shape(1, "w2") == (64, 64)
    assert mlp.replicated("norm2")
    attn = tp_attn_shards(4096, 32, 8, 128, 8)            # llama-3 geometry over 8 ranks: one KV head each
    assert attn.local_shape(3, "w_qkv") == (4096, (4 + 2) * 128) and attn.local_shape(3, "wo") == (512, 4096)
    with pytest.raises(ValueError, match="GQA groups"):
        tp_attn_shards(4096, 32, 8, 128, 16)
    ep = expert_shards(64, 8, {"w13": (2048, 2048), "w2": (1024, 2048)})
    assert ep.equal_shards and ep.owned_ranges(2, "w2")[0].row_lo == 16 * 1024


def test_zero_slices_and_eligibility():
    sl = zero_slices(1000, 4)
    assert sl == [(0, 256), (256, 256), (512, 256), (768, 232)] and sum(n for _, n in sl) == 1000
    assert zero_slices(300, 4)[2:] == [(300, 0), (300, 0)]
    assert rs_eligible(["bf16"], ["bf16"], ["adamw"]) and not rs_eligible(["bf16"], ["fp32"], ["adamw"])
    assert not rs_eligible(["bf16"], ["bf16"], ["adamw", "muon"])


def test_responsibilities_and_source_policy():
    objs = {"W_0": 1000, "O_0": 3000, "Aux_0": 64}
    z3 = responsibility_map(objs, scheme_from_flags(4, opt_shard="zero3"))
    assert [(s.lo, s.hi) for s in z3["W_0"]] == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    z1 = responsibility_map(objs, scheme_from_flags(4, opt_shard="zero1rs"))
    assert all(s.lo == 0 and s.hi == 1000 for s in z1["W_0"]) and len(z1["O_0"]) == 4 and z1["O_0"][1].lo == 768
    logical, writes = compile_source_policy("dedup", z1, private=["Aux_0"])
    assert logical == {"W_0": 1000, "O_0": 3000, "Aux_0@0": 64, "Aux_0@1": 64, "Aux_0@2": 64, "Aux_0@3": 64}
    assert [w.source for w in writes if w.logical_id == "W_0"] == [0]
    _, simple = compile_source_policy("simple", z1)
    assert len([w for w in simple if w.logical_id == "W_0"]) == 4
    # dp2 x tp2: the dp slice is replicated across the tp pair; dedup keeps one writer per slice
    mesh = responsibility_map({"O_0": 1024}, scheme_from_flags(4, tp=2, opt_shard="zero1rs"))
    _, w = compile_source_policy("dedup", mesh)
    assert sorted((x.source, x.lo) for x in w) == [(0, 0), (2, 512)]


def test_topology_toml_and_local(tmp_path):
    p = tmp_path / "topo.toml"
    p.write_text('[hosts.box]\ndevices = [0, 1]\nbacking_gib = 32\n[hosts.far]\naddress = "me@far"\ndevices = [0]\n'
                 '[groups.train]\nmembers = ["box:0", "box:1", "far:0"]\n')
    t = load_topology(str(p))
    g = t.group()
    assert g.world == 3 and g.coordinator.key == "box:0" and t.host_of(g.members[2]).address == "me@far"
    assert t.hosts["box"].local and not t.hosts["far"].local
    p.write_text('[hosts.box]\ndevices = [0]\n[groups.g]\nmembers = ["box:1"]\n')
    with pytest.raises(ValueError, match="no device 1"):
        load_topology(str(p))
    assert local_topology(4).group().world == 4


def test_group_annotation_stamps_communicating_tasks():
    import dataclasses
    from dataflow_b200.models.families import resolve_family
    fam = resolve_family("llama3")
    prog = fam.lower(fam.presets["tiny"]())
    s = scheme_from_flags(4, tp=2)
    out = annotate_groups(prog, s, rank=3, group_names={"tp": "tp_group_1"})
    opt = next(t for t in out.tasks if (t.compute_block_key or "").startswith("optimizer_block"))
    assert opt.comm_groups == {"dp": "dp", "tp": "tp_group_1"} and opt.block_params["axes"]["tp"]["rank"] == 1
    blk = next(t for t in out.tasks if "fwd" in t.id and "block" in t.id)
    assert blk.compute_block_key.startswith("tp_")
    assert out.metadata["scheme"]["world"] == 4
    assert annotate_groups(prog, ParallelismScheme.solo(), 0) is prog


def test_daemon_start_status_stop(tmp_path):
    sock = str(tmp_path / "d.sock")
    tool = os.path.join(ROOT, "tools/train/dataflowd.py")
    env = {**os.environ, "PYTHONPATH": ROOT}
    assert subprocess.call([sys.executable, tool, "start", "--socket", sock, "--fake", "--backing-gib", "0.05"], env=env) == 0
    try:
        for _ in range(150):
            if subprocess.call([sys.executable, tool, "status", "--socket", sock], env=env, stdout=subprocess.DEVNULL,
                               stderr=subprocess.DEVNULL) == 0:
                break
            time.sleep(0.2)
        else:
            pytest.fail("daemon did not come up: " + open(sock[:-5] + ".log").read()[-2000:])
        assert subprocess.call([sys.executable, tool, "stop", "--socket", sock], env=env) == 0
        for _ in range(100):
            if not os.path.exists(sock):
                break
            time.sleep(0.1)
        assert not os.path.exists(sock)
    finally:
        subprocess.call([sys.executable, os.path.join(ROOT, "tools/train/daemonize.py"), "--pidfile", sock[:-5] + ".pid", "--kill"],
                        stderr=subprocess.DEVNULL)


@pytest.mark.parametrize("parallel,preset", [("tp", "llama3:tiny"), ("ep", "olmoe:tiny"), ("ep", "dsv32:tiny")])
def test_train_cli_runs_tensor_and_expert_parallel_jobs_on_cpu_ranks(parallel, preset, tmp_path):
    """`train.py train --gpus 2 --parallel tp|ep` end to end on two gloo ranks: packed data, loop, result file."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / f"{parallel}.json"
    cmd = [sys.executable, os.path.join(root, "tools", "train", "train.py"), "train", "--preset", preset, "--steps", "3", "--device", "cpu",
           "--gpus", "2", "--parallel", parallel, "--out", str(out), "--dtype-policy", "fp32"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=root)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-2500:]
    res = json.loads(out.read_text())
    assert len(res["losses"]) == 3 and min(res["losses"][1:]) < res["losses"][0]       # three steps of a short, decaying schedule
    assert res["meta"]["world"] == 2


@pytest.mark.parametrize("parallel,preset", [("tp", "llama3:tiny"), ("ep", "olmoe:tiny"), ("ep", "dsv3:tiny")])
def test_tensor_and_expert_parallel_jobs_resume_bitwise(parallel, preset, tmp_path):
    """Every rank's cut of the model is recorded per rank; a resumed run continues the interrupted curve exactly."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, os.path.join(root, "tools", "train", "train.py"), "train", "--preset", preset, "--steps", "4", "--device", "cpu",
            "--gpus", "2", "--parallel", parallel, "--dtype-policy", "fp32", "--checkpoint-dir", str(tmp_path / "ck")]
    a = subprocess.run(base + ["--checkpoint-every", "2", "--out", str(tmp_path / "a.json")], capture_output=True, text=True, timeout=600, cwd=root)
    assert a.returncode == 0, a.stdout[-1000:] + a.stderr[-2500:]
    rec = json.loads((tmp_path / "ck" / "step_000002" / "checkpoint_record.json").read_text())
    assert rec["scheme"]["world"] == 2 and rec["scheme"]["parallel"] == parallel
    assert any(k.endswith("@1") for k in rec["logical_objects"])
    b = subprocess.run(base + ["--resume", str(tmp_path / "ck" / "step_000002"), "--out", str(tmp_path / "b.json")], capture_output=True,
                       text=True, timeout=600, cwd=root)
    assert b.returncode == 0, b.stdout[-1000:] + b.stderr[-2500:]
    assert json.loads((tmp_path / "a.json").read_text())["losses"] == json.loads((tmp_path / "b.json").read_text())["losses"]


def test_plain_and_weighted_data_parallel_jobs_match_one_process(tmp_path):
    """`--parallel co`: replicas with all-reduced gradients.  Two ranks running 2 + 2 rounds, or 3 + 1 rounds (weighted), walk
    the same curve as one process running the 4 rounds of the same packed steps."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, os.path.join(root, "tools", "train", "train.py"), "train", "--preset", "llama3:tiny", "--steps", "3", "--device", "cpu",
            "--dtype-policy", "fp32"]

    def run(extra, name):
        out = tmp_path / f"{name}.json"
        r = subprocess.run(base + extra + ["--out", str(out)], capture_output=True, text=True, timeout=600, cwd=root)
        assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2500:]
        return json.loads(out.read_text())["losses"]

    solo = run(["--ga-rounds", "4"], "solo")
    even = run(["--gpus", "2", "--parallel", "co", "--ga-rounds", "2"], "even")
    weighted = run(["--gpus", "2", "--parallel", "co", "--rounds", "3,1"], "weighted")
    # the order in which round gradients are summed differs (per rank, then over ranks): noise of that size only
    assert even == pytest.approx(solo, rel=2e-4)
    assert weighted == pytest.approx(solo, rel=2e-4)


def test_data_parallel_replicas_of_a_tensor_parallel_group_match_one_process(tmp_path):
    """A 2 x 2 mesh on four CPU ranks: two tensor-parallel groups of two ranks, the groups data-parallel replicas of each
    other (gradients summed over the replicas in front of the optimizer), against one process running all the rounds."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, os.path.join(root, "tools", "train", "train.py"), "train", "--preset", "llama3:tiny", "--steps", "3", "--device", "cpu",
            "--dtype-policy", "fp32"]

    def run(extra, name):
        out = tmp_path / f"{name}.json"
        r = subprocess.run(base + extra + ["--out", str(out)], capture_output=True, text=True, timeout=900, cwd=root)
        assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2500:]
        return json.loads(out.read_text())

    solo = run(["--ga-rounds", "4"], "solo")
    mesh = run(["--gpus", "4", "--parallel", "tp", "--tp-size", "2", "--ga-rounds", "2", "--checkpoint-dir", str(tmp_path / "ck"),
                "--checkpoint-every", "2"], "mesh")
    assert mesh["meta"]["world"] == 4 and mesh["tokens_per_step"] == solo["tokens_per_step"]
    assert mesh["losses"] == pytest.approx(solo["losses"], rel=5e-4)
    rec = json.loads((tmp_path / "ck" / "step_000002" / "checkpoint_record.json").read_text())
    assert rec["scheme"]["world"] == 4 and sorted(os.listdir(tmp_path / "ck" / "step_000002" / "programs")) == [f"rank{i}.json" for i in range(4)]
    again = run(["--gpus", "4", "--parallel", "tp", "--tp-size", "2", "--ga-rounds", "2", "--checkpoint-dir", str(tmp_path / "ck"),
                 "--resume", str(tmp_path / "ck" / "step_000002")], "again")
    assert again["losses"] == pytest.approx(mesh["losses"], rel=1e-5)


@pytest.mark.parametrize("preset", ["olmoe:tiny", "dsv3:tiny"])
def test_replicas_of_an_expert_parallel_group_match_one_process(preset, tmp_path):
    """A 2 x 2 mesh on four CPU ranks: the experts are split over pairs of ranks, the pairs are replicas of each other.
    Replicated parameters sum their gradients over all four ranks, expert stacks over the two ranks that hold the same
    experts.  Oracle: one process with all experts running every rank's rounds."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, os.path.join(root, "tools", "train", "train.py"), "train", "--preset", preset, "--steps", "3", "--device", "cpu",
            "--dtype-policy", "fp32"]

    def run(extra, name):
        out = tmp_path / f"{name}.json"
        r = subprocess.run(base + extra + ["--out", str(out)], capture_output=True, text=True, timeout=900, cwd=root)
        assert r.returncode == 0, r.stdout[-1000:] + r.stderr[-2500:]
        return json.loads(out.read_text())

    solo = run(["--ga-rounds", "4"], "solo")
    ck = tmp_path / "ck"
    mesh = run(["--gpus", "4", "--parallel", "ep", "--ep-size", "2", "--ga-rounds", "1", "--checkpoint-dir", str(ck), "--checkpoint-every", "3"],
               "mesh")
    assert mesh["meta"]["world"] == 4 and mesh["tokens_per_step"] == solo["tokens_per_step"]
    assert mesh["losses"] == pytest.approx(solo["losses"], rel=1e-3)
    assert mesh["losses"][-1] < mesh["losses"][0]

    # ranks 0 and 2 (1 and 3) hold the same experts and every replicated parameter: after three steps their weights and
    # optimizer state are the same bytes; ranks 0 and 1 hold different experts
    def hashes(r):
        m = json.loads((ck / "step_000003" / f"rank{r}" / "snapshot_manifest.json").read_text())
        return {e["id"]: e["hash"] for e in m["slices"]}
    h = [hashes(r) for r in range(4)]
    assert h[0] == h[2] and h[1] == h[3]
    assert h[0]["W_embed"] == h[1]["W_embed"] and h[0]["O_head"] == h[1]["O_head"]
    moe_layers = [k for k in h[0] if k.startswith("W_") and h[0][k] != h[1][k]]
    assert moe_layers and all(k[2:].isdigit() for k in moe_layers)


def _abi_worker(rank, world, port, out):
    import os
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from dataflow_b200.parallel.zero import DpGroup
    g = DpGroup(rank, world, None)
    t = torch.full((4,), float(rank + 1))
    g.all_reduce(t)
    b = torch.full((3,), float(rank))
    g.broadcast(b, root=1)
    r = torch.full((2,), float(rank + 1))
    g.reduce(r, root=0)
    full = torch.zeros(world * 2)
    g.all_gather(torch.full((2,), float(rank)), full)
    rs = torch.zeros(2)
    g.reduce_scatter(torch.arange(world * 2, dtype=torch.float32) * (rank + 1), rs)
    out[rank] = (t.tolist(), b.tolist(), r.tolist(), full.tolist(), rs.tolist())
    dist.destroy_process_group()


def test_group_objects_answer_the_whole_collective_abi():
    """all_reduce / broadcast / reduce / all_gather / reduce_scatter through a group object on two CPU ranks: the list an
    executable may rely on under every launcher (reduce leaves non-root tensors untouched)."""
    import torch.multiprocessing as mp
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_abi_worker, args=(world, 29733, out), nprocs=world, join=True)
        got = dict(out)
    assert got[0][0] == got[1][0] == [3.0] * 4
    assert got[0][1] == got[1][1] == [1.0] * 3
    assert got[0][2] == [3.0, 3.0] and got[1][2] == [2.0, 2.0]
    assert got[0][3] == got[1][3] == [0.0, 0.0, 1.0, 1.0]
    assert got[0][4] == [0.0, 3.0] and got[1][4] == [6.0, 9.0]


def test_sharded_optimizer_state_restores_at_another_world_size(tmp_path):
    """ZeRO-1 on two CPU ranks, checkpoint, resume on FOUR ranks (the same global batch): the optimizer state is recorded as
    spans of logical planes (``O_0.m`` ...), every rank of the new job reads the spans that cover its new slice, and the
    curve continues where the two-rank run would have gone (up to the order of the gradient sums)."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    base = [sys.executable, os.path.join(root, "tools", "train", "train.py"), "train", "--preset", "llama3:tiny", "--steps", "4", "--device", "cpu",
            "--parallel", "zero1", "--dtype-policy", "bf16_master", "--checkpoint-dir", str(tmp_path / "ck")]
    a = subprocess.run(base + ["--gpus", "2", "--ga-rounds", "2", "--checkpoint-every", "2", "--out", str(tmp_path / "a.json")],
                       capture_output=True, text=True, timeout=900, cwd=root)
    assert a.returncode == 0, a.stdout[-1000:] + a.stderr[-2500:]
    rec = json.loads((tmp_path / "ck" / "step_000002" / "checkpoint_record.json").read_text())
    assert rec["scheme"]["world"] == 2
    planes = [k for k in rec["logical_objects"] if k.startswith("O_0.")]
    assert sorted(planes) == ["O_0.m", "O_0.master", "O_0.v"] and not any("@" in k for k in rec["logical_objects"] if k.startswith("O_"))
    b = subprocess.run(base + ["--gpus", "4", "--ga-rounds", "1", "--resume", str(tmp_path / "ck" / "step_000002"), "--out", str(tmp_path / "b.json")],
                       capture_output=True, text=True, timeout=900, cwd=root)
    assert b.returncode == 0, b.stdout[-1000:] + b.stderr[-2500:]
    la, lb = json.loads((tmp_path / "a.json").read_text())["losses"], json.loads((tmp_path / "b.json").read_text())["losses"]
    assert len(la) == len(lb) == 4 and la[:2] == lb[:2]
    for x, y in zip(la[2:], lb[2:]):
        assert abs(x - y) / x < 2e-3, (la, lb)


def _probe_worker(rank, world, port, out):
    import os
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from dataflow_b200.lowering import resolve_hardware
    from dataflow_b200.run.scaling import hardware_as_shared
    hw = hardware_as_shared(resolve_hardware("b200"), world, 0, probe=lambda dev: (40.0 - 10.0 * rank, 30.0 + 5.0 * rank))
    out[rank] = (hw.h2d_gbs, hw.d2h_gbs, hw.link_gbs)
    dist.destroy_process_group()


def test_multi_rank_plans_are_priced_with_the_measured_concurrent_host_rate():
    """Every rank measures its host link while the others do the same; the slowest figure (times 0.95) caps the hardware row all
    ranks plan with, so the plans stay identical; one rank alone, or ``DATAFLOW_PCIE_PROBE=0``, keeps the preset."""
    import torch.multiprocessing as mp
    from dataflow_b200.lowering import resolve_hardware
    from dataflow_b200.run.scaling import hardware_as_shared
    base = resolve_hardware("b200")
    assert hardware_as_shared(base, 1, 0) == base
    assert hardware_as_shared(base, 4, None) == base.shared(4)
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_probe_worker, args=(2, 29741, out), nprocs=2, join=True)
        got = dict(out)
    assert got[0] == got[1]
    h2d, d2h, link = got[0]
    assert h2d == pytest.approx(0.95 * 30.0) and d2h == pytest.approx(0.95 * 30.0) and link == base.h2d_gbs
