"""Analytic workloads: schema validation, pricing, the model library through planner + simulator, and the HTTP API."""
import pytest

from dataflow_b200.sim.policies import get_all_policies
from dataflow_b200.sim.simulator import run as simulate
from dataflow_b200.sim.workloads import (MODEL_LIBRARY, ParallelismConfig, SubOp, TrainingConfig, WorkloadCost, WorkloadProgram,
                                         compute_summary, get_hardware, get_model, preview_workload, realize_workload, resolve_cost,
                                         trace_training_model)


def test_schema_refuses_bad_programs():
    ok = {"schema": "dataflow-workload/v1", "objects": [{"id": "w", "bytes": 8}],
          "tasks": [{"id": "t", "inputs": ["w"], "outputs": [{"id": "y", "bytes": 4}]}]}
    WorkloadProgram.model_validate(ok)
    for bad in ({**ok, "schema": "v0"},
                {**ok, "tasks": [{"id": "t", "inputs": ["nope"]}]},
                {**ok, "tasks": [{"id": "t", "inputs": ["w"], "mutates": ["y"]}]},
                {**ok, "tasks": ok["tasks"] * 2},
                {**ok, "final_locations": {"ghost": "fast"}}):
        with pytest.raises(ValueError):
            WorkloadProgram.model_validate(bad)


def test_cost_resolution_uses_the_hardware_row():
    b200, h100 = get_hardware("B200"), get_hardware("h100")
    mm = WorkloadCost(ops=[SubOp(kind="matmul", flops=1e12, dtype="bf16")])
    assert resolve_cost(mm, b200) < resolve_cost(mm, h100)
    assert resolve_cost(mm, b200) == pytest.approx(1e12 / (1669e12 * 0.84) * 1e6 + b200.launch_us)
    f8 = WorkloadCost(ops=[SubOp(kind="matmul", flops=1e12, dtype="fp8_e4m3")])
    assert resolve_cost(f8, b200) < resolve_cost(mm, b200)
    both = WorkloadCost(ops=mm.ops + [SubOp(kind="memory", bytes=6.5e9)], combine="max")
    assert resolve_cost(both, b200) == pytest.approx(max(resolve_cost(mm, b200), 6.5e9 / (6524e9 * 0.9) * 1e6 + b200.launch_us))
    with pytest.raises(ValueError):
        resolve_cost(WorkloadCost(ops=[SubOp(kind="scale_up", bytes=1e6)]), get_hardware("RTX_5090"))


def test_llama3_8b_parameter_count_and_flops():
    prog = trace_training_model(get_model("llama3_8b"), TrainingConfig(rounds=2))
    assert prog.metadata["total_params"] == pytest.approx(8.03e9, rel=0.01)
    pv = preview_workload(prog, get_hardware("B200"))
    tokens = 2 * 16384
    # 6 N T for the matmuls plus the attention term
    assert pv["total_flops"] > 6 * 7.5e9 * tokens
    assert pv["total_flops"] < 6 * 8.03e9 * tokens * 1.25


@pytest.mark.parametrize("name", sorted(MODEL_LIBRARY))
def test_every_library_model_plans_and_simulates(name):
    model = get_model(name)
    par = ParallelismConfig(ep_group_size=8 if any(l.mlp.kind == "moe" for l in model.layers) else 1, dp=8, zero_stage=3)
    prog = trace_training_model(model, TrainingConfig(tokens_per_round=8192, rounds=2, recompute="full", parallel=par))
    hw = get_hardware("B200")
    chain = realize_workload(prog, hw, int(150 * (1 << 30)))
    planned = get_all_policies()["pressurefit"](chain, chain.fast_memory_capacity)
    log = simulate(planned)
    s = compute_summary(planned, log, prog)
    assert s["peak_fast_bytes"] <= chain.fast_memory_capacity
    assert s["tokens_per_s"] > 0 and 0 <= s["recompute_pct"] < 50
    assert s["makespan_us"] >= preview_workload(prog, hw)["compute_only_us"] * 0.999


def test_summary_says_where_the_compute_time_goes():
    prog = trace_training_model(get_model("llama3_8b"), TrainingConfig(tokens_per_round=16384, rounds=2, recompute="selective"))
    hw = get_hardware("B200")
    chain = realize_workload(prog, hw, int(150 * (1 << 30)))
    planned = get_all_policies()["pressurefit"](chain, chain.fast_memory_capacity)
    s = compute_summary(planned, simulate(planned), prog, hw)
    assert abs(sum(s["compute_pct_by_kind"].values()) - 100.0) < 1e-6
    # a dense transformer at 8k context: the matmuls take most of the time, attention a visible part, element-wise the rest
    assert s["compute_pct_by_kind"]["matmul"] > 50 and s["compute_pct_by_kind"]["attention"] > 3
    assert 0 < s["mfu_pct"] < 100 and s["hardware_peak_tflops"] == hw.tflops("bf16")
    assert s["top_ops"][0]["us"] >= s["top_ops"][-1]["us"] and len(s["top_ops"]) == 10
    assert s["top_ops"][0]["calls"] >= 32          # one entry per op NAME: 32 layers, two rounds
    assert abs(sum(s["flops_by_phase"].values()) - s["total_flops"]) < 1e-6 * s["total_flops"]
    assert 0 <= s["from_slow_util_pct"] <= 100 and s["primary_unit"] == "tokens" and s["primary_count"] == 2 * 16384


def test_expert_parallel_is_priced_on_the_scale_up_fabric():
    model = get_model("olmoe_1b_7b")
    solo = trace_training_model(model, TrainingConfig())
    ep8 = trace_training_model(model, TrainingConfig(parallel=ParallelismConfig(ep_group_size=8)))
    names = lambda p: {op.name for t in p.tasks for op in t.cost.ops}
    fabric = lambda p: {op.name for t in p.tasks for op in t.cost.ops if op.kind == "scale_up"}
    assert {"block.moe.dispatch.a2a", "block.moe.combine.a2a", "block.moe.dispatch.a2a.bwd"} <= fabric(ep8) and not fabric(solo)
    w = lambda p: sum(o.bytes for o in p.objects if o.id.startswith("W_") and o.id[2:].isdigit())
    assert w(ep8) < w(solo) / 4


def test_http_api_preview_and_simulate():
    from fastapi.testclient import TestClient
    from dataflow_b200.sim.app.api import create_app
    c = TestClient(create_app())
    assert c.get("/api/health").json()["ok"]
    page = c.get("/")
    assert page.status_code == 200 and "text/html" in page.headers["content-type"]
    for needle in ('id="timeline"', 'id="memory"', "/api/simulate", "/api/presets", 'id="compare"', 'id="sweep"', 'id="measured"', 'id="subops"'):
        assert needle in page.text
    presets = c.get("/api/presets").json()
    assert "B200" in presets["hardware"] and "llama3_8b" in presets["models"] and "pressurefit" in presets["policies"]
    body = {"model": "llama3_8b", "training": {"rounds": 2, "tokens_per_round": 8192}, "hardware": "B200"}
    pv = c.post("/api/workloads/preview", json=body).json()["preview"]
    assert pv["tasks"] > 100 and pv["compute_only_us"] > 0
    sim = c.post("/api/simulate", json={**body, "fast_memory_gib": 40, "policy": "pressurefit", "memory_trace": True}).json()
    assert sim["summary"]["peak_fast_bytes"] <= 40 * (1 << 30)
    assert sim["summary"]["tokens_per_s"] > 0 and sim["timeline"] and sim["memory_trace"]
    assert sim["summary"]["from_slow_bytes"] > 0 and sim["summary"]["to_slow_bytes"] > 0      # a 40 GiB budget forces traffic
    assert c.post("/api/simulate", json={**body, "policy": "nope"}).status_code == 404
    assert c.post("/api/workloads/preview", json={"hardware": "B200"}).status_code == 422
    assert c.post("/api/workloads/preview", json={**body, "hardware": "abacus"}).status_code == 404
    tiny = {"schema": "dataflow-workload/v1", "objects": [{"id": "w", "bytes": 1024}],
            "tasks": [{"id": "t", "inputs": ["w"], "outputs": [{"id": "y", "bytes": 512}],
                       "cost": {"ops": [{"kind": "fixed", "runtime_us": 7.0}]}}]}
    r = c.post("/api/simulate", json={"program": tiny, "hardware": "H100", "policy": "all_resident"}).json()
    assert r["summary"]["makespan_us"] >= 7.0


def test_traced_blocks_reproduce_published_model_sizes_and_the_6nd_rule():
    """Every layer is a module traced on shape-only tensors; the parameter counts that fall out are the published ones, and
    forward + backward FLOPs per token are 6 x active parameters plus attention."""
    from dataflow_b200.sim.workloads.builders import MODEL_LIBRARY, TrainingBuilder
    want = {"llama3_8b": (8.03, 8.03), "llama3_70b": (70.55, 70.55), "qwen3_moe_30b_a3b": (30.5, 3.35), "olmoe_1b_7b": (6.92, 1.28),
            "deepseek_v3": (671.0, 37.6), "kimi_k2": (1026.0, 32.9), "gpt_oss_120b": (116.8, 5.7)}
    for name, (total, active) in want.items():
        prog = trace_training_model(get_model(name), TrainingConfig())
        assert prog.metadata["total_params"] / 1e9 == pytest.approx(total, rel=5e-3), name
        assert prog.metadata["active_params"] / 1e9 == pytest.approx(active, rel=1e-2), name
    model = get_model("llama3_8b")
    b = TrainingBuilder(model, TrainingConfig(seq_len=4096, tokens_per_round=16384))
    tr = b.trace(model.layers[0])
    per_token = (tr.flops("fwd") + tr.flops("bwd")) / 16384
    matmul = 6.0 * tr.active_params
    attn = 3.5 * 2.0 * 4096 * 32 * (128 + 128) * 0.5             # forward + 2.5x backward of the causal score / value products
    assert per_token == pytest.approx(matmul + attn, rel=1e-3)
    # what is kept for the backward: everything autograd would keep, or without what element-wise work rebuilds
    assert tr.saved_bytes() / 16384 == pytest.approx(136 * 1024 + 136, rel=1e-3)
    assert tr.saved_bytes(selective=True) / 16384 == pytest.approx((136 - 16 - 28) * 1024 + 136, rel=1e-3)
    assert {s.name for s in tr.saved if s.cheap} == {"block.norm1", "block.norm2", "block.mlp.swiglu"}


def test_tensor_and_expert_parallel_layouts_divide_what_a_rank_holds():
    from dataflow_b200.sim.workloads.builders import MODEL_LIBRARY, TrainingBuilder
    model = get_model("deepseek_v3")
    solo = TrainingBuilder(model, TrainingConfig()).trace(model.layers[10])
    ep = TrainingBuilder(model, TrainingConfig(parallel=ParallelismConfig(ep_group_size=8))).trace(model.layers[10])
    tp = TrainingBuilder(model, TrainingConfig(parallel=ParallelismConfig(tp=8))).trace(model.layers[10])
    assert ep.total_params == solo.total_params == tp.total_params
    experts = sum(p.numel for p in solo.params if p.kind == "experts")
    assert ep.local_params == pytest.approx(solo.local_params - experts * 7 / 8)
    assert tp.local_params < solo.local_params and any(op.kind == "scale_up" for op in tp.fwd)
    assert sum(op.flops for op in tp.fwd if "mla.core" in op.name) == pytest.approx(sum(op.flops for op in solo.fwd if "mla.core" in op.name) / 8)
