"""FLOP accounting, measured-duration replay and frozen-form rewriting of lowered programs."""
import dataclasses

import pytest

from dataflow_b200.blocks.optim import OptPolicy, freeze
from dataflow_b200.core.validate import validate_program
from dataflow_b200.lowering.flops import flop_report, print_table
from dataflow_b200.lowering.freeze import derive_freeze_plan, to_frozen_form
from dataflow_b200.lowering.planning import plan_program
from dataflow_b200.lowering.replay import replay_gap_pct, replay_makespan_us
from dataflow_b200.models.families import resolve_family
from dataflow_b200.run.presets import resolve_preset


def lowered(preset="llama3:tiny", **kw):
    fam, cfg = resolve_preset(preset)
    cfg = dataclasses.replace(cfg, **kw)
    f = resolve_family(fam)
    return f, cfg


def test_flop_report_is_complete_and_counts_recompute_separately():
    f, cfg = lowered(n_layers=3)
    p0 = f.lower(cfg)
    p2 = f.lower(cfg, recompute_levels={0: 2, 1: 2, 2: 2})
    r0, r2 = flop_report(p0), flop_report(p2, makespan_us=1e4)
    assert r0["completeness"] == [] and r2["completeness"] == []
    assert r0["recompute_flops"] == 0 and r2["recompute_flops"] > 0
    assert r2["effective_flops"] == pytest.approx(r0["effective_flops"])
    assert r2["hardware_flops"] == pytest.approx(r0["hardware_flops"] + r2["recompute_flops"])
    # forward + backward matmuls: about 6 FLOPs per parameter and token
    d = f.derive_dims(cfg)
    n_block = 3 * (d.d * (d.hq + 2 * d.hkv) * d.hd + d.hq * d.hd * d.d + 3 * d.d * d.F)
    tokens = p0.metadata["tokens_per_step"]
    blocks = r0["by_phase"]["fwd"]["flops"] + r0["by_phase"]["bwd"]["flops"] - r0["attention_flops"]
    assert blocks == pytest.approx(6 * n_block * tokens, rel=0.02)
    assert 0 < r0["attention_flops"] < r0["effective_flops"]
    assert "TFLOP/s" in print_table(r2)


def test_replay_with_measured_durations_isolates_scheduling_overhead():
    from dataflow_b200.run.driver import Trainer, synthetic_rounds
    f, cfg = lowered()
    tr = Trainer("llama3", cfg, budget_gib=None, device=None, seed=1)
    tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, 64, 0, 0))
    res = tr.last_result
    rep = replay_gap_pct(tr.program, res)
    assert rep["replay_us"] >= rep["compute_us"] * 0.999          # a schedule cannot beat its own compute time
    assert rep["measured_us"] >= rep["replay_us"] * 0.5
    # doubling every duration doubles an unconstrained replay
    dur = {iv.name: iv.end_us - iv.start_us for iv in res.trace.by_track("compute")}
    assert replay_makespan_us(tr.program, {k: 2 * v for k, v in dur.items()}) == pytest.approx(2 * rep["replay_us"], rel=0.05)
    tr.close()


def test_frozen_form_drops_updates_and_the_backward_of_a_frozen_prefix():
    f, cfg = lowered(n_layers=4, grad_accum_rounds=2)
    prog = f.lower(cfg)
    from dataflow_b200.models.llama3.model import block_fields, embed_fields, head_fields
    d = f.derive_dims(cfg)
    pol = freeze(OptPolicy(), layers=(0, 1), embed=True)
    plan = derive_freeze_plan(pol, 4, block_fields(d), embed_fields(d), head_fields(d))
    assert plan.frozen_layers == (0, 1) and plan.embed_frozen and not plan.head_frozen and plan.frozen_prefix == 2
    fz = to_frozen_form(prog, plan)
    validate_program(fz)
    ids = {t.id for t in fz.tasks}
    assert not any(i.startswith(("optimizer_0_0", "optimizer_0_1", "optimizer_embed")) for i in ids)
    assert not any(t.compute_block_key == "block_bwd" and t.block_params["layer"] < 2 for t in fz.tasks)
    assert any(t.compute_block_key == "block_bwd" and t.block_params["layer"] == 2 for t in fz.tasks)
    sizes = fz.object_sizes()
    assert "dW_0_0" not in sizes and "O_1" not in sizes and "dW_0_2" in sizes and "O_3" in sizes and "dW_embed_0" not in sizes
    assert not any(o.startswith("A_") and o.split("_")[-1] in ("0", "1") for o in sizes)       # contexts nobody reads
    assert "dy_0_0_1" not in sizes and "dy_0_0_2" in sizes
    # cheaper to run and plannable
    assert flop_report(fz)["effective_flops"] < flop_report(prog)["effective_flops"]
    planned = plan_program(fz, None)
    assert planned.makespan_us < plan_program(prog, None).makespan_us
    # a frozen layer in the middle keeps its (cheaper) backward
    mid = derive_freeze_plan(freeze(OptPolicy(), layers=(2,)), 4, block_fields(d), embed_fields(d), head_fields(d))
    assert mid.frozen_prefix == 0
    fm = to_frozen_form(prog, mid)
    validate_program(fm)
    b_old = next(t for t in prog.tasks if t.compute_block_key == "block_bwd" and t.block_params["layer"] == 2)
    b_new = next(t for t in fm.tasks if t.id == b_old.id)
    assert b_new.runtime_us < b_old.runtime_us and "dW_0_2" not in fm.object_sizes()
    # field-level freezing only annotates
    part = derive_freeze_plan(freeze(OptPolicy(), pairs=((1, "w_qkv"),)), 4, block_fields(d), embed_fields(d), head_fields(d))
    fp = to_frozen_form(prog, part)
    assert any(t.block_params.get("frozen_fields") == ["w_qkv"] for t in fp.tasks) and len(fp.tasks) == len(prog.tasks)
