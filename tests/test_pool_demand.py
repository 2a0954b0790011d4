"""Pools sized from a dry run of the plan on the virtual-time backend, and the engine corner the dry run found."""
import dataclasses
from types import SimpleNamespace

import pytest

from dataflow_b200.lowering import resolve_hardware
from dataflow_b200.models.families import resolve_family
from dataflow_b200.run.driver import Trainer, plan_at_budget, synthetic_rounds
from dataflow_b200.runtime import Engine, FakeBackend, Session
from dataflow_b200.runtime.pool_demand import PoolDemand, dry_run_pools

BUDGET = int(0.02 * (1 << 30))


@pytest.fixture(scope="module")
def tight():
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), n_layers=6, grad_accum_rounds=4)
    planned = plan_at_budget(fam, cfg, BUDGET, resolve_hardware("b200"), leeway_bytes=0, lower_kwargs={"resident_params": True})
    sizes = {}
    for o in planned.program.initial_objects:
        sizes.setdefault(o.id, o.size_bytes)
    return fam, cfg, planned, sizes


def test_the_dry_run_measures_what_the_plans_ledger_cannot(tight):
    _, _, planned, sizes = tight
    d = dry_run_pools(planned.program, sizes, planned.object_capacity, keep_resident=True, dispatch_ahead=2)
    assert isinstance(d, PoolDemand) and d.backing_overflows == 0 and d.fast_peak <= d.fast_capacity
    # the session's backing pool holds transient copies only; the plan's backing peak minus the store's size says less than they need
    from_ledger = max(planned.peak_backing_bytes - sum(sizes.values()), 0)
    assert d.backing_peak > from_ledger
    small = dry_run_pools(planned.program, sizes, planned.object_capacity, backing_capacity=from_ledger + (1 << 20), keep_resident=True, dispatch_ahead=2)
    right = dry_run_pools(planned.program, sizes, planned.object_capacity, backing_capacity=int(d.backing_peak * 1.02) + (1 << 20), keep_resident=True, dispatch_ahead=2)
    assert small.backing_overflows > 0 and right.backing_overflows == 0
    # under strict pacing this plan fragments the fast pool: requests fail for want of a hole, and the report prices them
    strict = dry_run_pools(planned.program, sizes, planned.object_capacity, keep_resident=True, dispatch_ahead=0)
    assert strict.fast_overflows > 0 and strict.fast_overflow_bytes >= strict.fast_overflows * 512 and not strict.fits


def test_an_object_the_valve_evicted_ends_on_the_device_when_the_program_wants_it_there(tight):
    """Dispatching ahead at a budget this tight makes the realised order leave the plan; the pressure valve then evicts a
    weight whose last reader has run.  The program keeps weights on the device from step to step, so the engine brings it
    back before it checks the final locations (it used to fail the run with FinalLocationError)."""
    _, _, planned, sizes = tight
    be = FakeBackend()
    ses = Session(be)
    ses.native.ensure_pools(int(planned.object_capacity), 1 << 30, 0.0, False)
    eng = Engine(be, session=ses)
    evictions = 0
    for step in range(3):
        res = eng.execute(planned.program, None, None, run_args={"step": step + 1}, manage_pools=False, keep_resident=True, dispatch_ahead=2)
        res.raise_if_failed()
        evictions += res.pressure_evictions
    assert evictions > 0                                 # the case is the one the fix is for
    held = ses.native.resident()
    want = {o for o, loc in planned.program.final_locations.items() if loc == "fast"}
    assert want and want <= set(held)


def test_pool_fitting_keeps_the_first_plan_unless_the_second_is_better(tight):
    fam, cfg, planned, sizes = tight
    stub = SimpleNamespace(program=planned.program, planned=planned, fam=fam, hw=resolve_hardware("b200"), verbose=False, pool_demand=None)
    got = Trainer._fit_pools(stub, cfg, sizes, planned.object_capacity, 1000, True, BUDGET, True, None, 0, {"resident_params": True},
                             replan=True, dispatch_ahead=0, min_cut=1 << 20)
    d = stub.pool_demand
    assert got >= int(d.backing_peak * 1.02) and d.fast_capacity >= planned.object_capacity
    if stub.planned is not planned:                    # a second plan is taken only when it overflows less and is not slower by more than 1 %
        assert stub.planned.makespan_us <= planned.makespan_us * 1.01 and stub.program is stub.planned.program
    # without permission to plan again, and without a budget, the plan is never touched
    for kw in ({"replan": False}, {"replan": True}):
        s2 = SimpleNamespace(program=planned.program, planned=planned, fam=fam, hw=stub.hw, verbose=False, pool_demand=None)
        Trainer._fit_pools(s2, cfg, sizes, planned.object_capacity, 1000, True, BUDGET if not kw["replan"] else None, True, None, 0,
                           {"resident_params": True}, dispatch_ahead=0, **kw)
        assert s2.planned is planned
    # a dry run that cannot finish leaves the sizing that was asked for
    broken = SimpleNamespace(program=None, planned=planned, fam=fam, hw=stub.hw, verbose=False, pool_demand=None)
    assert Trainer._fit_pools(broken, cfg, sizes, planned.object_capacity, 12345, True, BUDGET, True, None, 0, {}, replan=True) == 12345


def test_pool_sizing_runs_on_a_trainer_and_training_goes_on(monkeypatch):
    """The sizing a device run does before its first step, exercised on the CPU backend: dry run, backing pool from the
    measured peak, one allocation for the fast pool; steps afterwards allocate nothing more."""
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), n_layers=4, dtype_policy="fp32")
    tr = Trainer("llama3", cfg, budget_gib=0.03, device=None, hyper={"lr": 1e-3}, leeway_bytes=0, lower_kwargs={"resident_params": True})
    try:
        sizes = dict(tr.store.sizes)
        tr._size_pools(cfg, sizes, int(0.03 * (1 << 30)), 0, True, None, {"resident_params": True}, True, None, tr.keep_resident)
        assert tr.pool_mode == "slab" and tr.pool_demand is not None and tr.pool_demand.backing_overflows == 0
        assert tr.session.native.backing_slab()[1] >= tr.pool_demand.backing_peak
        assert tr.session.native.fast_slab()[1] >= tr.planned.peak_fast_bytes
        losses = [tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, 64, 0, 0)) for _ in range(3)]
        assert losses[-1] < losses[0]
        monkeypatch.setenv("DATAFLOW_POOL_FIT", "0")             # the switch: sizes from the plan's peaks, no dry run
        tr.pool_demand = None
        tr._size_pools(cfg, sizes, int(0.03 * (1 << 30)), 0, True, None, {"resident_params": True}, True, None, tr.keep_resident)
        assert tr.pool_demand is None
        with pytest.raises(ValueError, match="pool mode"):
            tr._size_pools(cfg, sizes, None, 0, True, None, None, False, "paged", tr.keep_resident)
    finally:
        tr.close()


def test_the_headline_configuration_ends_with_no_overflow_in_either_pool():
    """Llama-3-8B, 131 072 tokens per step in 8 rounds, 60 GiB: the first plan fills the device pool to 98 % and two 1.2 GiB
    requests per step find no hole; the pinned pool sized from the plan's ledger is less than half of what the transient
    copies need.  After fitting: a plan for about 1.2 GiB less in the same pool, no overflow anywhere, and a predicted step
    that is not slower."""
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["llama3_8b"](), seq_len=4096, batch=4, grad_accum_rounds=8, dtype_policy="bf16_split_master")
    hw = resolve_hardware("b200")
    budget = 60 << 30
    kw = {"resident_params": True}
    planned = plan_at_budget(fam, cfg, budget, hw, lower_kwargs=kw)
    sizes = {}
    for o in planned.program.initial_objects:
        sizes.setdefault(o.id, o.size_bytes)
    for t in planned.program.tasks:
        for out in t.outputs:
            if out.location == "backing" and out.id.startswith("loss_"):
                sizes[out.id] = out.size_bytes
    from dataflow_b200.lowering.planning import DEFAULT_PROGRAM_LEEWAY_BYTES
    pool = planned.object_capacity + min(DEFAULT_PROGRAM_LEEWAY_BYTES * 3 // 4, 1 << 30)
    ledger = max(planned.peak_backing_bytes - sum(sizes.values()), 0) + (64 << 20)
    first = dry_run_pools(planned.program, sizes, pool, backing_capacity=ledger, keep_resident=True, dispatch_ahead=2)
    assert first.backing_overflows > 20                      # the pinned pool was the one that overflowed
    stub = SimpleNamespace(program=planned.program, planned=planned, fam=fam, hw=hw, verbose=False, pool_demand=None)
    backing = Trainer._fit_pools(stub, cfg, sizes, pool, ledger, True, budget, True, None, None, kw, replan=True)
    assert backing > 1.5 * ledger and stub.planned.makespan_us <= planned.makespan_us * 1.01
    final = dry_run_pools(stub.program, sizes, pool, backing_capacity=backing, keep_resident=True, dispatch_ahead=2, steps=3)
    assert final.fits and final.fast_peak <= pool


def test_bench_plan_only_runs_without_a_device(capsys):
    """``bench.py --plan-only``: the bench configuration planned and its pools fitted on the CPU; says so in its output and
    never prints a bench line."""
    import importlib.util
    import json
    import os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_script", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    assert bench.main(["--plan-only", "--layers", "4", "--tokens-per-gpu", "32768", "--budget-gib", "12"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["plan_only"] and "not a measurement" in out["note"] and "metric" not in out and "value" not in out
    assert out["config"]["rounds"] == 2 and out["fitted"]["pools"]["backing_overflows_per_step"] == 0
    assert out["fitted"]["predicted_ms_per_step"] <= out["first_plan"]["predicted_ms_per_step"] * 1.01


def test_every_process_arrives_at_the_same_plan():
    """Ranks of a sharded run plan by themselves and must hold the same plan: the same inputs give the same plan in every
    process, whatever its string-hash seed (planners iterate over sets and dicts of object names)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = (
        "import dataclasses, hashlib, json\n"
        "from dataflow_b200.core import to_sim_chain\n"
        "from dataflow_b200.lowering import resolve_hardware\n"
        "from dataflow_b200.models.families import resolve_family\n"
        "from dataflow_b200.parallel.zero import zero_lower_kwargs\n"
        "from dataflow_b200.run.driver import plan_at_budget\n"
        "fam = resolve_family('llama3')\n"
        "cfg = dataclasses.replace(fam.presets['tiny'](), n_layers=6, grad_accum_rounds=4)\n"
        "out = []\n"
        "for kw, gib in (({'resident_params': True}, 0.02), (zero_lower_kwargs('fsdp', 1, 2), 0.02), ({'resident_params': True}, 0.014)):\n"
        "    p = plan_at_budget(fam, cfg, int(gib * (1 << 30)), resolve_hardware('b200'), leeway_bytes=0, lower_kwargs=kw)\n"
        "    ch = to_sim_chain(p.program)\n"
        "    rows = [[t.id, list(t.releases_after), [x.obj_id for x in t.offload_after], [x.obj_id for x in t.prefetch_after]] for t in ch.tasks]\n"
        "    out.append([hashlib.sha256(json.dumps(rows).encode()).hexdigest()[:16], p.policy, round(p.makespan_us, 3)])\n"
        "print(json.dumps(out))\n")
    seen = set()
    for seed in ("1", "2", "777"):
        env = dict(os.environ, PYTHONHASHSEED=seed, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600, env=env, cwd=root)
        assert r.returncode == 0, r.stderr[-2000:]
        seen.add(r.stdout.strip().splitlines()[-1])
    assert len(seen) == 1, seen
