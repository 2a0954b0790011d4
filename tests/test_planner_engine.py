import pytest

from chains import train_chain
from dataflow_b200.core import from_sim_chain
from dataflow_b200.runtime import DeadlockError, Engine, FakeBackend, compare_to_sim_eventlog
from dataflow_b200.sim import run
from dataflow_b200.sim.policies.pressurefit import PlanningError, pressurefit


@pytest.mark.parametrize("cap", [20000, 6000, 3000, 2200, 1800])
def test_pressurefit_fits_and_engine_matches_simulator_exactly(cap):
    r = pressurefit(train_chain(), cap)
    log = run(r.chain)
    assert log.peak_fast_memory_bytes <= cap
    assert r.makespan >= r.lower_bound
    res = Engine(FakeBackend()).execute(from_sim_chain(r.chain)).raise_if_failed()
    assert compare_to_sim_eventlog(res.trace, log) == []
    assert res.slab_overflows == 0 and res.makespan_us == log.makespan


def test_ample_budget_is_compute_bound_after_preload():
    r = pressurefit(train_chain(L=4, rounds=1), 10 ** 9)
    assert r.makespan <= r.lower_bound * 1.35      # first load and last write-back cannot overlap compute


def test_infeasible_budget_raises():
    with pytest.raises(PlanningError):
        pressurefit(train_chain(), 1000)       # optimizer task alone needs 1600 bytes


def test_engine_session_reuse_allocates_nothing_in_steady_state():
    r = pressurefit(train_chain(L=4, rounds=2), 3000)
    prog = from_sim_chain(r.chain)
    eng = Engine(FakeBackend())
    eng.execute(prog).raise_if_failed()
    before = eng.session.vendor_allocs()
    for _ in range(3):
        res = eng.execute(prog).raise_if_failed()
        assert res.vendor_allocs == 0
    assert eng.session.vendor_allocs() == before


def test_engine_deadlock_is_reported_not_hung():
    from dataflow_b200.core import ObjectSpec, OutputSpec, Program, TaskSpec
    p = Program("d", (ObjectSpec("x", 90, "fast"),), (TaskSpec("a", inputs=("x",), outputs=(OutputSpec("y", 20),)),),
                fast_memory_capacity=100)
    res = Engine(FakeBackend()).execute(p)
    assert res.outcome.kind.value == "FAILED" and res.outcome.error_kind == "DeadlockError"
    with pytest.raises(DeadlockError):
        res.raise_if_failed()


def test_transfer_time_distortion_changes_timing_not_results():
    r = pressurefit(train_chain(L=4, rounds=2), 2500)
    prog = from_sim_chain(r.chain)
    be = FakeBackend()
    be.transfer_time_scale = 3.0
    res = Engine(be).execute(prog)
    assert res.outcome.ok and res.makespan_us >= r.makespan


# ---------------------------------------------------------------- lookahead (oracle-in-the-loop) planner
@pytest.mark.parametrize("cap", [20000, 6000, 3000, 2200, 1800])
def test_lookahead_fits_and_engine_matches_simulator_exactly(cap):
    from dataflow_b200.sim.policies.lookahead import lookahead
    r = lookahead(train_chain(), cap)
    log = run(r.chain)
    assert log.peak_fast_memory_bytes <= cap
    assert log.makespan == r.makespan >= r.lower_bound
    res = Engine(FakeBackend()).execute(from_sim_chain(r.chain)).raise_if_failed()
    assert compare_to_sim_eventlog(res.trace, log) == []
    assert res.makespan_us == log.makespan


def test_lookahead_unbounded_moves_only_what_must_move():
    from dataflow_b200.sim.policies.lookahead import lookahead
    ch = train_chain(L=4, rounds=2)
    r = lookahead(ch, None)
    log = run(r.chain)
    loads = [iv for iv in log.task_intervals if iv.track == "from_slow"]
    stores = [iv for iv in log.task_intervals if iv.track == "to_slow"]
    preplaced = [o for o in r.chain.initial_memory if o.location == "fast"]
    # tok + W, O come in once each (up front or by prefetch); W, O are written back once
    assert len(loads) + len(preplaced) == 9 and len(stores) == 8


def test_plan_program_auto_takes_the_better_planner():
    from dataflow_b200.lowering.planning import plan_program
    prog = from_sim_chain(train_chain())
    a = plan_program(prog, 3000, leeway_bytes=0, policy="auto")
    b = plan_program(prog, 3000, leeway_bytes=0, policy="pressurefit")
    c = plan_program(prog, 3000, leeway_bytes=0, policy="lookahead")
    assert a.makespan_us <= min(b.makespan_us, c.makespan_us) + 1e-9
    assert c.policy.startswith("lookahead:")


def test_plan_program_wide_adds_the_span_planners(monkeypatch):
    from dataflow_b200.lowering.planning import plan_program
    from dataflow_b200.runtime import Engine, FakeBackend
    prog = from_sim_chain(train_chain())
    a = plan_program(prog, 2500, leeway_bytes=0, policy="auto")
    w = plan_program(prog, 2500, leeway_bytes=0, policy="wide")
    assert w.makespan_us <= a.makespan_us + 1e-9 and w.candidates > a.candidates
    monkeypatch.setenv("DATAFLOW_PLANNER", "wide")          # the run-wide switch replaces "auto"
    e = plan_program(prog, 2500, leeway_bytes=0)
    assert e.makespan_us == w.makespan_us and e.policy == w.policy
    res = Engine(FakeBackend()).execute(w.program).raise_if_failed()        # what the wide portfolio picks runs on the engine
    assert res.peak_fast_bytes <= 2500


@pytest.mark.parametrize("cap", [None, 20000, 3000])
def test_every_registered_policy_produces_a_plan_the_simulator_accepts(cap):
    from dataflow_b200.sim.policies import get_all_policies
    ch = train_chain(L=4, rounds=2)
    lower = sum(t.runtime for t in ch.tasks)
    for name, fn in get_all_policies().items():
        if name == "all_resident" and cap == 3000:
            with pytest.raises(PlanningError):
                fn(ch, cap)
            continue
        planned = fn(ch, cap)
        log = run(planned)
        assert log.makespan >= lower, name
        if cap is not None:
            assert log.peak_fast_memory_bytes <= cap, name


@pytest.mark.parametrize("cap", [6000, 2200])
def test_dispatch_ahead_keeps_results_and_capacity(cap):
    """Launching up to two tasks behind an unfinished one changes when the host dispatches, not what runs."""
    r = pressurefit(train_chain(), cap)
    prog = from_sim_chain(r.chain)
    strict = Engine(FakeBackend()).execute(prog).raise_if_failed()
    ahead = Engine(FakeBackend()).execute(prog, dispatch_ahead=2).raise_if_failed()
    assert ahead.peak_fast_bytes <= cap          # (virtual time is only meaningful under strict pacing: no makespan claim)
    assert [iv.name for iv in ahead.trace.by_track("compute")] == [iv.name for iv in strict.trace.by_track("compute")]


def test_static_placement_packs_lifetimes_and_the_engine_honours_it():
    """Dry-run lifetimes -> offsets with no overlap in (time, address); a run with the placement allocates exactly there,
    escapes nothing, and reproduces the dynamic run's schedule and peak."""
    import dataclasses
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import plan_at_budget
    from dataflow_b200.runtime import Engine, FakeBackend, Session, synthetic_resolver
    from dataflow_b200.runtime.placement import PlacementError, compute_placement, peak_live_bytes, record_lifetimes
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), n_layers=4)
    planned = plan_at_budget(fam, cfg, int(0.016 * (1 << 30)), leeway_bytes=0)
    prog = planned.program
    lts = record_lifetimes(prog)
    assert len(lts) > 40 and any(lt.occurrence > 0 for lt in lts)            # something was evicted and came back
    pl = compute_placement(lts)
    for i, a in enumerate(lts):
        for b in lts[i + 1:]:
            if a.start < b.end and b.start < a.end:
                oa, ob = pl.offsets[(a.object_id, a.occurrence)], pl.offsets[(b.object_id, b.occurrence)]
                assert oa + a.size <= ob or ob + b.size <= oa
    peak = peak_live_bytes(lts)
    assert peak <= pl.top <= 1.15 * peak                                    # little is lost to packing
    with pytest.raises(PlacementError):
        compute_placement(lts, capacity=peak - 512)
    be = FakeBackend()
    sess = Session(be)
    sess.native.ensure_pools(pl.top, 0, 0.0)
    eng = Engine(be, session=sess)
    base = Engine(FakeBackend()).execute(prog, synthetic_resolver)
    res = eng.execute(prog, synthetic_resolver, manage_pools=False, record_allocs=True, placement=pl)
    res.raise_if_failed()
    assert res.placement_escapes == 0 and res.slab_overflows == 0
    assert res.makespan_us == pytest.approx(base.makespan_us) and res.peak_fast_bytes == base.peak_fast_bytes
    slab_base = sess.native.fast_slab()[0]
    seen = {}
    for oid, size, ptr, kind in res.stats["allocs"]:
        if kind == 1:
            k = seen.get(oid, 0)
            seen[oid] = k + 1
            assert ptr - slab_base == pl.offsets[(oid, k)]


def test_placement_escape_valve_keeps_a_run_alive_when_the_plan_does_not_match():
    """A placement whose offsets collide (here: everything at offset 0) cannot be honoured; the engine falls back to the
    dynamic allocator for the colliding buffers, counts the escapes, and finishes with the same result."""
    from dataflow_b200.models.families import resolve_family
    from dataflow_b200.run.driver import plan_at_budget
    from dataflow_b200.runtime import Engine, FakeBackend, synthetic_resolver
    from dataflow_b200.runtime.placement import Placement, record_lifetimes
    fam = resolve_family("llama3")
    prog = plan_at_budget(fam, fam.presets["tiny"](), None).program
    lts = record_lifetimes(prog)
    bad = Placement({(lt.object_id, lt.occurrence): 0 for lt in lts}, 0, lts)
    base = Engine(FakeBackend()).execute(prog, synthetic_resolver)
    res = Engine(FakeBackend()).execute(prog, synthetic_resolver, placement=bad)
    res.raise_if_failed()
    assert res.placement_escapes > 0
    assert res.makespan_us == pytest.approx(base.makespan_us) and res.peak_fast_bytes == base.peak_fast_bytes


# ---------------------------------------------------------------- pressure-eviction valve
def test_pressure_eviction_valve_pages_an_unplanned_program_through_a_small_memory():
    """No directives at all and a capacity that cannot hold what the chain leaves resident: without the valve this is a
    deadlock; with it the engine evicts the resident whose next use is farthest (writing it back first when it has no
    current backing copy), reloads it in front of the task that reads it, and counts every eviction."""
    from dataflow_b200.core import ObjectSpec, OutputSpec, Program, TaskSpec
    p = Program("paging",
                (ObjectSpec("A", 10, "fast"), ObjectSpec("R", 40, "fast")),
                (TaskSpec("t0", inputs=("A",), outputs=(OutputSpec("Z", 60),), runtime_us=5.0),
                 TaskSpec("t1", inputs=("A", "R"), outputs=(OutputSpec("W", 10),), runtime_us=5.0),
                 TaskSpec("t2", inputs=("Z", "W"), outputs=(OutputSpec("V", 10),), runtime_us=5.0)),
                final_locations={"V": "fast"}, fast_memory_capacity=100, backing_memory_capacity=1000,
                bandwidth_from_slow=10, bandwidth_to_slow=10)
    res = Engine(FakeBackend()).execute(p, record_events=True)
    res.raise_if_failed()
    assert res.pressure_evictions >= 2                    # R made room for Z, then Z made room for R
    assert res.peak_fast_bytes <= 100
    kinds = [e.kind for e in res.trace.events]
    assert "evict_writeback" in kinds and "evict_reload" in kinds
    names = [iv.name for iv in res.trace.intervals]
    # R leaves before t0 can write Z, and is back before t1 reads it
    assert names.index("to_slow:R") < names.index("t0") < names.index("from_slow:R") < names.index("t1")


def test_pressure_eviction_valve_survives_a_plan_made_for_a_larger_memory():
    """A planned chain run in less memory than it was planned for (the realised state has left the plan): the valve keeps
    it alive inside the smaller capacity, the final locations still hold, and the same plan in its own capacity needs no
    eviction at all."""
    import dataclasses
    r = pressurefit(train_chain(L=4, rounds=2), 3000)
    prog = from_sim_chain(r.chain)
    calm = Engine(FakeBackend()).execute(prog).raise_if_failed()
    assert calm.pressure_evictions == 0
    tight = dataclasses.replace(prog, fast_memory_capacity=int(calm.peak_fast_bytes * 0.93))
    res = Engine(FakeBackend()).execute(tight)
    res.raise_if_failed()
    assert res.pressure_evictions > 0 and res.peak_fast_bytes <= tight.fast_memory_capacity
    assert res.makespan_us >= calm.makespan_us
    # a task whose own inputs and outputs exceed the capacity still ends in a reported deadlock, not a hang
    impossible = dataclasses.replace(prog, fast_memory_capacity=1000)
    bad = Engine(FakeBackend()).execute(impossible)
    assert bad.outcome.error_kind in ("DeadlockError", "LedgerError")


def test_annotators_see_every_task_and_transfer_under_renamed_labels():
    """A recording annotator gets one balanced range per task launch and per transfer issue; ``annotate_rename`` changes the
    displayed names only (the run's trace keeps the program's ids)."""
    from dataflow_b200.runtime.annotate import RecordingAnnotator
    r = pressurefit(train_chain(L=3, rounds=1), 2500)
    prog = from_sim_chain(r.chain)
    rec = RecordingAnnotator()
    res = Engine(FakeBackend()).execute(prog, annotator=rec, annotate_rename=lambda n, k: f"[{k}] {n}").raise_if_failed()
    assert rec.depth_ok()
    assert rec.names("[task] ") == [f"[task] {t.id}" for t in prog.tasks]
    moved = [i.name for i in res.trace.intervals if i.track in ("from_slow", "to_slow")]
    assert sorted(rec.names("[transfer] ")) == sorted(f"[transfer] {n}" for n in moved) and moved
    assert all(not i.name.startswith("[") for i in res.trace.intervals)
    plain = Engine(FakeBackend()).execute(prog).raise_if_failed()
    assert plain.makespan_us == res.makespan_us


def test_malformed_plans_end_in_typed_errors_never_in_a_crash():
    """Random single edits of valid plans (directives dropped, added, doubled, moved) on the virtual-time backend: the
    engine either runs the program (its valves absorb what is only a capacity problem) or refuses it with one of its typed
    errors; whatever the simulator accepts, the engine accepts."""
    import random
    from dataclasses import replace
    from dataflow_b200.sim import TransferTrigger as T
    from dataflow_b200.sim.errors import SimulationError
    from dataflow_b200.sim.policies import get_all_policies
    rng = random.Random(21)
    known = {"ExecutionError", "DeadlockError", "FinalLocationError", "ValidationError", "CapacityError"}
    seen = set()
    for pol, cap in (("lookahead", 3000), ("max_reduce", 2600)):
        good = get_all_policies()[pol](train_chain(L=4, rounds=2), cap)
        objs = list(good.sizes())
        for _ in range(120):
            tasks = list(good.tasks)
            i = rng.randrange(len(tasks))
            t = tasks[i]
            kind = rng.choice(["drop_prefetch", "drop_release", "add_release", "add_prefetch", "add_offload", "dup_release"])
            if kind == "drop_prefetch" and t.prefetch_after:
                t = replace(t, prefetch_after=t.prefetch_after[1:])
            elif kind == "drop_release" and t.releases_after:
                t = replace(t, releases_after=t.releases_after[1:])
            elif kind == "add_release":
                t = replace(t, releases_after=t.releases_after + [rng.choice(objs)])
            elif kind == "add_prefetch":
                t = replace(t, prefetch_after=t.prefetch_after + [T(rng.choice(objs))])
            elif kind == "add_offload":
                t = replace(t, offload_after=t.offload_after + [T(rng.choice(objs))])
            elif kind == "dup_release" and t.releases_after:
                t = replace(t, releases_after=t.releases_after + [t.releases_after[0]])
            else:
                continue
            tasks[i] = t
            bad = replace(good, tasks=tasks)
            try:
                run(bad, validate=False)
                sim_ok = True
            except SimulationError:
                sim_ok = False
            try:
                res = Engine(FakeBackend()).execute(from_sim_chain(bad))
                outcome = "ok" if res.outcome.ok else res.outcome.error_kind
            except Exception as e:       # noqa: BLE001  (validation refuses before the engine starts)
                outcome = type(e).__name__
            seen.add(outcome)
            assert outcome == "ok" or outcome in known, (kind, outcome)
            if sim_ok:
                assert outcome == "ok", (kind, outcome)
    assert "ok" in seen and len(seen) >= 3
