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
