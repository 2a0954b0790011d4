"""The span model, the lane timeline, the shadow, and the planners built on them."""
from dataclasses import replace

import numpy as np
import pytest

from chains import train_chain
from dataflow_b200.sim import Object, OutputAlloc, Task, TaskChain, run
from dataflow_b200.sim.policies import PlanningError, get_all_policies
from dataflow_b200.sim.policies.max_reduce import max_reduce, reduce_to_fit
from dataflow_b200.sim.policies.min_grow import GrowKnobs, grow_static, min_grow
from dataflow_b200.sim.policies.reactive import belady_reactive
from dataflow_b200.sim.policies.roundtrip import build_plan, roundtrip_planner
from dataflow_b200.sim.policies.shadow import Shadow
from dataflow_b200.sim.policies.sliding_window import sliding_window, window_plan
from dataflow_b200.sim.policies.spans import LaneTimeline, SpanPlan, static_minimum
from dataflow_b200.sim.simulator import Simulator, compute_lower_bound
from dataflow_b200.sim.validate import chain_problems


# ------------------------------------------------------------------------------------------------------------------- spans
def test_max_plan_level_is_the_peak_the_simulator_sees():
    ch = train_chain(L=4, rounds=2).bare()
    plan = SpanPlan(ch).fill_max()
    plan.check()
    planned = plan.emit(None)
    assert chain_problems(planned) == []
    log = run(planned)
    # everything placed up front, nothing moved in: the accounting and the run agree on the peak
    assert log.peak_fast_memory_bytes == int(plan.level.max())
    assert not [iv for iv in log.task_intervals if iv.track == "from_slow"]


def test_min_plan_holds_exactly_what_tasks_touch():
    ch = train_chain(L=4, rounds=2).bare()
    plan = SpanPlan(ch).fill_min(0.0)
    plan.check()
    assert np.array_equal(plan.level, static_minimum(ch))
    planned = plan.emit(int(plan.level.max()))
    assert chain_problems(planned) == []


def test_cut_and_add_keep_level_and_spans_consistent():
    ch = train_chain(L=4, rounds=1).bare()
    plan = SpanPlan(ch).fill_max()
    before = plan.level.copy()
    o = "W0"
    (a, b), = plan.spans[o]
    touches = plan.touch[o]
    lo, hi = touches[0] + 1, touches[1] - 1
    plan.cut(o, lo, hi)
    assert plan.spans[o] == [[a, touches[0]], [touches[1], b]]
    assert np.array_equal(before[lo:hi + 1] - plan.level[lo:hi + 1], np.full(hi - lo + 1, float(plan.facts[o].size)))
    plan.add(o, lo, hi)                       # fills the gap: the three pieces merge back into one span
    assert plan.spans[o] == [[a, b]] and np.array_equal(plan.level, before)
    c = plan.copy()
    c.cut(o, lo, hi)
    assert plan.spans[o] == [[a, b]] and np.array_equal(plan.level, before)      # the copy is independent


def test_emit_offloads_only_what_has_no_current_backing_copy():
    # w has a backing copy and is only read: cutting it is a release.  y is produced in fast memory: cutting it is an offload.
    ch = TaskChain([Object("w", 100, "backing", "weight"), Object("x", 10, "fast")],
                   [Task("a", ["x", "w"], [OutputAlloc("y", 50)], 10), Task("b", ["x"], [], 10), Task("c", ["x"], [], 10),
                    Task("d", ["x"], [], 10), Task("e", ["x", "w", "y"], [], 10)], {}, None, None, 10, 10)
    plan = SpanPlan(ch).fill_max()
    plan.cut("w", 1, 2)
    plan.cut("y", 1, 2)
    planned = plan.emit(1000)
    assert planned.tasks[0].releases_after == ["w"] and [t.obj_id for t in planned.tasks[0].offload_after] == ["y"]
    assert sorted(t.obj_id for t in planned.tasks[2].prefetch_after) == ["w", "y"]
    assert chain_problems(planned) == [] and run(planned).makespan >= 50


def test_lane_timeline_books_earliest_and_latest_free_intervals():
    lane = LaneTimeline()
    lane.book(10, 5)                                     # [10, 15)
    lane.book(20, 5)                                     # [20, 25)
    assert lane.earliest(0, 10) == 0 and lane.earliest(0, 11) == 25      # a gap of exactly 10 before the first booking
    assert lane.earliest(12, 3) == 15 and lane.earliest(12, 6) == 25
    assert lane.latest(30, 5) == 25 and lane.latest(22, 5) == 15
    assert lane.latest(22, 6) == 4                       # [15, 20) is too short: the interval before the first booking
    assert lane.latest(22, 6, not_before=5) is None
    assert lane.latest(9, 10) is None and lane.latest(10, 10) == 0


# ------------------------------------------------------------------------------------------------------------------ shadow
def test_shadow_run_replays_to_the_same_log():
    ch = train_chain(L=4, rounds=2)
    planned = get_all_policies()["lookahead"](ch, 3000)
    sh = Shadow(planned.bare(), 3000, initial=planned.initial_memory)
    for t in planned.tasks:
        sh.step()
        for o in t.releases_after:
            sh.release(o)
        for tr in t.offload_after:
            sh.offload(tr.obj_id)
        for tr in t.prefetch_after:
            sh.prefetch(tr.obj_id)
        sh.commit()
    chain, log = sh.result()
    ref = run(planned)
    assert [(iv.task_id, iv.start, iv.end) for iv in log.task_intervals] == [(iv.task_id, iv.start, iv.end) for iv in ref.task_intervals]
    assert log.peak_fast_memory_bytes == ref.peak_fast_memory_bytes
    assert chain.tasks == planned.tasks


def test_shadow_queries_and_fork_independence():
    ch = TaskChain([Object("w", 100, "backing", "weight"), Object("x", 10, "fast")],
                   [Task("a", ["x"], [OutputAlloc("y", 20)], 5), Task("b", ["x", "y"], [], 50), Task("c", ["y", "w"], [], 5)],
                   {}, 200, None, 10, 10)
    sh = Shadow(ch)
    sh.step()
    assert sh.now == 5 and sh.where("w") == (None, "live") and sh.where("y") == ("live", None)
    assert sh.eta("w") is None and sh.needs_offload("y") and sh.needs_offload("x")        # both exist only in fast memory
    sh.prefetch("w")
    stall, err = sh.lookahead(2)                         # on a fork: w arrives during b, c does not wait
    assert err is None and stall == 0
    assert sh.where("w") == (None, "live") and sh.open is not None and sh.idx == 0        # the shadow itself did not move
    sh.commit()
    assert sh.where("w")[0] == "inbound" and sh.eta("w") == 15 and sh.lane_clear("from_slow") == 15
    f = sh.fork()
    f.step(); f.commit()
    assert f.idx == 2 and sh.idx == 1 and f.where("w")[0] == "live" and sh.where("w")[0] == "inbound"
    # without the fetch the last task cannot start, and the probe says so instead of raising
    bare = Shadow(ch)
    bare.step(); bare.commit(); bare.step()
    stall, err = bare.lookahead(1)
    assert stall is None and "not live" in str(err)


# --------------------------------------------------------------------------------------------------------------- planners
NEW = {"max_reduce": max_reduce, "min_grow": min_grow, "roundtrip": roundtrip_planner, "belady_reactive": belady_reactive,
       "sliding_window": sliding_window}


@pytest.mark.parametrize("name", sorted(NEW))
@pytest.mark.parametrize("cap", [None, 20000, 6000, 3000, 2300])
def test_planners_fit_the_capacity_and_emit_valid_chains(name, cap):
    ch = train_chain(L=6, rounds=2)
    try:
        planned = NEW[name](ch, cap)
    except PlanningError:
        assert name == "sliding_window" and cap is not None and cap <= 3000     # the pattern does not know the capacity
        return
    assert chain_problems(planned) == []
    log = run(planned)
    assert log.makespan >= compute_lower_bound(ch)
    if cap is not None:
        assert log.peak_fast_memory_bytes <= cap
    assert [t.bare() for t in planned.tasks] == [t.bare() for t in ch.bare().tasks]      # only directives were added


@pytest.mark.parametrize("name", sorted(NEW))
def test_planners_report_a_capacity_nothing_fits(name):
    ch = train_chain(L=4, rounds=1)
    with pytest.raises((PlanningError, ValueError)):
        NEW[name](ch, 1000)                  # the optimizer task alone holds 1600 bytes


def test_with_room_for_everything_nothing_moves_twice():
    ch = train_chain(L=4, rounds=2)
    lower = compute_lower_bound(ch)
    for name in ("max_reduce", "min_grow", "roundtrip"):
        log = run(NEW[name](ch, 10 ** 9))
        moved_in = [iv.task_id for iv in log.task_intervals if iv.track == "from_slow"]
        assert moved_in == [], name          # placed up front, never fetched
        assert log.makespan <= lower * 1.25, name      # compute plus the write-back of the results at the end


def test_max_reduce_is_pure_accounting_and_monotone_in_capacity():
    ch = train_chain(L=6, rounds=2).bare()
    cuts = []
    for cap in (8000, 5000, 3000):
        plan = SpanPlan(ch).fill_max()
        cuts.append(reduce_to_fit(plan, float(cap)))
        assert float(plan.level.max()) <= cap
        plan.check()
    assert cuts[0] <= cuts[1] <= cuts[2] and cuts[2] > 0
    with pytest.raises(PlanningError, match="nothing resident can be away"):
        reduce_to_fit(SpanPlan(ch).fill_max(), 1500.0)


def test_min_grow_grows_from_the_minimum_and_the_simulator_picks():
    ch = train_chain(L=6, rounds=2).bare()
    least = SpanPlan(ch).fill_min(0.0)
    grown = grow_static(ch, 4000, GrowKnobs(0.0, 1.0, "time"))
    grown.check()
    assert float(grown.level.max()) <= 4000
    # growth only adds residency: every span of the minimum lies inside a span of the grown plan
    for o, spans in least.spans.items():
        for a, b in spans:
            assert any(ga <= a and b <= gb for ga, gb in grown.spans[o]), o
    ms_least = Simulator(least.emit(4000)).run().makespan
    ms_grown = run(min_grow(ch, 4000)).makespan
    assert ms_grown < ms_least


def test_roundtrip_books_trips_only_where_the_level_needs_them():
    ch = train_chain(L=6, rounds=2).bare()
    roomy = build_plan(ch, 10.0 ** 9)
    assert all(len(s) <= 1 for s in roomy.spans.values()) and not roomy.tails
    tight = build_plan(ch, 3000.0)
    assert any(len(s) > 1 for s in tight.spans.values())
    over = tight.level > 3000
    in_flight = np.zeros(tight.n)
    for o, a, b in tight.tails:
        in_flight[a:b + 1] += tight.facts[o].size
    assert not np.any(tight.level - in_flight > 3000)           # over the cap only where an offload is still holding its copy


def test_sliding_window_is_a_fixed_pattern():
    ch = train_chain(L=6, rounds=2).bare()
    p2 = window_plan(ch, 2)
    for o, spans in p2.spans.items():
        touches = p2.touch[o]
        for a, b in spans:
            inside = [u for u in touches if a <= u <= b]
            assert inside and a >= inside[0] - 2 and b <= inside[-1] + 2, (o, a, b)
    wide, narrow = run(sliding_window(ch, 20000, 4)), run(sliding_window(ch, 20000, 1))
    assert wide.peak_fast_memory_bytes > narrow.peak_fast_memory_bytes
    # the same plan whatever the capacity, as long as it fits
    assert sliding_window(ch, 20000, 2).tasks == sliding_window(ch, 10 ** 9, 2).tasks


def test_reactive_fetches_late_and_keeps_the_lane_in_need_order():
    ch = train_chain(L=6, rounds=2)
    planned = belady_reactive(ch, 3000)
    log = run(planned)
    need = {}
    for i, t in enumerate(planned.tasks):
        for o in t.inputs:
            need.setdefault(o, []).append(i)
    # every fetch is fired at most `horizon` tasks before a use of the object, and never after it
    for i, t in enumerate(planned.tasks):
        for tr in t.prefetch_after:
            nxt = [u for u in need[tr.obj_id] if u > i]
            assert nxt and nxt[0] - i <= 64
    assert log.peak_fast_memory_bytes <= 3000


# ------------------------------------------------------------------------------------------- refinement and diagnostics
def test_lead_refinement_fires_a_late_fetch_earlier_and_only_keeps_gains():
    from dataflow_b200.sim import TransferTrigger
    from dataflow_b200.sim.policies.refine import refine_leads
    # w is fetched right before its use: c waits 100 us.  Fired after a instead, it arrives in time.
    ch = TaskChain([Object("w", 1000, "backing", "weight"), Object("x", 10, "fast")],
                   [Task("a", ["x"], [], 60), Task("b", ["x"], [], 60, prefetch_after=[TransferTrigger("w")]),
                    Task("c", ["x", "w"], [], 10, releases_after=["w"])], {}, 2000, None, 10, 10)
    log = run(ch)
    assert log.stalls == {"c": 100.0}
    better, log2, moves = refine_leads(ch, log)
    assert moves == 1 and log2.makespan == log.makespan - 60 and [t.obj_id for t in better.tasks[0].prefetch_after] == ["w"]
    assert chain_problems(better) == []
    # nothing waits any more: a second pass changes nothing and returns the same chain
    again, log3, moves3 = refine_leads(better, log2)
    assert moves3 == 0 and again is better
    # where the earlier fetch does not fit (capacity leaves no room for w during a) the move is refused
    tight = replace(ch, fast_memory_capacity=1010, tasks=[replace(ch.tasks[0], workspace_bytes=900)] + ch.tasks[1:])
    same, _, moves4 = refine_leads(tight)
    assert run(same).makespan <= run(tight).makespan and run(same).peak_fast_memory_bytes <= 1010


def test_pressurefit_diagnostics_describe_the_search():
    from dataflow_b200.sim.policies.pressurefit import pressurefit
    r = pressurefit(train_chain(L=4, rounds=2), 3000)
    d = r.diagnostics()
    assert d.task_count == len(r.chain.tasks) and d.fast_memory_capacity == 3000 and d.forced_peak_bytes == 1600
    assert d.candidate_count == len(r.candidates) and 0 < d.valid_candidate_count <= d.candidate_count
    assert d.selected == r.chosen.name and d.selected_makespan_us == r.makespan and d.spread >= 1.0
    assert {c.status for c in d.candidates} <= {"ok", "repaired", "failed"} and all(c.wall_s >= 0 for c in d.candidates)
    text = d.format(4)
    assert "candidates valid" in text and d.selected in text and "x lower bound" in text


def test_pressurefit_repairs_locally_before_it_shrinks_the_capacity():
    import importlib
    pf = importlib.import_module("dataflow_b200.sim.policies.pressurefit")
    ch = train_chain(L=6, rounds=2).bare()
    spec = next(s for s in pf.RESIDENCY_SPECS if s.name == "belady")
    rule = next(r for r in pf.PREFETCH_RULES if r.name == "window_2")
    planned, log, repairs, err = pf._verify_candidate(ch, 2600, spec, rule)
    only_global = pf._verify_candidate(ch, 2600, spec, rule, local_repairs=0)
    assert planned is not None and log.peak_fast_memory_bytes <= 2600
    if only_global[0] is not None:
        assert log.makespan <= only_global[1].makespan * 1.05


@pytest.mark.parametrize("name", sorted(NEW))
@pytest.mark.parametrize("cap", [6000, 3000])
def test_the_engine_reproduces_the_simulated_log_of_every_planner(name, cap):
    from dataflow_b200.core import from_sim_chain
    from dataflow_b200.runtime import Engine, FakeBackend, compare_to_sim_eventlog
    try:
        planned = NEW[name](train_chain(L=6, rounds=2), cap)
    except PlanningError:
        pytest.skip("the fixed pattern does not fit this capacity")
    log = run(planned)
    res = Engine(FakeBackend()).execute(from_sim_chain(planned)).raise_if_failed()
    assert compare_to_sim_eventlog(res.trace, log) == []
    assert res.makespan_us == log.makespan and res.peak_fast_bytes <= cap


def test_random_chains_every_planner_emits_valid_plans_the_engine_reproduces():
    """A small sample of the fuzz that was run over thousands of plans while the planners were written: random forward /
    backward chains and training chains, capacities from a hair above the largest task's own need to unbounded; every plan
    passes the static validator, stays under its capacity, and runs on the virtual-time engine to the simulator's log."""
    import importlib.util
    import os
    import random
    from dataflow_b200.core import from_sim_chain
    from dataflow_b200.runtime import Engine, FakeBackend, compare_to_sim_eventlog
    from dataflow_b200.sim.validate import ValidationError
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("oracle_tool", os.path.join(root, "tools", "bench", "pressurefit_exact_oracle.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    rng = random.Random(11)
    pols = {k: v for k, v in get_all_policies().items() if k != "all_resident"}
    checked = 0
    for c in range(10):
        chain = (replace(tool.random_chain(rng, rng.choice([4, 6, 8, 10])).bare(), fast_memory_capacity=None) if c % 2
                 else train_chain(L=rng.choice([2, 3, 5]), rounds=rng.choice([1, 2, 3])).bare())
        need = float(static_minimum(chain).max())
        for frac in (1.02, 1.5, None):
            cap = None if frac is None else int(need * frac)
            for name, fn in pols.items():
                try:
                    planned = fn(chain, cap)
                except (PlanningError, ValidationError):
                    assert name == "sliding_window", (name, c, frac)        # only the capacity-blind pattern may give up
                    continue
                assert chain_problems(planned) == [], (name, c, frac)
                log = run(planned)
                assert cap is None or log.peak_fast_memory_bytes <= cap, (name, c, frac)
                res = Engine(FakeBackend()).execute(from_sim_chain(planned)).raise_if_failed()
                assert compare_to_sim_eventlog(res.trace, log) == [] and res.makespan_us == log.makespan, (name, c, frac)
                checked += 1
    assert checked > 200
