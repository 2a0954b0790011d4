"""Chains at the edges of the schema through every planner, the validator and the engine: nothing to do, sizes of zero, no
bandwidth, no capacity, objects nobody reads, outputs born in backing memory."""
import pytest

from dataflow_b200.core import from_sim_chain
from dataflow_b200.runtime import Engine, FakeBackend
from dataflow_b200.sim import Object, OutputAlloc, Task, TaskChain, run
from dataflow_b200.sim.policies import PlanningError, get_all_policies
from dataflow_b200.sim.validate import chain_problems

CASES = {
    "empty": TaskChain([], [], {}, 100, None, 10, 10),
    "one task, nothing else": TaskChain([], [Task("a", [], [], 5)], {}, 100, None, 10, 10),
    "zero-size objects": TaskChain([Object("z", 0, "backing"), Object("x", 10, "fast")],
                                   [Task("a", ["x", "z"], [OutputAlloc("y", 0)], 0.0), Task("b", ["y", "z"], [], 1)], {"z": "backing"}, 100, None, 10, 10),
    "no capacity": TaskChain([Object("w", 50, "backing"), Object("x", 10, "fast")], [Task("a", ["x"], [], 1), Task("b", ["x", "w"], [], 1)],
                             {"w": "backing"}, None, None, 10, 10),
    "unused initial objects": TaskChain([Object("u", 50, "backing"), Object("v", 20, "fast"), Object("x", 10, "fast")], [Task("a", ["x"], [], 1)],
                                        {"v": "backing"}, 100, None, 10, 10),
    "output never read, final fast": TaskChain([Object("x", 10, "fast")], [Task("a", ["x"], [OutputAlloc("y", 20)], 1), Task("b", ["x"], [], 1)],
                                               {"y": "fast"}, 100, None, 10, 10),
    "output born in backing": TaskChain([Object("x", 10, "fast")],
                                        [Task("a", ["x"], [OutputAlloc("y", 20, "backing")], 1), Task("b", ["x"], [], 1), Task("c", ["y"], [], 1)],
                                        {}, 100, None, 10, 10),
}
# what is known not to be handled: Lookahead leaves an unread initial fast object that must end in backing memory to PressureFit
KNOWN = {("unused initial objects", "lookahead")}


@pytest.mark.parametrize("case", sorted(CASES))
def test_every_planner_handles_the_edge(case):
    chain = CASES[case]
    for name, plan in get_all_policies().items():
        try:
            planned = plan(chain, chain.fast_memory_capacity)
        except PlanningError:
            assert (case, name) in KNOWN, (case, name)
            continue
        assert chain_problems(planned) == [], (case, name)
        log = run(planned)
        res = Engine(FakeBackend()).execute(from_sim_chain(planned)).raise_if_failed()
        assert res.makespan_us == pytest.approx(log.makespan), (case, name)


def test_a_chain_without_bandwidth_is_planned_only_by_keeping_everything_resident():
    ch = TaskChain([Object("w", 50, "backing"), Object("x", 10, "fast")], [Task("a", ["x"], [], 1), Task("b", ["x", "w"], [], 1)], {}, 100, None, None, None)
    outcomes = {}
    for name, plan in get_all_policies().items():
        try:
            planned = plan(ch, 100)
            assert not [iv for iv in run(planned).task_intervals if iv.track != "compute"], name      # nothing moves
            outcomes[name] = "resident"
        except PlanningError as e:
            outcomes[name] = "refused"
            assert "bandwidth" in str(e) or "fits" in str(e), (name, e)
    assert outcomes["all_resident"] == outcomes["max_reduce"] == outcomes["min_grow"] == "resident"
    tight = {}
    for name in ("max_reduce", "min_grow", "roundtrip"):                # with too little room something would have to move: refused, by name
        with pytest.raises(PlanningError):
            get_all_policies()[name](ch, 55)
