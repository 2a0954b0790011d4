"""One invalid chain per rule of the static validator, each made by one edit of a valid annotated chain, plus the property that
what planners emit passes every stage."""
from dataclasses import replace

import pytest

from chains import train_chain
from dataflow_b200.sim import Object, OutputAlloc, Task, TaskChain, TransferTrigger, ValidationError, run, validate_chain
from dataflow_b200.sim.validate import RULES, chain_problems, check_capacity, validate_planning_input

T = TransferTrigger


def base() -> TaskChain:
    """w lives in backing and is fetched for b; y is parked in backing across b and fetched back for c; z must end in backing."""
    return TaskChain(
        [Object("w", 100, "backing", "weight"), Object("x", 10, "fast"), Object("k", 8, "fast"), Object("k", 8, "backing")],
        [Task("a", ["x"], [OutputAlloc("y", 20)], 5, prefetch_after=[T("w")], offload_after=[T("y")]),
         Task("b", ["x", "w"], [OutputAlloc("u", 20)], 5, releases_after=["w"], prefetch_after=[T("y")]),
         Task("c", ["y", "u", "k"], [OutputAlloc("z", 20)], 5, mutates_inputs=["u"], releases_after=["y", "u", "k"], offload_after=[T("z")]),
         Task("d", ["x"], [], 1, releases_after=["x"])],
        {"z": "backing", "k": "backing"}, 200, 400, 10, 10)


def edit(i: int, **kw):
    def f(ch: TaskChain) -> TaskChain:
        tasks = list(ch.tasks)
        tasks[i] = replace(tasks[i], **kw)
        return replace(ch, tasks=tasks)
    return f


def both(*fs):
    def f(ch):
        for g in fs:
            ch = g(ch)
        return ch
    return f


CASES = {
    # ids
    "bad-location": lambda ch: replace(ch, initial_memory=ch.initial_memory + [Object("q", 1, "disk")]),
    "negative-size": edit(0, workspace_bytes=-1),
    "duplicate-initial-object": lambda ch: replace(ch, initial_memory=ch.initial_memory + [Object("x", 10, "fast")]),
    "duplicate-task-id": lambda ch: replace(ch, tasks=ch.tasks + [Task("a", ["x"], [], 1)]),
    "duplicate-input": edit(3, inputs=["x", "x"]),
    "unknown-input": edit(0, inputs=["x", "nope"]),
    "output-reuses-id": edit(1, outputs=[OutputAlloc("y", 20)]),
    "mutation-not-an-input": edit(1, mutates_inputs=["k"]),
    "unknown-release-object": edit(0, releases_after=["u"]),           # u exists only from task b on
    "unknown-transfer-object": edit(0, prefetch_after=[T("w"), T("z")]),
    "unknown-final-object": lambda ch: replace(ch, final_locations={**ch.final_locations, "ghost": "fast"}),
    "missing-bandwidth": lambda ch: replace(ch, bandwidth_to_slow=None),
    # transfers
    "prefetch-already-resident": edit(0, prefetch_after=[T("w"), T("x")]),
    # x has only a fast copy; a drops it, b asks for it back
    "prefetch-without-backing-copy": both(edit(0, releases_after=["x"]), edit(1, inputs=["w"], prefetch_after=[T("y"), T("x")]),
                                          edit(3, inputs=[], releases_after=[])),
    "offload-not-resident": edit(0, offload_after=[T("y"), T("w")], prefetch_after=[]),
    "duplicate-transfer": edit(0, prefetch_after=[T("w"), T("w")]),
    "release-and-offload": edit(2, releases_after=["y", "u", "k", "z"]),
    "release-not-resident": edit(0, releases_after=["w"], prefetch_after=[]),
    "duplicate-release": edit(3, releases_after=["x", "x"]),
    # lifetimes
    # y was offloaded by a and never comes back for c
    "input-not-resident": both(edit(1, prefetch_after=[]), edit(2, releases_after=["u", "k"])),
    # w comes back after its only reader has run
    "prefetch-never-used": edit(2, prefetch_after=[T("w")]),
    # u is read by c and was never offloaded
    "release-loses-data": both(edit(1, releases_after=["w", "u"]), edit(2, releases_after=["y", "k"])),
    "final-not-on-backing": edit(2, offload_after=[]),
    "final-backing-stale": edit(2, mutates_inputs=["u", "k"], releases_after=["y", "u"]),
    "final-not-on-fast": lambda ch: replace(ch, final_locations={**ch.final_locations, "w": "fast"}),
    # capacity
    "initial-overflow": lambda ch: replace(ch, backing_memory_capacity=50),
    "task-cannot-fit": lambda ch: replace(ch, fast_memory_capacity=60),
}


def test_the_base_chain_is_valid_and_runs():
    ch = validate_chain(base())
    assert chain_problems(ch) == []
    assert run(ch).makespan > 0


@pytest.mark.parametrize("rule", sorted(CASES))
def test_each_rule_is_reported_by_its_code(rule):
    bad = CASES[rule](base())
    with pytest.raises(ValidationError) as e:
        validate_chain(bad)
    assert rule in e.value.rules, e.value.problems
    assert all(p.rule in RULES for p in e.value.found)
    assert all(str(p).startswith(p.rule + ":") for p in e.value.found)


def test_every_rule_has_a_case():
    assert set(CASES) == set(RULES) - {"already-planned"}


def test_a_stage_reports_all_of_its_problems_with_task_and_object():
    bad = edit(0, inputs=["x", "nope"])(edit(1, mutates_inputs=["k"])(base()))
    found = chain_problems(bad)
    assert [(p.rule, p.task, p.obj) for p in found] == [("unknown-input", "a", "nope"), ("mutation-not-an-input", "b", "k")]
    # a later stage does not run on a chain an earlier one rejected: the capacity problem stays hidden behind the id problems
    worse = replace(bad, fast_memory_capacity=60)
    assert {p.rule for p in chain_problems(worse)} == {"unknown-input", "mutation-not-an-input"}
    assert {p.rule for p in check_capacity(worse)} == {"task-cannot-fit"}


def test_release_then_prefetch_in_one_task_drops_and_refetches():
    ch = TaskChain([Object("w", 40, "backing"), Object("x", 1, "fast")],
                   [Task("p", ["x"], [], 1, prefetch_after=[T("w")]),
                    Task("a", ["w"], [], 5, releases_after=["w"], prefetch_after=[T("w")]),
                    Task("b", ["x"], [], 50),
                    Task("c", ["w"], [], 5, releases_after=["w"])], {}, 100, None, 10, 10)
    validate_chain(ch)
    log = run(ch)
    assert [iv.task_id for iv in log.task_intervals if iv.track == "from_slow"] == ["from_slow:w", "from_slow:w#1"]


def test_planning_input_must_be_bare_and_feasible():
    with pytest.raises(ValidationError) as e:
        validate_planning_input(base())
    assert e.value.rules == ["already-planned"]
    bare = base().bare()
    validate_planning_input(bare)
    with pytest.raises(ValidationError) as e:
        validate_planning_input(replace(bare, fast_memory_capacity=60))
    assert e.value.rules == ["task-cannot-fit"] and {p.task for p in e.value.found} == {"b", "c"}


@pytest.mark.parametrize("cap", [2500, 3000, 6000])
def test_what_every_policy_emits_passes_every_stage(cap):
    from dataflow_b200.sim.policies import get_all_policies
    for name, policy in get_all_policies().items():
        try:
            planned = policy(train_chain(L=4, rounds=2), cap)
        except Exception as exc:                          # a policy may find a capacity infeasible; that is not this test's subject
            assert "Planning" in type(exc).__name__ or "Validation" in type(exc).__name__, (name, exc)
            continue
        assert chain_problems(planned) == [], name


def test_the_command_line_validates_plans_simulates_and_compares(tmp_path, capsys):
    from dataflow_b200.sim.__main__ import main
    bare = tmp_path / "chain.json"
    planned = tmp_path / "planned.json"
    train_chain(L=4, rounds=2).save(bare)
    assert main(["validate", str(bare), "--planning-input"]) == 0
    assert main(["plan", str(bare), "--policy", "max_reduce", "--capacity-gib", str(3000 / 2 ** 30), "-o", str(planned)]) == 0
    assert "x compute-only" in capsys.readouterr().out and planned.exists()
    assert main(["validate", str(planned)]) == 0 and main(["validate", str(planned), "--planning-input"]) == 1      # it carries a plan now
    assert "already-planned" in capsys.readouterr().out
    assert main(["simulate", str(planned), "--stalls"]) == 0
    out = capsys.readouterr().out
    assert '"makespan_us"' in out and "from_slow: busy" in out
    assert main(["compare", str(bare), "--capacity-gib", str(3000 / 2 ** 30), "--policies", "max_reduce,lookahead,all_resident"]) == 0
    table = capsys.readouterr().out.strip().splitlines()
    assert len(table) == 3 and table[-1].startswith("all_resident") and "no plan" in table[-1]        # best first, failures last
    assert main(["plan", str(bare), "--policy", "nope"]) == 1 and main(["plan", str(bare), "--capacity-gib", "0.0000001"]) == 1
    bad = base()
    bad = replace(bad, tasks=[replace(bad.tasks[0], inputs=["x", "ghost"])] + bad.tasks[1:])
    bad.save(tmp_path / "bad.json")
    assert main(["validate", str(tmp_path / "bad.json")]) == 1
    assert "unknown-input" in capsys.readouterr().out


FIXTURES = __import__("os").path.join(__import__("os").path.dirname(__import__("os").path.abspath(__file__)), "fixtures", "invalid_chains")


def test_the_invalid_chains_on_disk_are_the_cases_above_and_the_tools_refuse_them(tmp_path, capsys):
    """One JSON file per rule under ``tests/fixtures/invalid_chains`` (for the command line, the HTTP route and anything else
    that reads chains from files).  ``DATAFLOW_WRITE_FIXTURES=1`` rewrites them from the cases of this module."""
    import json
    import os
    from dataflow_b200.sim.__main__ import main
    if os.environ.get("DATAFLOW_WRITE_FIXTURES") == "1":
        os.makedirs(FIXTURES, exist_ok=True)
        for rule, make in CASES.items():
            with open(os.path.join(FIXTURES, rule + ".json"), "w") as f:
                json.dump({"rule": rule, "meaning": RULES[rule], "chain": make(base()).to_dict()}, f, indent=1)
        with open(os.path.join(FIXTURES, "valid.json"), "w") as f:
            json.dump({"rule": None, "meaning": "the chain every case is one edit away from", "chain": base().to_dict()}, f, indent=1)
    names = sorted(n[:-5] for n in os.listdir(FIXTURES) if n.endswith(".json"))
    assert names == sorted(list(CASES) + ["valid"])
    for rule in CASES:
        with open(os.path.join(FIXTURES, rule + ".json")) as f:
            doc = json.load(f)
        chain = TaskChain.from_dict(doc["chain"])
        assert chain == CASES[rule](base()), rule                       # the file is what the case builds
        assert rule in {p.rule for p in chain_problems(chain)}, rule
        path = tmp_path / (rule + ".json")
        chain.save(path)
        assert main(["validate", str(path)]) == 1 and rule in capsys.readouterr().out
    with open(os.path.join(FIXTURES, "valid.json")) as f:
        assert chain_problems(TaskChain.from_dict(json.load(f)["chain"])) == []


def test_what_the_simulator_refuses_for_its_structure_the_validator_refuses_first():
    """Random single edits of valid plans (a directive dropped, added, doubled, moved later, a release turned into an offload).
    Whenever the simulator rejects the edited chain for a reason other than capacity at run time, the static validator
    has already rejected it; the other way round is allowed (the validator also refuses what the simulator tolerates, like
    a transfer listed twice)."""
    import random
    from dataflow_b200.sim.errors import SimulationCapacityError, SimulationError
    from dataflow_b200.sim.policies import get_all_policies
    rng = random.Random(5)
    pols = get_all_policies()

    def mutate(ch):
        tasks = list(ch.tasks)
        i = rng.randrange(len(tasks))
        t = tasks[i]
        objs = list(ch.sizes())
        kind = rng.choice(["drop_prefetch", "drop_offload", "add_release", "add_prefetch", "add_offload", "dup_prefetch", "dup_release", "move_prefetch_late", "swap"])
        if kind == "drop_prefetch" and t.prefetch_after:
            t = replace(t, prefetch_after=t.prefetch_after[1:])
        elif kind == "drop_offload" and t.offload_after:
            t = replace(t, offload_after=t.offload_after[1:])
        elif kind == "add_release":
            t = replace(t, releases_after=t.releases_after + [rng.choice(objs)])
        elif kind == "add_prefetch":
            t = replace(t, prefetch_after=t.prefetch_after + [T(rng.choice(objs))])
        elif kind == "add_offload":
            t = replace(t, offload_after=t.offload_after + [T(rng.choice(objs))])
        elif kind == "dup_prefetch" and t.prefetch_after:
            t = replace(t, prefetch_after=t.prefetch_after + [t.prefetch_after[0]])
        elif kind == "dup_release" and t.releases_after:
            t = replace(t, releases_after=t.releases_after + [t.releases_after[0]])
        elif kind == "move_prefetch_late" and t.prefetch_after and i + 2 < len(tasks):
            tr = t.prefetch_after[0]
            t = replace(t, prefetch_after=t.prefetch_after[1:])
            j = rng.randrange(i + 1, len(tasks))
            tasks[j] = replace(tasks[j], prefetch_after=tasks[j].prefetch_after + [tr])
        elif kind == "swap" and t.releases_after:
            t = replace(t, releases_after=t.releases_after[1:], offload_after=t.offload_after + [T(t.releases_after[0])])
        else:
            return None
        tasks[i] = t
        return replace(ch, tasks=tasks)

    refused_by_both = tolerated = 0
    for L, R, cap, pol in ((4, 2, 3000, "lookahead"), (5, 2, 2600, "max_reduce"), (3, 3, 2400, "min_grow")):
        good = pols[pol](train_chain(L=L, rounds=R), cap)
        assert chain_problems(good) == []
        for _ in range(250):
            bad = mutate(good)
            if bad is None:
                continue
            static = chain_problems(bad)
            try:
                run(bad, validate=False)
                structural = None
            except SimulationCapacityError as e:
                structural = None if e.kind in ("fast-deadlock", "stuck-transfers") else e       # memory ran out at run time: not a static matter
            except SimulationError as e:
                structural = e
            if structural is not None:
                assert static, f"{pol}: the simulator refused ({structural}) what the validator passed"
                refused_by_both += 1
            elif static:
                tolerated += 1
    assert refused_by_both > 150 and tolerated > 10
