import pytest

from dataflow_b200.sim import (Object, OutputAlloc, SimulationCapacityError, SimulationError, Task, TaskChain,
                               TransferTrigger, ValidationError, run)


def iv(log):
    return {i.task_id: (i.start, i.end) for i in log.task_intervals}


def test_prefetch_then_compute_and_offload():
    ch = TaskChain([Object("w", 100, "backing"), Object("x", 10, "fast")],
                   [Task("a", ["x"], [OutputAlloc("y", 20)], 5, prefetch_after=[TransferTrigger("w")]),
                    Task("b", ["y", "w"], [OutputAlloc("z", 20)], 5, releases_after=["y", "w"], offload_after=[TransferTrigger("z")])],
                   {"z": "backing"}, 200, None, 10, 10)
    log = run(ch)
    t = iv(log)
    assert t["from_slow:w"] == (5, 15) and t["b"] == (15, 20) and t["to_slow:z"] == (20, 22)
    assert log.peak_fast_memory_bytes == 150 and log.stalls["b"] == 10


def test_transfer_charged_at_start_and_head_blocks():
    # cap leaves room for only one of the two prefetched objects until 'a' releases x
    ch = TaskChain([Object("p", 60, "backing"), Object("q", 60, "backing"), Object("x", 50, "fast")],
                   [Task("a", ["x"], [], 10, prefetch_after=[TransferTrigger("p"), TransferTrigger("q")]),
                    Task("b", ["x"], [], 100, releases_after=["x"]),
                    Task("c", ["p", "q"], [], 5, releases_after=["p", "q"])],
                   {}, 130, None, 10, 10)
    t = iv(run(ch))
    assert t["from_slow:p"] == (10, 16)
    assert t["from_slow:q"][0] == 110       # blocked until x is released at the end of b
    assert t["c"][0] == 116


def test_deferred_prefetch_waits_for_offload():
    ch = TaskChain([Object("x", 40, "fast")],
                   [Task("a", ["x"], [], 5, mutates_inputs=["x"], offload_after=[TransferTrigger("x")], prefetch_after=[TransferTrigger("x")]),
                    Task("b", ["x"], [], 5, releases_after=["x"])],
                   {}, 100, None, 10, 10)
    t = iv(run(ch))
    assert t["to_slow:x"] == (5, 9) and t["from_slow:x"] == (9, 13) and t["b"][0] == 13


def test_dead_everywhere_release_frees_backing():
    ch = TaskChain([Object("x", 40, "backing")],
                   [Task("p", [], [], 1, prefetch_after=[TransferTrigger("x")]),
                    Task("a", ["x"], [], 5, releases_after=["x"])], {}, 100, 40, 10, 10)
    log = run(ch, snapshots=True)
    assert log.events[-1].backing_bytes == 0


def test_tie_order_from_slow_before_task_end():
    ch = TaskChain([Object("w", 50, "backing"), Object("x", 10, "fast")],
                   [Task("a", ["x"], [], 5, prefetch_after=[TransferTrigger("w", 5.0)]),
                    Task("b", ["x"], [], 5),
                    Task("c", ["w"], [], 1)], {}, 100, None, 10, 10)
    t = iv(run(ch))
    assert t["c"][0] == 10      # transfer ending exactly when b ends is visible to c immediately


def test_workspace_is_charged_only_while_running():
    ch = TaskChain([Object("x", 10, "fast")], [Task("a", ["x"], [], 5, workspace_bytes=80), Task("b", ["x"], [OutputAlloc("y", 85)], 5)],
                   {}, 100, None, None, None)
    assert run(ch).peak_fast_memory_bytes == 95


def test_deadlock_is_an_error_with_context():
    ch = TaskChain([Object("x", 90, "fast")], [Task("a", ["x"], [OutputAlloc("y", 20)], 5)], {}, 100)
    with pytest.raises(SimulationCapacityError) as e:
        run(ch, validate=False)
    assert e.value.kind == "fast-deadlock" and e.value.overage_bytes == 10
    with pytest.raises(ValidationError) as v:            # the static pass sees it before the clock starts
        run(ch)
    assert v.value.rules == ["task-cannot-fit"]


def test_dirty_release_of_needed_object_is_refused():
    ch = TaskChain([Object("x", 10, "fast")],
                   [Task("a", ["x"], [], 5, mutates_inputs=["x"], releases_after=["x"]), Task("b", ["x"], [], 5)], {}, 100, None, 10, 10)
    with pytest.raises(SimulationError):
        run(ch, validate=False)
    with pytest.raises(ValidationError) as v:
        run(ch)
    assert v.value.rules == ["release-loses-data", "input-not-resident"]      # both ends of the same mistake


def test_final_location_checked():
    ch = TaskChain([Object("x", 10, "fast")], [Task("a", ["x"], [], 5, mutates_inputs=["x"])], {"x": "backing"}, 100, None, 10, 10)
    with pytest.raises(SimulationError):
        run(ch, validate=False)
    with pytest.raises(ValidationError) as v:
        run(ch)
    assert v.value.rules == ["final-not-on-backing"]


def test_stall_report_names_the_blocking_transfer():
    from dataflow_b200.sim import build_stall_report
    # W arrives late: the task stalls on it; the report names W and the lane shows the busy time
    ch = TaskChain([Object("W", 400, "backing", "weight"), Object("x", 10, "fast")],
                   [Task("a", ["x"], [OutputAlloc("y", 10)], 50, prefetch_after=[TransferTrigger("W")]),
                    Task("b", ["y", "W"], [OutputAlloc("z", 10)], 50)],
                   {}, 1000, None, 4, 4)
    log = run(ch)
    rep = build_stall_report(ch, log)
    assert rep.stall_us == pytest.approx(100.0)
    (s,) = rep.stalls
    assert s.task_id == "b" and s.waited_inputs == ("W",) and s.blocking_object == "W" and not s.waited_capacity
    assert rep.by_object_type == {"weight": pytest.approx(100.0)}
    assert rep.lanes["from_slow"].transfers == 1 and rep.lanes["from_slow"].busy_us == pytest.approx(100.0)
    assert "waiting for inputs ['W']" in rep.format()


def test_reference_stream_orders_first_touches():
    from dataflow_b200.sim import compute_reference_stream, next_ref_time
    from dataflow_b200.sim.reference_stream import stall_free_starts
    tasks = [Task("a", ["x"], [OutputAlloc("y", 1)], 10), Task("b", ["y", "w"], [], 5), Task("c", ["x"], [], 1)]
    st = stall_free_starts(tasks)
    refs = compute_reference_stream(tasks, st)
    assert [(r.obj_id, r.ref_t) for r in refs] == [("x", 0.0), ("y", 0.0), ("w", 10.0)]
    assert next_ref_time("x", tasks[1:], st) == 15.0 and next_ref_time("q", tasks, st) is None
