import json

import pytest

from dataflow_b200.core import (ObjectSpec, OutputSpec, Program, RecomputeOption, RecomputeRewrite, TaskSpec,
                                TensorMeta, TransferDirective, ValidationError, collect_problems, from_sim_chain,
                                load_program, program_content_id, program_from_dict, program_to_dict, save_program,
                                to_sim_chain, to_webapp_program, validate_program)


def small_program(**kw):
    return Program(
        "t", initial_objects=(ObjectSpec("w", 100, "backing", "parameter", persistent=True), ObjectSpec("x", 10, "fast", "input")),
        tasks=(TaskSpec("a", inputs=("x",), outputs=(OutputSpec("y", 20),), runtime_us=5,
                        prefetch_after=(TransferDirective("w"),), compute_block_key="k", block_params={"layer": 0}),
               TaskSpec("b", inputs=("y", "w"), outputs=(OutputSpec("z", 20),), runtime_us=5, releases_after=("y", "w"),
                        offload_after=(TransferDirective("z", 3.0),))),
        final_locations={"z": "backing"}, fast_memory_capacity=200, bandwidth_from_slow=10, bandwidth_to_slow=10, **kw)


def test_roundtrip_and_content_id(tmp_path):
    p = small_program(recompute_rewrites=(RecomputeRewrite("y", "a", "ra", (RecomputeOption(0, 20, 0.0), RecomputeOption(1, 0, 4.0))),))
    d = program_to_dict(p)
    assert program_from_dict(json.loads(json.dumps(d))) == p
    assert program_content_id(p) == program_content_id(d) and program_content_id(p).startswith("p-")
    save_program(p, tmp_path / "p.json")
    assert load_program(tmp_path / "p.json") == p
    # optional fields are omitted when default; persistent only when true
    assert "host" not in d["tasks"][0] and d["initial_objects"][0]["persistent"] is True
    assert "persistent" not in d["initial_objects"][1]


def test_schema_version_refused():
    d = program_to_dict(small_program())
    d["schema_version"] = "other/v9"
    with pytest.raises(ValueError):
        program_from_dict(d)


def test_validation_collects_all_problems():
    bad = Program("bad", initial_objects=(ObjectSpec("x", 10, "fast"), ObjectSpec("x", 10, "fast")),
                  tasks=(TaskSpec("a", inputs=("nope",), mutates=("other",), outputs=(OutputSpec("x", 5),)),
                         TaskSpec("a", inputs=("x",), prefetch_after=(TransferDirective("x"),))),
                  final_locations={"ghost": "backing"})
    probs = collect_problems(bad)
    text = "\n".join(probs)
    for frag in ("listed twice", "does not exist", "not an input", "not fresh", "duplicate task id",
                 "bandwidth_from_slow", "unknown object 'ghost'"):
        assert frag in text, (frag, text)
    with pytest.raises(ValidationError):
        validate_program(bad)


def test_tensor_meta_must_fit():
    p = Program("t", initial_objects=(ObjectSpec("x", 10, "fast", tensor=TensorMeta("fp32", (4, 4))),))
    assert any("dense tensor needs" in s for s in collect_problems(p))


def test_host_device_mix_refused():
    p = Program("t", initial_objects=(ObjectSpec("x", 10, "backing"),),
                tasks=(TaskSpec("h", inputs=("x",), mutates=("x",), host=True), TaskSpec("d", inputs=("x",))))
    assert any("mixes host and device" in s for s in collect_problems(p))


def test_sim_conversion_roundtrip():
    p = small_program()
    chain = to_sim_chain(p)
    assert [t.id for t in chain.tasks] == ["a", "b"] and chain.tasks[0].prefetch_after[0].obj_id == "w"
    back = from_sim_chain(chain, "t")
    assert [t.releases_after for t in back.tasks] == [t.releases_after for t in p.tasks]
    doc = to_webapp_program(p)
    assert doc["schema_version"] == "dataflow/v1" and len(doc["tasks"]) == 2


def test_documents_that_are_not_programs_are_refused_by_name():
    from dataflow_b200.core import program_from_dict
    from dataflow_b200.core.jsonio import program_to_dict
    good = program_to_dict(Program("p", (ObjectSpec("x", 8, "fast"),), (TaskSpec("a", inputs=("x",), outputs=(OutputSpec("y", 8),)),)))
    assert program_from_dict(good).name == "p"
    for bad, needle in (([1, 2], "not an object"), ({k: v for k, v in good.items() if k != "name"}, "key 'name' is missing"),
                        ({**good, "tasks": None}, "TypeError"), ({**good, "tasks": ["not a task"]}, "Error"),
                        ({**good, "initial_objects": 5}, "TypeError")):
        with pytest.raises(ValueError, match=needle) as e:
            program_from_dict(bad)
        assert "not a dataflow-rt/v1 program" in str(e.value) and not isinstance(e.value, KeyError)
    with pytest.raises(ValueError, match="unsupported schema_version"):
        program_from_dict({**good, "schema_version": "other/v9"})
