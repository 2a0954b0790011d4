"""Checkpoint record layer (validation refusals, restore-plan resolution) and the train-side checkpoint:
bitwise resume of a solo CPU run."""
import copy
import dataclasses
import os

import pytest

from dataflow_b200.checkpoint import RecordError, build_record, read_record, resolve_targets, validate_record, write_record
from dataflow_b200.models.families import resolve_family
from dataflow_b200.run.checkpointing import list_checkpoints, load_checkpoint, peek, resolve_resume, save_checkpoint
from dataflow_b200.run.driver import Trainer, synthetic_rounds


def good_record():
    return build_record(
        step=7, seed=1, scheme={"world": 2},
        logical_objects={"W_0": {"bytes": 100}, "O_0@0": {"bytes": 40}, "O_0@1": {"bytes": 40}},
        snapshots=[{"path": "rank0", "source": "0", "objects": {"W_0": 100, "O_0": 40}},
                   {"path": "rank1", "source": "1", "objects": {"W_0": 100, "O_0": 40}}],
        slices={"W_0": [{"snapshot": 0, "snapshot_range": [0, 100], "object_range": [0, 100], "hash": "aa"},
                        {"snapshot": 1, "snapshot_range": [0, 100], "object_range": [0, 100], "hash": "aa"}],
                "O_0@0": [{"snapshot": 0, "snapshot_object": "O_0", "snapshot_range": [0, 40], "object_range": [0, 40], "hash": "b0"}],
                "O_0@1": [{"snapshot": 1, "snapshot_object": "O_0", "snapshot_range": [0, 40], "object_range": [0, 40], "hash": "b1"}]})


def test_record_roundtrip_and_replica_reader_rule(tmp_path):
    rec = good_record()
    write_record(str(tmp_path), rec)
    assert read_record(str(tmp_path)) == rec
    plans = resolve_targets(rec, ["W_0"])
    assert len(plans) == 1 and plans[0]["snapshot"] == 0          # lowest-index covering snapshot
    rank = resolve_targets(rec, {"1": ["W_0", "O_0"]})
    ids = {r["id"] for p in rank for r in p["remap"]}
    assert ids == {"W_0", "O_0@1"}                                 # bare id resolved to the source's own object


@pytest.mark.parametrize("mutate,needle", [
    (lambda r: r.update(schema="other/v9"), "foreign checkpoint schema"),
    (lambda r: r["slices"]["W_0"][1].update(hash="zz"), "drifted"),
    (lambda r: r["slices"].update(W_0=[{"snapshot": 0, "snapshot_range": [0, 60], "object_range": [0, 60], "hash": "a"}]),
     "covered by no slice"),
    (lambda r: r["slices"]["W_0"].append({"snapshot": 1, "snapshot_range": [0, 50], "object_range": [30, 80], "hash": "c"}),
     "partially overlap"),
    (lambda r: r["slices"]["W_0"][0].update(snapshot=5), "names snapshot 5"),
    (lambda r: r["snapshots"][0]["objects"].update(W_0=10), "does not hold bytes"),
])
def test_record_refusals(mutate, needle):
    rec = copy.deepcopy(good_record())
    mutate(rec)
    with pytest.raises(RecordError, match=needle):
        validate_record(rec)


def test_element_boundary_rule():
    rec = good_record()
    rec["slices"]["W_0"] = [{"snapshot": 0, "snapshot_range": [0, 50], "object_range": [0, 50], "hash": "a"},
                            {"snapshot": 1, "snapshot_range": [50, 100], "object_range": [50, 100], "hash": "b"}]
    validate_record(rec, {"W_0": {"element_bytes": 2}})
    with pytest.raises(RecordError, match="element boundaries"):
        validate_record(rec, {"W_0": {"element_bytes": 4}})


def test_no_record_no_checkpoint(tmp_path):
    os.makedirs(tmp_path / "step_000003" / "rank0")
    assert list_checkpoints(str(tmp_path)) == [] and resolve_resume("latest", str(tmp_path)) is None
    with pytest.raises(RecordError, match="not a complete checkpoint"):
        read_record(str(tmp_path / "step_000003"))


@pytest.mark.parametrize("lower_kwargs", [None, {"resident_params": True}])
def test_solo_resume_is_bitwise(tmp_path, lower_kwargs):
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32")
    hyper = {"lr": 2e-3, "weight_decay": 0.1}
    data = [synthetic_rounds(cfg, 2, 0, 64, 11, s) for s in range(6)]

    def mk():
        return Trainer("llama3", cfg, budget_gib=None, device=None, hyper=hyper, seed=3, leeway_bytes=0, lower_kwargs=lower_kwargs)
    tr = mk()
    data = [synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, s) for s in range(6)]
    straight = []
    for s in range(6):
        straight.append(tr.step(data[s]))
        if s == 2:
            sdir = save_checkpoint(tr, str(tmp_path), 3, seed=3, client_payload={"losses": list(straight)}, keep_last=2)
    tr.close()
    assert peek(sdir)["step"] == 3 and resolve_resume("latest", str(tmp_path)) == sdir
    tr2 = mk()
    tr2.step(data[0])                      # state that the restore must overwrite (and a resident copy to drop)
    rec = load_checkpoint(tr2, sdir)
    assert rec["client_payload"]["losses"] == straight[:3] and tr2.step_index == 3
    resumed = [tr2.step(data[s]) for s in range(3, 6)]
    tr2.close()
    assert resumed == straight[3:]


def test_damaged_checkpoints_are_refused_by_name_and_latest_skips_them(tmp_path):
    """A slice cut short, a flipped byte, a missing slice file, a damaged manifest, a damaged record: each is refused with an
    error that says what is wrong; a directory whose record does not parse is no checkpoint, so "latest" is the step before."""
    import glob
    from dataflow_b200.service.wire import ServiceError
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32")
    tr = Trainer("llama3", cfg, budget_gib=None, device=None, hyper={"lr": 2e-3}, seed=3, leeway_bytes=0)
    try:
        tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, 0))
        first = save_checkpoint(tr, str(tmp_path), 1, seed=3)
        tr.step(synthetic_rounds(cfg, tr.rounds, tr.T, 64, 11, 1))
        second = save_checkpoint(tr, str(tmp_path), 2, seed=3)
        assert resolve_resume("latest", str(tmp_path)) == second
        big = max(glob.glob(os.path.join(second, "rank0", "*.bin")), key=os.path.getsize)
        whole = open(big, "rb").read()
        for damage, needle in ((whole[:len(whole) // 2], "does not match its recorded hash"),
                               (whole[:100] + bytes([whole[100] ^ 0xFF]) + whole[101:], "does not match its recorded hash"), (None, "cannot be read")):
            if damage is None:
                os.remove(big)
            else:
                open(big, "wb").write(damage)
            with pytest.raises(ServiceError, match=needle):
                load_checkpoint(tr, second)
        open(big, "wb").write(whole)
        load_checkpoint(tr, second)                                   # intact again: loads
        manifest = os.path.join(second, "rank0", "snapshot_manifest.json")
        text = open(manifest).read()
        open(manifest, "w").write(text[:len(text) // 2])
        with pytest.raises(ServiceError, match="manifest .* is damaged"):
            load_checkpoint(tr, second)
        open(manifest, "w").write(text)
        record = os.path.join(second, "checkpoint_record.json")
        text = open(record).read()
        open(record, "w").write(text[:len(text) // 2])
        with pytest.raises(RecordError, match="is damaged"):
            read_record(second)
        assert [s for s, _ in list_checkpoints(str(tmp_path))] == [1] and resolve_resume("latest", str(tmp_path)) == first
        assert load_checkpoint(tr, first)["step"] == 1 and tr.step_index == 1
    finally:
        tr.close()
