"""Engine service: wire handshake, store verbs, registration by content hash, runs on the fake and
host backends, error codes, snapshot → restore bitwise round trip with remap, leases parking a run,
cancel, and a tiny llama3 trained through the daemon (init-as-program)."""
import dataclasses
import os
import socket
import struct
import threading
import time

import pytest

from chains import train_chain
from dataflow_b200.core import (ObjectSpec, OutputSpec, Program, TaskSpec, from_sim_chain, program_content_id,
                                program_to_dict)
from dataflow_b200.service import EngineClient, ServiceError
from dataflow_b200.service.wire import Conn
from dataflow_b200.sim.policies.pressurefit import pressurefit
from dataflow_b200.testing.server_process import engine_client


def planned_program(cap=3000):
    return from_sim_chain(pressurefit(train_chain(L=4, rounds=2), cap).chain, "svc")


def put_initial(c, prog, fill=1):
    for o in prog.initial_objects:
        c.put_object(o.id, bytes([fill]) * o.size_bytes)


def test_handshake_refuses_foreign_schema():
    with engine_client(fake=True) as c:
        s = socket.socket(socket.AF_UNIX)
        s.connect(c.server.config.socket_path)
        conn = Conn(s)
        conn.send({"schema": "other/s9"})
        rep, _ = conn.recv()
        assert rep["ok"] is False and rep["error"]["code"] == "SCHEMA_VERSION_SKEW"
        conn.close()


def test_store_verbs_and_error_codes():
    with engine_client(fake=True) as c:
        c.put_object("a", b"hello world")
        assert c.get_object("a") == b"hello world" and c.get_object("a", 6, 5) == b"world"
        c.duplicate_object("a", "b")
        c.protect_object("b")
        with pytest.raises(ServiceError) as e:
            c.release_object("b")
        assert e.value.code == "PROTECTED"
        with pytest.raises(ServiceError) as e:
            c.get_object("nope")
        assert e.value.code == "UNKNOWN_OBJECT"
        with pytest.raises(ServiceError) as e:
            c.call("frobnicate")
        assert e.value.code == "UNKNOWN_OP"
        with pytest.raises(ServiceError) as e:
            c.create_object("huge", 1 << 40)
        assert e.value.code == "CAPACITY"
        c.materialize_object("z", 4096, "zeros")
        c.materialize_object("t", 4096, "tokens", vocab=100, seed=1)
        assert max(struct.unpack("<1024i", c.get_object("t"))) < 100
        assert c.wipe()["released"] == 3 and [o["id"] for o in c.list_objects()] == ["b"]


def test_register_by_content_hash_and_run_on_fake_backend():
    prog = planned_program()
    with engine_client(fake=True) as c:
        reg = c.register_program(prog, {"kind": "synthetic"})
        assert reg["prog_id"] == program_content_id(program_to_dict(prog))
        with pytest.raises(ServiceError) as e:
            c.register_program(prog, expect_prog_id="p-000000000000")
        assert e.value.code == "VERSION_SKEW"
        with pytest.raises(ServiceError) as e:
            c.run(reg["prog_id"])
        assert e.value.code == "MISSING_INPUTS"
        put_initial(c, prog)
        c.put_object("W0", b"x" * 3)
        with pytest.raises(ServiceError) as e:
            c.run(reg["prog_id"])
        assert e.value.code == "BINDING_MISMATCH"
        put_initial(c, prog)
        out = c.run(reg["prog_id"], trace=True)
        assert out["state"] == "done" and out["slab_overflows"] == 0
        names = {i["name"] for i in out["trace"]["intervals"]}
        assert "f0_0" in names and any(n.startswith("from_slow:") for n in names)
        assert c.run_status(out["run_id"])["state"] == "done"
        assert any(ev["kind"] == "run_done" for ev in c.run_events())
        # jitter changes timing, never the outcome
        reg2 = c.register_program(dataclasses.replace(prog, name="jit"), {"kind": "jitter", "seed": 3})
        assert c.run(reg2["prog_id"])["state"] == "done"


def test_failed_run_reports_typed_error():
    bad = Program("dead", (ObjectSpec("x", 90, "backing"),),
                  (TaskSpec("a", inputs=("x",), outputs=(OutputSpec("y", 20),)),), fast_memory_capacity=100)
    with engine_client(fake=True) as c:
        reg = c.register_program(bad, {"kind": "synthetic"})
        c.put_object("x", b"\0" * 90)
        with pytest.raises(ServiceError) as e:
            c.run(reg["prog_id"])
        assert e.value.code == "RUN_FAILED" and "deadlock" in e.value.message.lower()
        assert c.health()["status"] == "ok"          # the daemon survives


def test_snapshot_restore_roundtrip_with_remap_and_corruption(tmp_path):
    with engine_client(fake=True) as c:
        a, b = os.urandom(300_000), os.urandom(5000)
        c.put_object("A", a)
        c.put_object("B", b)
        job = c.snapshot(str(tmp_path / "s1"), slices=["A", {"id": "B", "offset": 1000, "size": 2000, "as": "Bmid"}])
        st = c.wait_snapshot(job["job_id"])
        assert st["state"] == "done" and len(st["hashes"]) == 2
        c.wipe(force=True)
        r = c.restore_snapshot(str(tmp_path / "s1"), remap=[{"from": "A", "size": len(a)},
                                                            {"from": "Bmid", "from_offset": 1000, "size": 2000, "to": "B2",
                                                             "to_offset": 0, "to_size": 2000}])
        assert r["state"] == "done", r
        assert c.get_object("A") == a and c.get_object("B2") == b[1000:3000]
        # flip one byte on disk: restore must refuse
        f = sorted((tmp_path / "s1").glob("slice00000_*.bin"))[0]
        raw = bytearray(f.read_bytes())
        raw[10] ^= 0xFF
        f.write_bytes(raw)
        c.wipe(force=True)
        r = c.restore_snapshot(str(tmp_path / "s1"))
        assert r["state"] == "failed" and "hash" in r["message"]
        with pytest.raises(ServiceError) as e:
            c.restore_snapshot(str(tmp_path / "missing"))
        assert e.value.code == "UNKNOWN_SNAPSHOT"


def test_run_is_parked_while_a_snapshot_holds_leases():
    prog = planned_program()
    with engine_client(fake=True) as c:
        reg = c.register_program(prog, {"kind": "synthetic"})
        put_initial(c, prog)
        store = c.server.store
        store.acquire_leases(["W0"])                         # as a snapshot in progress would
        done = {}

        def runner():
            with EngineClient(c.server.config.socket_path) as c2:
                done["out"] = c2.run(reg["prog_id"])
        t = threading.Thread(target=runner)
        t.start()
        time.sleep(0.3)
        assert "out" not in done                             # parked, not failed
        store.release_leases(["W0"])
        t.join(timeout=20)
        assert done["out"]["state"] == "done"


def test_train_tiny_llama3_through_the_daemon():
    from dataflow_b200.models.families import build_init_program, resolve_family
    from dataflow_b200.lowering.planning import plan_program
    from dataflow_b200.register import canonical_spec
    from dataflow_b200.run.driver import synthetic_rounds
    fam = resolve_family("llama3")
    cfg = dataclasses.replace(fam.presets["tiny"](), dtype_policy="fp32")
    spec = canonical_spec("llama3", cfg, {"lr": 1e-3}, seed=4)
    planned = plan_program(fam.lower(cfg), None)
    prog = planned.program
    with engine_client(backing_gib=0.2, device=None) as c:
        init = build_init_program(prog)
        for o in init.initial_objects:
            c.create_object(o.id, o.size_bytes)
        ireg = c.register_program(init, spec)
        assert ireg["host"] and c.run(ireg["prog_id"])["state"] == "done"
        c.unregister_program(ireg["prog_id"])
        # registration with a placement dry run: the daemon packs every fast allocation of a run ahead of time, reports the
        # extent, refuses a capacity that cannot hold it, and runs on the placement it found
        with pytest.raises(ServiceError) as bad:
            c.register_program(prog, spec, prepare_placement=True, placement_capacity=4096)
        assert bad.value.code == "BAD_REQUEST" and "no static placement fits" in str(bad.value)
        reg = c.register_program(prog, spec, prepare_placement=True)
        pl = reg["placement"]
        assert pl["allocations"] > 20 and pl["extent_bytes"] >= pl["peak_live_bytes"] > 0
        losses = []
        R = cfg.grad_accum_rounds
        for step in range(3):
            for r, (tk, tg) in enumerate(synthetic_rounds(cfg, R, cfg.tokens_per_round, 64, 9, 0)):
                c.put_object(f"tokens_0_{r}", tk.numpy().tobytes())
                c.put_object(f"targets_0_{r}", tg.numpy().tobytes())
            out = c.run(reg["prog_id"], args={"step": step + 1, "valid_rows": cfg.tokens_per_round * R},
                        fetch=[f"loss_0_{r}" for r in range(R)])
            losses.append(sum(out["fetched"].values()))
            assert out["placement_escapes"] == 0 and out["slab_overflows"] == 0
        assert losses[-1] < losses[0] and 6.5 < losses[0] < 7.5


def test_boot_probe_reports_host_bandwidth():
    """The daemon measures what its own slab delivers (copy, bf16 add) at boot; a slab too small for the probe skips it."""
    from dataflow_b200.service.hostbw import measure_host_bw
    from dataflow_b200.service.store import HostSlab
    slab = HostSlab(40 << 20)
    got = measure_host_bw(slab, mib=16)
    assert set(got) == {"host_copy_gbs", "host_bf16_add_gbs"} and all(v > 0 for v in got.values())
    assert bytes(slab.bytes_view(0, 64)) == bytes(64)            # the probe leaves the slab zeroed
    assert measure_host_bw(slab, mib=32) == {} and measure_host_bw(slab, mib=0) == {}
