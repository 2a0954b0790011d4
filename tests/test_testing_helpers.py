"""The helpers other tests and the verification tools are built from: daemons in child processes, parity through the
client, the gradient checks."""
import os
import signal
import time

import pytest
import torch

from dataflow_b200.testing.client_parity import client_model_step, fetch_host_tensor, fetch_views, with_backing_retention
from dataflow_b200.testing.gradcheck import (CheckReport, check_accumulation, check_block_backward, check_model_step,
                                             check_recompute_equivalence, cos_sim, rel_l2)
from dataflow_b200.testing.server_process import SharedServer, engine_client, out_of_process_server, spawn_server


def test_cos_sim_and_rel_l2():
    a = torch.tensor([1.0, 2.0, 3.0])
    assert cos_sim(a, 2 * a) == pytest.approx(1.0) and cos_sim(a, -a) == pytest.approx(-1.0)
    assert cos_sim(torch.zeros(3), torch.zeros(3)) == 1.0 and cos_sim(torch.zeros(3), a) == 0.0
    assert rel_l2(a, a) == 0.0 and rel_l2(2 * a, a) == pytest.approx(1.0)
    rep = CheckReport("f", 1.0, 1.0, {"w": 0.5, "z": 0.9}, {"w": 1.0, "z": 0.0}, {"w": 0.8, "z": 1.0})
    assert rep.failures() == {"w": 0.5} and not rep and "lowest cosine 0.80000" in rep.summary()      # z has no gradient to compare


def test_out_of_process_daemon_serves_and_is_reaped():
    with out_of_process_server(0.05, fake=True) as c:
        assert c.health()["ok"]
        c.put_object("x", b"abcd")
        assert c.get_object("x") == b"abcd"
        sp = c.server_process
        pid = sp.proc.pid
        assert sp.alive
    assert not sp.alive
    with pytest.raises(ProcessLookupError):
        os.kill(pid, 0)


def test_spawned_daemon_runs_extra_source_and_reports_a_failed_boot():
    sp = spawn_server(0.05, fake=True, extra_source="from dataflow_b200.service.registry import register_program_resolver\n"
                                                    "register_program_resolver('extra_kind', lambda spec, env: (lambda task: None))")
    try:
        assert "extra_kind" in sp.client.list_resolvers() and "model_family" in sp.client.list_resolvers()
    finally:
        sp.close()
    with pytest.raises(RuntimeError, match="exited with"):
        spawn_server(0.05, fake=True, extra_source="raise SystemExit(3)")


def test_shared_server_blanks_between_tests_and_replaces_a_dead_daemon():
    s = SharedServer(0.05, fake=True)
    try:
        c = s.fresh()
        c.put_object("a", b"1234")
        c.protect_object("a")
        c2 = s.fresh()
        assert c2 is c and c2.list_objects() == [] and s.respawns == 0       # same daemon, blank again (protected objects too)
        os.kill(s.sp.proc.pid, signal.SIGKILL)
        time.sleep(0.2)
        c3 = s.fresh()
        assert s.respawns == 1 and c3 is not c and c3.health()["ok"]
    finally:
        s.close()


def test_fetches_through_the_client_are_copies_with_the_layouts_fields():
    from dataflow_b200.blocks.layouts import Field, PackedLayout
    lay = PackedLayout((Field("w", (2, 3), "fp32", "param", None), Field("b", (4,), "bf16", "param", None)))
    w = torch.arange(6, dtype=torch.float32).reshape(2, 3)
    b = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.bfloat16)
    offs = lay.offsets()
    raw = bytearray(lay.size_bytes)
    raw[offs["w"]:offs["w"] + 24] = w.numpy().tobytes()
    raw[offs["b"]:offs["b"] + 8] = b.view(torch.int16).numpy().tobytes()
    with engine_client(fake=True) as c:
        c.put_object("obj", bytes(raw))
        v = fetch_views(c, "obj", lay)
        assert torch.equal(v["w"], w) and torch.equal(v["b"], b)
        v["w"].zero_()                                                        # a copy: the daemon's bytes are untouched
        assert torch.equal(fetch_views(c, "obj", lay)["w"], w)
        assert fetch_host_tensor(c, "obj", "uint8").numel() == lay.size_bytes
        c.put_object("short", bytes(8))
        with pytest.raises(ValueError, match="ends at"):
            fetch_views(c, "short", lay)


def test_backing_retention_pins_final_locations():
    from dataflow_b200.core import ObjectSpec, OutputSpec, Program, TaskSpec
    p = Program("p", (ObjectSpec("x", 8, "fast"),), (TaskSpec("a", inputs=("x",), outputs=(OutputSpec("y", 8),)),), final_locations={"x": "fast"})
    q = with_backing_retention(p, ["y", "x"])
    assert dict(q.final_locations) == {"x": "backing", "y": "backing"} and dict(p.final_locations) == {"x": "fast"}


@pytest.mark.parametrize("family", ["llama3", "olmoe"])
def test_a_step_through_the_daemon_matches_the_twins_gradients(family):
    with engine_client(backing_gib=0.3, device=None) as c:
        rep = client_model_step(c, family, tol=0.25 if family == "olmoe" else 2e-2)
    assert rep, rep.summary()
    assert min(rep.grad_cos.values()) > (0.95 if family == "olmoe" else 0.999)


def test_recompute_gives_the_gradients_of_saved_contexts():
    dist = check_recompute_equivalence("llama3", device=None)
    assert dist and max(dist.values()) <= 1e-6
    with pytest.raises(AssertionError, match="did not honour"):
        check_recompute_equivalence("llama3", device=None, layers=[])         # nothing lowered with recompute: the check says so


def test_a_step_of_two_rounds_is_the_sum_of_its_rounds():
    dist = check_accumulation("llama3", device=None)
    assert dist and max(dist.values()) < 5e-4


def test_block_backward_reports_only_the_blocks_fields_with_cosines():
    rep = check_block_backward("llama3", device=None, kind_layer=1)
    assert rep, rep.summary()
    assert rep.grad_rel_l2 and all(k.startswith("layers.1.") for k in rep.grad_rel_l2)
    assert set(rep.grad_cos) == set(rep.grad_rel_l2) and min(rep.grad_cos.values()) > 0.999


def test_a_daemon_survives_malformed_traffic():
    """Garbage, truncated and lying frames on fresh connections: the daemon closes or answers with an error and keeps serving
    its other clients; what it stored is untouched."""
    import socket
    with out_of_process_server(0.05, fake=True) as c:
        path = c.server_process.socket_path
        c.put_object("keep", b"x" * 64)
        frames = [os.urandom(300) + b"\n", b"hello world\n", b"[1,2,3]\n", b"42\n", b"\n", b"\x00" * 100 + b"\n",
                  b'{"schema":"other/v9","op":"health"}\n',
                  b'{"schema":"dataflow-service/s1","op":"put_object","id":"a","payload_bytes":-5}\n',
                  b'{"schema":"dataflow-service/s1","op":"put_object","id":"a","payload_bytes":"many"}\n',
                  b'{"schema":"dataflow-service/s1","op":"put_object","id":"a","payload_bytes":99999999999}\nabc',
                  b'{"schema":"dataflow-service/s1","op":"hea',
                  b'{"schema":"dataflow-service/s1","op":"health","x":' + b"[" * 3000 + b"]" * 3000 + b"}\n",
                  b'{"schema":"dataflow-service/s1","op":"create_object","id":17,"size":"big"}\n']
        for data in frames:
            s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            s.settimeout(2.0)
            s.connect(path)
            try:
                s.sendall(data)
                try:
                    s.recv(4096)
                except (socket.timeout, ConnectionError):
                    pass
            finally:
                s.close()
            assert c.server_process.alive, data[:40]
        assert c.health()["ok"] and c.get_object("keep") == b"x" * 64 and "a" not in [o["id"] if isinstance(o, dict) else o for o in c.list_objects()]
