"""Peer plane protocol battery: rendezvous sends over an in-memory link with scripted loss, duplication and
corruption; NACK back-off; inactivity; dedup; group table; collective queue.  All faults are made on the host."""
import pytest

from dataflow_b200.service.peer import protocol as P
from dataflow_b200.service.peer.core import CollectiveQueue, PeerCore
from dataflow_b200.service.peer.groups import GroupTable
from dataflow_b200.service.peer.transports import FaultPlan, MemLink


class Box:
    """A tiny store: reservations by xid, committed objects by id."""

    def __init__(self, cap=1 << 30):
        self.res, self.objs, self.cap, self.refuse = {}, {}, cap, 0

    def reserve(self, xid, size):
        if self.refuse > 0:
            self.refuse -= 1
            raise MemoryError("no room yet")
        if size > self.cap:
            raise MemoryError("too big")
        self.res[xid] = bytearray(size)

    def land(self, xid, off, payload):
        self.res[xid][off:off + len(payload)] = payload

    def commit(self, xid, dest):
        if dest is None:
            return bytes(self.res[xid])
        self.objs[dest] = bytes(self.res.pop(xid))
        return self.objs[dest]

    def drop(self, xid):
        self.res.pop(xid, None)


def pair(plan_ab=None, plan_ba=None, chunk=1 << 10, clock=None):
    link = MemLink(plan_ab, plan_ba)
    ba, bb = Box(), Box()
    mk = lambda name, side, box: PeerCore(name, link.emitter(side), reserve=box.reserve, land=box.land, commit=box.commit,
                                          drop=box.drop, chunk_bytes=chunk, clock=clock)
    a, b = mk("a", "a", ba), mk("b", "b", bb)
    link.attach("a", a)
    link.attach("b", b)
    return link, a, b, ba, bb


def test_eager_and_chunked_sends_arrive_bit_exact():
    link, a, b, _, bb = pair()
    small, big = b"x" * 100, bytes(range(256)) * 4000 + b"tail"          # 1 MB-ish in 1 KiB chunks
    assert len(big) > P.EAGER_MAX
    x1, x2 = a.start_send("b", "small", small), a.start_send("b", "big", big, dest_id="big_copy")
    link.pump()
    assert bb.objs == {"small": small, "big_copy": big}
    assert a.status(x1)["state"] == a.status(x2)["state"] == "COMPLETE" and b.stats["received"] == 2


@pytest.mark.parametrize("plan", [
    FaultPlan(drop={"CHUNK": {1, 5}}),                        # lost chunks -> DONE finds a hole -> whole resend
    FaultPlan(duplicate={"CHUNK": {0, 2}, "RTS": {0}, "DONE": {0}}),
    FaultPlan(corrupt={"CHUNK": {3}}),                        # crc mismatch -> resend
])
def test_faults_on_the_data_path_are_repaired(plan):
    link, a, b, _, bb = pair(plan_ab=plan)
    big = bytes(range(256)) * 400
    x = a.start_send("b", "obj", big)
    link.pump()
    assert bb.objs["obj"] == big and a.status(x)["state"] == "COMPLETE"
    assert plan.log, "the fault never fired"
    assert not b.receivers and len(bb.res) == 0


def test_duplicate_rts_after_commit_is_answered_from_the_dedup_ring():
    link, a, b, _, bb = pair()
    x = a.start_send("b", "o", b"abc")
    link.pump()
    before = dict(b.stats)
    b.handle("a", P.rts(x, "o", 3, P.checksum(b"abc"), inline=b""), b"abc")
    link.pump()
    assert b.stats["received"] == before["received"] and b.stats["duplicates"] == before["duplicates"] + 1


def test_nack_backoff_then_success_and_exhaustion():
    now = [0.0]
    link, a, b, _, bb = pair(clock=lambda: now[0])
    bb.refuse = 2
    x = a.start_send("b", "o", b"y" * (P.EAGER_MAX + 5))
    link.pump()
    assert a.status(x)["state"] == "BACKOFF"
    for _ in range(2):
        now[0] += 1.0
        a.tick()
        link.pump()
    assert a.status(x)["state"] == "COMPLETE" and a.status(x)["retries"] == 2
    bb.refuse = 100
    y = a.start_send("b", "p", b"z" * (P.EAGER_MAX + 5))
    for _ in range(P.NACK_RETRIES + 2):
        link.pump()
        now[0] += 10.0
        a.tick()
    assert a.status(y)["state"] == "FAILED" and "refused" in a.status(y)["error"]


def test_inactivity_fails_the_sender_and_frees_the_receiver():
    now = [0.0]
    link, a, b, _, bb = pair(plan_ab=FaultPlan(drop={"DONE": {0}}), clock=lambda: now[0])
    x = a.start_send("b", "o", b"q" * (P.EAGER_MAX + 1))
    link.pump()
    assert a.status(x)["state"] == "DONE_SENT" and len(bb.res) == 1
    now[0] += P.INACTIVITY_S + 1
    a.tick()
    b.tick()
    assert a.status(x)["state"] == "FAILED" and not bb.res and not b.receivers


def test_peer_lost_fails_open_transfers():
    link, a, b, _, bb = pair(plan_ab=FaultPlan(drop={"DONE": {0}}))
    x = a.start_send("b", "o", b"q" * (P.EAGER_MAX + 1))
    link.pump()
    a.peer_lost("b")
    b.peer_lost("a")
    assert a.status(x)["state"] == "FAILED" and not bb.res


def test_group_table_barrier_and_collective_queue():
    t = GroupTable()
    g = t.create("dp", ["a", "b", "c"], "hostmem", "a")
    t.ack("dp", "b")
    assert t.get("dp").state == "FORMING"
    t.ack("dp", "c")
    assert t.wait_ready("dp", 0.1).state == "READY" and g.rank_of("c") == 2
    t.create("slow", ["a", "b"], "hostmem", "a")
    with pytest.raises(RuntimeError, match="never acknowledged"):
        t.wait_ready("slow", 0.05)
    q = CollectiveQueue("dp")
    q.push("all_reduce", 1024, "fp32")
    q.match({"seq": 1, "op": "all_reduce", "nbytes": 1024, "dtype": "fp32"})
    q.push("all_gather", 64, "bf16")
    with pytest.raises(RuntimeError, match="mismatch"):
        q.match({"seq": 2, "op": "all_reduce", "nbytes": 64, "dtype": "bf16"})


# ------------------------------------------------------------------ two daemons over loopback TCP
import threading
import time

from dataflow_b200.service import EngineClient, EngineConfig, Server


def boot(tmp_path, name):
    cfg = EngineConfig(socket_path=str(tmp_path / f"{name}.sock"), slab_backing_gib=0.05, fake=True, peer_name=name,
                       peer_listen="127.0.0.1:0", peer_chunk_bytes=1 << 16)
    srv = Server(cfg)
    t = threading.Thread(target=srv.serve_forever, daemon=True)
    t.start()
    for _ in range(200):
        try:
            c = EngineClient(cfg.socket_path, "test", timeout=30.0)
            return srv, c
        except OSError:
            time.sleep(0.02)
    raise RuntimeError("daemon did not come up")


def test_two_daemons_send_objects_form_a_group_and_detect_a_cut_link(tmp_path):
    sa, ca = boot(tmp_path, "a")
    sb, cb = boot(tmp_path, "b")
    try:
        port_b = cb.call("list_peers")["port"]
        ca.peer_connect("b", f"127.0.0.1:{port_b}")
        for _ in range(100):
            if cb.list_peers():
                break
            time.sleep(0.02)
        assert ca.list_peers()[0]["peer"] == "b" and cb.list_peers()[0]["peer"] == "a"
        blob = bytes(range(256)) * 2000                         # 512 KB: rendezvous path in 64 KiB chunks
        ca.put_object("w", blob)
        out = ca.send_object("b", "w", "w_from_a")
        assert out["state"] == "done" and cb.get_object("w_from_a") == blob
        ca.put_object("tiny", b"hello")
        ca.send_object("b", "tiny")
        assert cb.get_object("tiny") == b"hello"
        # group + star all-reduce (both members must issue the collective: run them on threads)
        ca.create_peer_group("dp", ["a", "b"], backend="hostmem")
        assert cb.list_peer_groups()[0]["state"] == "READY"
        res = {}
        th = [threading.Thread(target=lambda k=k, c=c: res.__setitem__(k, c.coll_bench("dp"))) for k, c in (("a", ca), ("b", EngineClient(sb.config.socket_path, "t2")))]
        [t.start() for t in th]
        [t.join(30) for t in th]
        assert res["a"]["ok"] and res["b"]["ok"] and res["a"]["got"] == 3.0
        # a cut link is noticed by both sides and fails the group; failures are made on the host
        ca.call("debug_sever", peer="b")
        for _ in range(200):
            if not ca.list_peers()[0]["up"] and not cb.list_peers()[0]["up"]:
                break
            time.sleep(0.02)
        assert not ca.list_peers()[0]["up"] and not cb.list_peers()[0]["up"]
        assert ca.list_peer_groups()[0]["state"] == "ERROR"
    finally:
        for c in (ca, cb):
            try:
                c.shutdown()
            except Exception:       # noqa: BLE001
                pass
