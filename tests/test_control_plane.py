"""Integration tests of the C++ lighthouse / manager servers over real sockets.

Scenarios follow the reference's in-process server tests (src/lighthouse.rs:913-954,
1040-1142; src/manager.rs:504-718; torchft/lighthouse_test.py).
"""

import threading
import time
import urllib.error
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from datetime import timedelta

import pytest

from torchft_b200 import _control as C

SEC = timedelta(seconds=1)


def make_lighthouse(**kw):
    kw.setdefault("bind", "[::]:0")
    kw.setdefault("min_replicas", 1)
    return C.Lighthouse(**kw)


def make_manager(lh, replica_id, world_size=1, store="store:0"):
    return C.Manager(
        replica_id=replica_id,
        lighthouse_addr=lh.address(),
        hostname="localhost",
        bind="[::]:0",
        store_addr=store,
        world_size=world_size,
        heartbeat_interval=timedelta(milliseconds=50),
        connect_timeout=5 * SEC,
    )


def requester(rid, step=10, shrink_only=False):
    return {"replica_id": rid, "address": "", "store_address": "", "step": step, "world_size": 1, "shrink_only": shrink_only}


def test_lighthouse_heartbeat_and_quorum_e2e():
    lh = make_lighthouse(join_timeout_ms=1)
    try:
        client = C.LighthouseClient(lh.address(), 5 * SEC)
        client.heartbeat("foo")
        q = client.quorum(requester("foo"), 5 * SEC)
        assert q["quorum_id"] == 1
        assert [p["replica_id"] for p in q["participants"]] == ["foo"]
        assert q["participants"][0]["step"] == 10
        assert q["created"] > 0
    finally:
        lh.shutdown()


def test_lighthouse_quorum_id_stable_until_membership_changes():
    # a is usually served alone (fast quorum) just before b asks.  b is then a minority of the
    # heartbeating replicas and gets its quorum when a's heartbeat has aged out, so the expiry is
    # short here and b keeps heartbeating while it waits, as a manager does.
    lh = make_lighthouse(join_timeout_ms=1, heartbeat_timeout_ms=1000)
    stop = threading.Event()

    def keep_b_alive():
        beat = C.LighthouseClient(lh.address(), 5 * SEC)
        while not stop.is_set():
            beat.heartbeat("b")
            stop.wait(0.1)

    try:
        a = C.LighthouseClient(lh.address(), 5 * SEC)
        q1 = a.quorum(requester("a", step=1), 5 * SEC)
        q2 = a.quorum(requester("a", step=2), 5 * SEC)
        assert q1["quorum_id"] == q2["quorum_id"]
        b = C.LighthouseClient(lh.address(), 5 * SEC)
        with ThreadPoolExecutor(3) as ex:
            fa = ex.submit(a.quorum, requester("a", step=3), 5 * SEC)
            time.sleep(0.02)
            ex.submit(keep_b_alive)
            fb = ex.submit(b.quorum, requester("b", step=0), 10 * SEC)
            try:
                qa, qb = fa.result(), fb.result()
            finally:
                stop.set()
        ids = {p["replica_id"] for p in qb["participants"]}
        assert "b" in ids
        assert qb["quorum_id"] > q1["quorum_id"]
    finally:
        stop.set()
        lh.shutdown()


def test_lighthouse_join_during_shrink():
    """A newcomer asking during a shrink-only round is held back, then admitted."""
    lh = make_lighthouse(min_replicas=1, join_timeout_ms=1000, quorum_tick_ms=10)
    try:
        c = [C.LighthouseClient(lh.address(), 5 * SEC) for _ in range(3)]
        # 1. quorum {0, 1}: both are known to be alive, so the first request waits for the second
        c[0].heartbeat("replica0")
        c[1].heartbeat("replica1")
        with ThreadPoolExecutor(3) as ex:
            f0 = ex.submit(c[0].quorum, requester("replica0", 1), 5 * SEC)
            f1 = ex.submit(c[1].quorum, requester("replica1", 1), 5 * SEC)
            q0, q1 = f0.result(), f1.result()
        assert len(q0["participants"]) == 2 and q0 == q1
        first_id = q0["quorum_id"]
        # 2. replica2 asks to join, then the old members ask with shrink_only
        with ThreadPoolExecutor(3) as ex:
            f2 = ex.submit(c[2].quorum, requester("replica2", 1), 5 * SEC)
            time.sleep(0.1)
            f0 = ex.submit(c[0].quorum, requester("replica0", 2, shrink_only=True), 5 * SEC)
            f1 = ex.submit(c[1].quorum, requester("replica1", 2, shrink_only=True), 5 * SEC)
            q0 = f0.result()
            f1.result()
            assert [p["replica_id"] for p in q0["participants"]] == ["replica0", "replica1"]
            assert q0["quorum_id"] == first_id  # same members, same id
            assert not f2.done()  # still waiting
            # 3. the next quorum without shrink_only admits replica2
            f0 = ex.submit(c[0].quorum, requester("replica0", 3), 5 * SEC)
            f1 = ex.submit(c[1].quorum, requester("replica1", 3), 5 * SEC)
            q2 = f2.result()
            f0.result()
            f1.result()
        assert [p["replica_id"] for p in q2["participants"]] == ["replica0", "replica1", "replica2"]
        assert q2["quorum_id"] == first_id + 1
    finally:
        lh.shutdown()


def test_lighthouse_join_latency():
    lh = make_lighthouse(min_replicas=1, join_timeout_ms=100)
    m = make_manager(lh, "latency")
    try:
        client = C.ManagerClient(m.address(), 5 * SEC)
        t0 = time.time()
        client.quorum(rank=0, step=0, checkpoint_metadata="", shrink_only=False, timeout=5 * SEC)
        assert time.time() - t0 < 0.4
    finally:
        m.shutdown()
        lh.shutdown()


def test_manager_should_commit_barrier():
    lh = make_lighthouse()
    m = make_manager(lh, "rep", world_size=2)
    try:
        c0 = C.ManagerClient(m.address(), 5 * SEC)
        c1 = C.ManagerClient(m.address(), 5 * SEC)
        with ThreadPoolExecutor(2) as ex:
            for votes, expect in [((True, True), True), ((True, False), False), ((False, False), False), ((True, True), True)]:
                f0 = ex.submit(c0.should_commit, 0, 1, votes[0], 5 * SEC)
                f1 = ex.submit(c1.should_commit, 1, 1, votes[1], 5 * SEC)
                assert f0.result() is expect and f1.result() is expect
    finally:
        m.shutdown()
        lh.shutdown()


def test_manager_quorum_and_checkpoint_metadata():
    lh = make_lighthouse()
    m = make_manager(lh, "rep_id", world_size=1, store="store_addr")
    try:
        c = C.ManagerClient(m.address(), 5 * SEC)
        with pytest.raises(RuntimeError, match="rank not found"):
            c.checkpoint_metadata(0, 5 * SEC)
        q = c.quorum(rank=0, step=123, checkpoint_metadata="addr", shrink_only=False, timeout=5 * SEC)
        assert q.quorum_id == 1
        assert q.replica_rank == 0 and q.replica_world_size == 1
        assert q.max_step == 123 and q.max_rank == 0 and q.max_world_size == 1
        assert q.store_address == "store_addr"
        assert not q.heal and q.recover_src_rank is None and q.recover_dst_ranks == []
        assert c.checkpoint_metadata(0, 5 * SEC) == "addr"
        with pytest.raises(RuntimeError, match="rank not found"):
            c.checkpoint_metadata(1, 5 * SEC)
    finally:
        m.shutdown()
        lh.shutdown()


def test_two_managers_heal_at_step_zero():
    lh = make_lighthouse(min_replicas=2, join_timeout_ms=10000)
    managers = [make_manager(lh, f"rep_{i}", store=f"store_{i}") for i in range(2)]
    try:
        def ask(i):
            c = C.ManagerClient(managers[i].address(), 5 * SEC)
            return c.quorum(rank=0, step=0, checkpoint_metadata=f"meta{i}", shrink_only=False, timeout=10 * SEC)

        with ThreadPoolExecutor(2) as ex:
            r = list(ex.map(ask, range(2)))
        # replica ids carry no uuid here, so rep_0 sorts first and is the primary
        assert not r[0].heal and r[0].recover_dst_ranks == [1]
        assert r[1].heal and r[1].recover_src_rank == 0
        assert r[1].recover_src_manager_address == managers[0].address()
        assert r[0].store_address == r[1].store_address == "store_0"
        assert r[0].quorum_id == r[1].quorum_id == 1
        assert r[0].replica_world_size == 2 and r[1].replica_rank == 1
    finally:
        for m in managers:
            m.shutdown()
        lh.shutdown()


def test_quorum_timeout_surfaces_quickly():
    lh = make_lighthouse(min_replicas=2)
    m = make_manager(lh, "lonely", world_size=2)
    try:
        c = C.ManagerClient(m.address(), 5 * SEC)
        t0 = time.time()
        with pytest.raises(TimeoutError, match="status: Cancelled, message.*Timeout expired"):
            c.quorum(rank=0, step=0, checkpoint_metadata="", shrink_only=False, timeout=timedelta(milliseconds=10))
        assert time.time() - t0 < 1.0
        t0 = time.time()
        with pytest.raises(TimeoutError, match="status: Cancelled, message.*Timeout expired"):
            c.should_commit(0, 0, True, timedelta(milliseconds=10))
        assert time.time() - t0 < 1.0
    finally:
        m.shutdown()
        lh.shutdown()


def test_manager_reports_lighthouse_timeout_to_all_ranks():
    """min_replicas=2 but only one group: the group's single lighthouse request times out."""
    lh = make_lighthouse(min_replicas=2)
    m = make_manager(lh, "solo", world_size=1)
    try:
        c = C.ManagerClient(m.address(), 5 * SEC)
        with pytest.raises(TimeoutError, match="lighthouse quorum timed out|Timeout expired"):
            c.quorum(rank=0, step=0, checkpoint_metadata="", shrink_only=False, timeout=timedelta(milliseconds=200))
    finally:
        m.shutdown()
        lh.shutdown()


def test_connect_failure_is_runtime_error():
    t0 = time.time()
    with pytest.raises(RuntimeError, match="failed to connect"):
        C.ManagerClient("http://127.0.0.1:1", timedelta(milliseconds=300))
    assert time.time() - t0 < 5.0


def test_heartbeat_timeout_sanity():
    lh = make_lighthouse(heartbeat_timeout_ms=100)
    lh.shutdown()


def test_dashboard_http():
    lh = make_lighthouse(join_timeout_ms=1)
    m = make_manager(lh, "dash")
    try:
        c = C.ManagerClient(m.address(), 5 * SEC)
        c.quorum(rank=0, step=7, checkpoint_metadata="", shrink_only=False, timeout=5 * SEC)
        index = urllib.request.urlopen(lh.address() + "/").read().decode()
        assert "Lighthouse Dashboard" in index
        status = urllib.request.urlopen(lh.address() + "/status").read().decode()
        assert "Current quorum_id: 1" in status
        assert "dash" in status and "Step: 7" in status and "Heartbeats" in status
        js = urllib.request.urlopen(lh.address() + "/status.json").read().decode()
        assert '"quorum_id": 1' in js
        metrics = urllib.request.urlopen(lh.address() + "/metrics").read().decode()
        assert "torchft_quorum_id 1" in metrics and "torchft_quorum_participants 1" in metrics
        assert 'torchft_replica_step{replica_id="dash' in metrics and "torchft_heartbeat_age_seconds{" in metrics
        req = urllib.request.Request(lh.address() + "/replica/unknown/kill", method="POST")
        with pytest.raises(urllib.error.HTTPError) as ei:
            urllib.request.urlopen(req)
        assert ei.value.code == 500
        assert "failed to find replica" in ei.value.read().decode()
        with pytest.raises(urllib.error.HTTPError) as ei:
            urllib.request.urlopen(lh.address() + "/nope")
        assert ei.value.code == 404
    finally:
        m.shutdown()
        lh.shutdown()


def test_kill_rpc_exits_process():
    """Kill ends the process hosting the manager server (run in a child)."""
    import subprocess
    import sys

    code = r"""
import sys, time
from datetime import timedelta
from torchft_b200 import _control as C
C.set_log_enabled(False)
lh = C.Lighthouse(bind="[::]:0", min_replicas=1)
m = C.Manager(replica_id="victim", lighthouse_addr=lh.address(), hostname="localhost", bind="[::]:0",
              store_addr="s", world_size=1, heartbeat_interval=timedelta(milliseconds=100),
              connect_timeout=timedelta(seconds=5))
c = C.ManagerClient(m.address(), timedelta(seconds=5))
try:
    c.kill("bye", timedelta(seconds=5))
except Exception:
    pass
time.sleep(5)
sys.exit(0)
"""
    res = subprocess.run([sys.executable, "-c", code], timeout=60)
    assert res.returncode == 1


def test_lighthouse_cli_flags():
    with pytest.raises(ValueError, match="min_replicas is required"):
        C.lighthouse_main(["--bind", "[::]:0"])
    with pytest.raises(ValueError, match="unknown flag"):
        C.lighthouse_main(["--min_replicas", "1", "--bogus", "1"])


def _schema():
    """The published schema built with the protobuf runtime (no protoc needed)."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory

    fd = descriptor_pb2.FileDescriptorProto()
    fd.name = "tft_test.proto"
    fd.package = "torchft_test"
    fd.syntax = "proto3"
    T = descriptor_pb2.FieldDescriptorProto

    def add(msg, name, number, ftype, label=T.LABEL_OPTIONAL, proto3_optional=False):
        f = msg.field.add()
        f.name, f.number, f.type, f.label = name, number, ftype, label
        if proto3_optional:
            f.proto3_optional = True
            o = msg.oneof_decl.add()
            o.name = "_" + name
            f.oneof_index = len(msg.oneof_decl) - 1
        return f

    qm = fd.message_type.add()
    qm.name = "QuorumMember"
    add(qm, "replica_id", 1, T.TYPE_STRING)
    add(qm, "address", 2, T.TYPE_STRING)
    add(qm, "store_address", 3, T.TYPE_STRING)
    add(qm, "step", 4, T.TYPE_INT64)
    add(qm, "world_size", 5, T.TYPE_UINT64)
    add(qm, "shrink_only", 6, T.TYPE_BOOL)

    r = fd.message_type.add()
    r.name = "ManagerQuorumResponse"
    add(r, "quorum_id", 1, T.TYPE_INT64)
    add(r, "recover_src_manager_address", 2, T.TYPE_STRING)
    add(r, "recover_src_rank", 3, T.TYPE_INT64, proto3_optional=True)
    add(r, "recover_dst_ranks", 4, T.TYPE_INT64, label=T.LABEL_REPEATED)
    add(r, "store_address", 5, T.TYPE_STRING)
    add(r, "max_step", 6, T.TYPE_INT64)
    add(r, "max_rank", 7, T.TYPE_INT64, proto3_optional=True)
    add(r, "max_world_size", 8, T.TYPE_INT64)
    add(r, "replica_rank", 9, T.TYPE_INT64)
    add(r, "replica_world_size", 10, T.TYPE_INT64)
    add(r, "heal", 11, T.TYPE_BOOL)

    pool = descriptor_pool.DescriptorPool()
    pool.Add(fd)
    get = message_factory.GetMessageClass
    return get(pool.FindMessageTypeByName("torchft_test.QuorumMember")), get(
        pool.FindMessageTypeByName("torchft_test.ManagerQuorumResponse")
    )


def test_wire_format_matches_protobuf_runtime():
    QuorumMember, Response = _schema()
    d = {"replica_id": "réplica", "address": "http://h:1", "store_address": "h:2", "step": -3, "world_size": 2**40, "shrink_only": True}
    ours = C.encode_quorum_member(d)
    ref = QuorumMember(**d)
    assert QuorumMember.FromString(ours) == ref
    assert C.decode_quorum_member(ref.SerializeToString()) == d

    q = C.QuorumResult()
    q.quorum_id = 9
    q.recover_src_manager_address = "http://src:1"
    q.recover_src_rank = 0  # present although zero
    q.recover_dst_ranks = [1, 300, 70000]
    q.store_address = "store:3"
    q.max_step = 77
    q.max_rank = None
    q.max_world_size = 3
    q.replica_rank = 2
    q.replica_world_size = 5
    q.heal = True
    theirs = Response.FromString(C.encode_manager_quorum_response(q))
    assert theirs.HasField("recover_src_rank") and theirs.recover_src_rank == 0
    assert not theirs.HasField("max_rank")
    assert list(theirs.recover_dst_ranks) == [1, 300, 70000]
    assert theirs.max_step == 77 and theirs.heal and theirs.replica_world_size == 5

    back = C.decode_manager_quorum_response(theirs.SerializeToString())
    assert back.recover_src_rank == 0 and back.max_rank is None
    assert back.recover_dst_ranks == [1, 300, 70000]
    assert back.store_address == "store:3" and back.quorum_id == 9

    default = C.QuorumResult()
    assert default.replica_world_size == 1 and default.max_world_size == 1 and default.recover_src_rank is None


def test_force_reconfigure_bumps_quorum_id_without_membership_change():
    """A member whose step failed asks for a new quorum id; everybody gets it."""
    lh = make_lighthouse(min_replicas=2, join_timeout_ms=5000)
    managers = [make_manager(lh, f"fr_{i}") for i in range(2)]
    try:
        clients = [C.ManagerClient(m.address(), 5 * SEC) for m in managers]

        def ask(i, step, force):
            return clients[i].quorum(rank=0, step=step, checkpoint_metadata="", shrink_only=False, timeout=10 * SEC,
                                     force_reconfigure=force)

        with ThreadPoolExecutor(2) as ex:
            a = [f.result() for f in [ex.submit(ask, i, 1, False) for i in range(2)]]
            b = [f.result() for f in [ex.submit(ask, i, 2, False) for i in range(2)]]
            c = [f.result() for f in [ex.submit(ask, i, 3, i == 1) for i in range(2)]]
            d = [f.result() for f in [ex.submit(ask, i, 4, False) for i in range(2)]]
        assert a[0].quorum_id == a[1].quorum_id == b[0].quorum_id == b[1].quorum_id
        assert c[0].quorum_id == c[1].quorum_id == a[0].quorum_id + 1  # forced by replica 1 alone
        assert d[0].quorum_id == c[0].quorum_id  # and stable again afterwards
    finally:
        for m in managers:
            m.shutdown()
        lh.shutdown()


def test_wire_decoder_rejects_garbage_without_crashing():
    """Random and truncated payloads end in an exception or a value, never in a crash."""
    import random

    rng = random.Random(7)
    good = C.encode_quorum_member({"replica_id": "r", "address": "a", "store_address": "s", "step": 5, "world_size": 2, "shrink_only": False})
    samples = [bytes(rng.getrandbits(8) for _ in range(rng.randint(0, 64))) for _ in range(500)]
    samples += [good[:n] for n in range(len(good))]
    samples += [b"\x0a\xff\xff\xff\xff\x0f" + b"x" * 10, b"\xff" * 32, b"\x08" + b"\x80" * 20]
    outcomes = {"ok": 0, "error": 0}
    for payload in samples:
        for decode in (C.decode_quorum_member, C.decode_manager_quorum_response):
            try:
                decode(payload)
                outcomes["ok"] += 1
            except (RuntimeError, ValueError):
                outcomes["error"] += 1
    assert outcomes["error"] > 0 and outcomes["ok"] > 0


def test_wire_codec_round_trips_random_messages():
    """Random field values survive this codec -> protobuf runtime -> this codec unchanged."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    QuorumMember, Response = _schema()
    i64 = st.integers(min_value=-(2**63), max_value=2**63 - 1)
    text = st.text(max_size=40)

    @settings(max_examples=200, deadline=None)
    @given(rid=text, addr=text, store=text, step=i64, world=st.integers(0, 2**64 - 1), shrink=st.booleans())
    def member_round_trip(rid, addr, store, step, world, shrink):
        d = {"replica_id": rid, "address": addr, "store_address": store, "step": step, "world_size": world, "shrink_only": shrink}
        theirs = QuorumMember.FromString(C.encode_quorum_member(d))
        assert (theirs.replica_id, theirs.address, theirs.store_address, theirs.step, theirs.world_size, theirs.shrink_only) == (
            rid, addr, store, step, world, shrink)
        assert C.decode_quorum_member(theirs.SerializeToString()) == d

    @settings(max_examples=200, deadline=None)
    @given(qid=i64, src=text, src_rank=st.none() | i64, dst=st.lists(i64, max_size=6), store=text, max_step=i64,
           max_rank=st.none() | i64, heal=st.booleans())
    def response_round_trip(qid, src, src_rank, dst, store, max_step, max_rank, heal):
        q = C.QuorumResult()
        q.quorum_id, q.recover_src_manager_address, q.recover_src_rank, q.recover_dst_ranks = qid, src, src_rank, dst
        q.store_address, q.max_step, q.max_rank, q.heal = store, max_step, max_rank, heal
        theirs = Response.FromString(C.encode_manager_quorum_response(q))
        assert theirs.HasField("recover_src_rank") == (src_rank is not None)
        assert theirs.HasField("max_rank") == (max_rank is not None)
        back = C.decode_manager_quorum_response(theirs.SerializeToString())
        assert (back.quorum_id, back.recover_src_manager_address, back.recover_src_rank, back.recover_dst_ranks) == (qid, src, src_rank, dst)
        assert (back.store_address, back.max_step, back.max_rank, back.heal) == (store, max_step, max_rank, heal)

    member_round_trip()
    response_round_trip()


def test_extension_module_alias_has_the_reference_names():
    """``torchft_b200.torchft`` offers what code written for the reference imports from ``torchft.torchft``."""
    import torchft_b200 as torchft
    from torchft_b200 import _control
    from torchft_b200.torchft import Lighthouse, Manager, ManagerClient, QuorumResult

    assert Lighthouse is _control.Lighthouse and Manager is _control.Manager
    assert ManagerClient is _control.ManagerClient and QuorumResult is _control.QuorumResult
    for name in ("DistributedDataParallel", "DistributedSampler", "Manager", "Optimizer", "ProcessGroupBabyNCCL", "ProcessGroupGloo"):
        assert getattr(torchft, name) is not None
