"""gRPC-over-HTTP/2 compatibility of the control plane, checked against a real gRPC stack (grpcio).

* HPACK against RFC 7541 test vectors;
* a grpcio client (its own HPACK encoder, flow control and framing) calls this repository's
  lighthouse and manager servers with protobuf-runtime messages of the published schema;
* this repository's clients, switched to the gRPC wire protocol, call a grpcio server;
* the whole quorum / commit path with every client of the process on the gRPC protocol.
"""

import os
import subprocess
import sys
import threading
import time
from concurrent import futures
from datetime import timedelta

import pytest

from torchft_b200 import _control as C

grpc = pytest.importorskip("grpc")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _schema():
    """Messages of the published schema, built with the protobuf runtime (no protoc needed)."""
    from google.protobuf import descriptor_pb2, descriptor_pool, message_factory, timestamp_pb2

    pool = descriptor_pool.DescriptorPool()
    ts_fd = descriptor_pb2.FileDescriptorProto()
    timestamp_pb2.DESCRIPTOR.CopyToProto(ts_fd)
    pool.Add(ts_fd)
    fd = descriptor_pb2.FileDescriptorProto()
    fd.name = "tft_wire_test.proto"
    fd.package = "tft_wire_test"
    fd.syntax = "proto3"
    fd.dependency.append(ts_fd.name)
    T = descriptor_pb2.FieldDescriptorProto

    def message(name, *fields):
        m = fd.message_type.add()
        m.name = name
        for fname, number, ftype, extra in fields:
            f = m.field.add()
            f.name, f.number, f.type = fname, number, ftype
            f.label = T.LABEL_REPEATED if extra.get("repeated") else T.LABEL_OPTIONAL
            if "type_name" in extra:
                f.type_name = extra["type_name"]
            if extra.get("optional"):
                f.proto3_optional = True
                o = m.oneof_decl.add()
                o.name = "_" + fname
                f.oneof_index = len(m.oneof_decl) - 1

    message("QuorumMember", ("replica_id", 1, T.TYPE_STRING, {}), ("address", 2, T.TYPE_STRING, {}),
            ("store_address", 3, T.TYPE_STRING, {}), ("step", 4, T.TYPE_INT64, {}), ("world_size", 5, T.TYPE_UINT64, {}),
            ("shrink_only", 6, T.TYPE_BOOL, {}))
    message("Quorum", ("quorum_id", 1, T.TYPE_INT64, {}),
            ("participants", 2, T.TYPE_MESSAGE, {"repeated": True, "type_name": ".tft_wire_test.QuorumMember"}),
            ("created", 3, T.TYPE_MESSAGE, {"type_name": ".google.protobuf.Timestamp"}))
    message("LighthouseQuorumRequest", ("requester", 1, T.TYPE_MESSAGE, {"type_name": ".tft_wire_test.QuorumMember"}))
    message("LighthouseQuorumResponse", ("quorum", 1, T.TYPE_MESSAGE, {"type_name": ".tft_wire_test.Quorum"}))
    message("LighthouseHeartbeatRequest", ("replica_id", 1, T.TYPE_STRING, {}))
    message("Empty")
    message("ManagerQuorumRequest", ("rank", 1, T.TYPE_INT64, {}), ("step", 2, T.TYPE_INT64, {}),
            ("checkpoint_metadata", 3, T.TYPE_STRING, {}), ("shrink_only", 4, T.TYPE_BOOL, {}))
    message("ManagerQuorumResponse", ("quorum_id", 1, T.TYPE_INT64, {}), ("recover_src_manager_address", 2, T.TYPE_STRING, {}),
            ("recover_src_rank", 3, T.TYPE_INT64, {"optional": True}), ("recover_dst_ranks", 4, T.TYPE_INT64, {"repeated": True}),
            ("store_address", 5, T.TYPE_STRING, {}), ("max_step", 6, T.TYPE_INT64, {}),
            ("max_rank", 7, T.TYPE_INT64, {"optional": True}), ("max_world_size", 8, T.TYPE_INT64, {}),
            ("replica_rank", 9, T.TYPE_INT64, {}), ("replica_world_size", 10, T.TYPE_INT64, {}), ("heal", 11, T.TYPE_BOOL, {}))
    message("CheckpointMetadataRequest", ("rank", 1, T.TYPE_INT64, {}))
    message("CheckpointMetadataResponse", ("checkpoint_metadata", 1, T.TYPE_STRING, {}))
    message("ShouldCommitRequest", ("should_commit", 1, T.TYPE_BOOL, {}), ("rank", 2, T.TYPE_INT64, {}), ("step", 3, T.TYPE_INT64, {}))
    message("ShouldCommitResponse", ("should_commit", 1, T.TYPE_BOOL, {}))
    pool.Add(fd)

    class Schema:
        pass

    s = Schema()
    for m in fd.message_type:
        setattr(s, m.name, message_factory.GetMessageClass(pool.FindMessageTypeByName("tft_wire_test." + m.name)))
    return s


def _unary(channel, path, request, response_cls, timeout=10.0, **kw):
    call = channel.unary_unary(path, request_serializer=lambda m: m.SerializeToString(),
                               response_deserializer=response_cls.FromString)
    return call(request, timeout=timeout, **kw)


# ---------------------------------------------------------------- HPACK
def test_hpack_rfc7541_vectors():
    d = C.HpackDecoder()
    # C.4.1-C.4.3: three requests on one connection, Huffman-coded strings, growing dynamic table
    assert d.decode(bytes.fromhex("828684418cf1e3c2e5f23a6ba0ab90f4ff")) == [
        (b":method", b"GET"), (b":scheme", b"http"), (b":path", b"/"), (b":authority", b"www.example.com")]
    assert d.decode(bytes.fromhex("828684be5886a8eb10649cbf"))[-1] == (b"cache-control", b"no-cache")
    third = d.decode(bytes.fromhex("828785bf408825a849e95ba97d7f8925a849e95bb8e8b4bf"))
    assert third == [(b":method", b"GET"), (b":scheme", b"https"), (b":path", b"/index.html"),
                     (b":authority", b"www.example.com"), (b"custom-key", b"custom-value")]
    # C.3.1 without Huffman coding, fresh connection
    assert C.HpackDecoder().decode(bytes.fromhex("828684410f7777772e6578616d706c652e636f6d"))[-1] == (b":authority", b"www.example.com")
    # malformed: index 0, truncated string
    assert C.HpackDecoder().decode(b"\x80") is None
    assert C.HpackDecoder().decode(bytes.fromhex("400a6375")) is None


def test_huffman_round_trip_and_padding_rules():
    assert C.huffman_encode(b"www.example.com").hex() == "f1e3c2e5f23a6ba0ab90f4ff"
    assert C.huffman_encode(b"no-cache").hex() == "a8eb10649cbf"
    assert C.huffman_encode(b"custom-value").hex() == "25a849e95bb8e8b4bf"
    for s in (b"", b"/torchft.ManagerService/ShouldCommit", b"application/grpc", b"12345678m", bytes(range(256))):
        assert C.huffman_decode(C.huffman_encode(s)) == s
    assert C.huffman_decode(bytes.fromhex("f1e3c2e5f23a6ba0ab90f400")) is None  # padding must be ones
    assert C.huffman_decode(b"\xff\xff\xff\xff") is None  # more than 7 bits of padding / EOS


def test_encoder_output_is_read_by_own_decoder():
    headers = [(":status", "200"), ("content-type", "application/grpc"), ("grpc-status", "4"),
               ("grpc-message", "deadline%20exceeded"), ("x-new-name", "v" * 300)]
    for huffman in (False, True):
        block = C.hpack_encode(headers, huffman)
        assert C.HpackDecoder().decode(block) == [(k.encode(), v.encode()) for k, v in headers]


# ---------------------------------------------------------------- grpcio client -> our servers
def test_grpcio_client_talks_to_lighthouse_and_manager():
    S = _schema()
    lighthouse = C.Lighthouse(bind="[::]:0", min_replicas=1, join_timeout_ms=100, quorum_tick_ms=10)
    manager = None
    try:
        lh_port = lighthouse.address().rsplit(":", 1)[1]
        with grpc.insecure_channel(f"127.0.0.1:{lh_port}") as ch:
            _unary(ch, "/torchft.LighthouseService/Heartbeat", S.LighthouseHeartbeatRequest(replica_id="solo"), S.Empty)
            member = S.QuorumMember(replica_id="solo", address="http://a:1", store_address="s:1", step=7, world_size=1)
            resp = _unary(ch, "/torchft.LighthouseService/Quorum", S.LighthouseQuorumRequest(requester=member),
                          S.LighthouseQuorumResponse)
            assert [p.replica_id for p in resp.quorum.participants] == ["solo"]
            assert resp.quorum.participants[0].step == 7 and resp.quorum.quorum_id >= 1
            assert resp.quorum.created.seconds > 1_600_000_000
            # unknown method -> UNIMPLEMENTED, as any gRPC server answers
            with pytest.raises(grpc.RpcError) as err:
                _unary(ch, "/torchft.LighthouseService/Nope", S.Empty(), S.Empty)
            assert err.value.code() == grpc.StatusCode.UNIMPLEMENTED

        # a second lighthouse for the manager, so that "solo" above is not a heartbeating absentee here
        lighthouse.shutdown()
        lighthouse = C.Lighthouse(bind="[::]:0", min_replicas=1, join_timeout_ms=100, quorum_tick_ms=10)
        manager = C.Manager(replica_id="wire", lighthouse_addr=lighthouse.address(), hostname="127.0.0.1", bind="[::]:0",
                            store_addr="store:1", world_size=2, heartbeat_interval=timedelta(milliseconds=100),
                            connect_timeout=timedelta(seconds=5))
        mgr_port = manager.address().rsplit(":", 1)[1]
        with grpc.insecure_channel(f"127.0.0.1:{mgr_port}") as ch:
            # two local ranks ask concurrently on ONE channel: the calls are multiplexed streams and
            # the first must stay open until the second arrives
            results = {}

            def ask(rank):
                results[rank] = _unary(ch, "/torchft.ManagerService/Quorum",
                                       S.ManagerQuorumRequest(rank=rank, step=3, checkpoint_metadata=f"meta{rank}"),
                                       S.ManagerQuorumResponse, timeout=20.0)

            threads = [threading.Thread(target=ask, args=(r,)) for r in (0, 1)]
            threads[0].start()
            time.sleep(0.3)
            assert 0 not in results  # still waiting for rank 1
            threads[1].start()
            for t in threads:
                t.join(timeout=30)
            for rank in (0, 1):
                r = results[rank]
                assert r.replica_world_size == 1 and r.replica_rank == 0 and r.max_step == 3 and not r.heal
                assert r.HasField("max_rank") and r.max_rank == 0 and r.store_address == "store:1"
            meta = _unary(ch, "/torchft.ManagerService/CheckpointMetadata", S.CheckpointMetadataRequest(rank=1),
                          S.CheckpointMetadataResponse)
            assert meta.checkpoint_metadata == "meta1"
            votes = {}

            def vote(rank, value):
                votes[rank] = _unary(ch, "/torchft.ManagerService/ShouldCommit",
                                     S.ShouldCommitRequest(should_commit=value, rank=rank, step=3), S.ShouldCommitResponse)

            threads = [threading.Thread(target=vote, args=(0, True)), threading.Thread(target=vote, args=(1, False))]
            for t in threads:
                t.start()
            for t in threads:
                t.join(timeout=30)
            assert not votes[0].should_commit and not votes[1].should_commit
            # a request without a deadline is refused by the manager's quorum handler with a gRPC status
            with pytest.raises(grpc.RpcError) as err:
                _unary(ch, "/torchft.ManagerService/Quorum", S.ManagerQuorumRequest(rank=0, step=4), S.ManagerQuorumResponse,
                       timeout=None)
            assert err.value.code() == grpc.StatusCode.INVALID_ARGUMENT and "missing timeout" in err.value.details()
    finally:
        if manager is not None:
            manager.shutdown()
        lighthouse.shutdown()


def test_grpcio_client_deadline_is_enforced_by_the_server():
    S = _schema()
    lighthouse = C.Lighthouse(bind="[::]:0", min_replicas=2, join_timeout_ms=60000, quorum_tick_ms=10)
    try:
        port = lighthouse.address().rsplit(":", 1)[1]
        with grpc.insecure_channel(f"127.0.0.1:{port}") as ch:
            member = S.QuorumMember(replica_id="lonely", address="a", store_address="s", step=0, world_size=1)
            t0 = time.time()
            with pytest.raises(grpc.RpcError) as err:
                _unary(ch, "/torchft.LighthouseService/Quorum", S.LighthouseQuorumRequest(requester=member),
                       S.LighthouseQuorumResponse, timeout=0.3)
            assert err.value.code() in (grpc.StatusCode.DEADLINE_EXCEEDED, grpc.StatusCode.CANCELLED)
            assert time.time() - t0 < 3
            # the connection is still usable afterwards
            _unary(ch, "/torchft.LighthouseService/Heartbeat", S.LighthouseHeartbeatRequest(replica_id="lonely"), S.Empty)
    finally:
        lighthouse.shutdown()


# ---------------------------------------------------------------- our clients -> a grpcio server
class _Generic(grpc.GenericRpcHandler):
    def __init__(self, S, seen):
        self.S, self.seen = S, seen

    def service(self, details):
        S, seen = self.S, self.seen
        method = details.method
        metadata = dict(details.invocation_metadata)

        def heartbeat(request, context):
            seen.append((method, S.LighthouseHeartbeatRequest.FromString(request).replica_id, metadata.get("user-agent")))
            return S.Empty().SerializeToString()

        def should_commit(request, context):
            req = S.ShouldCommitRequest.FromString(request)
            seen.append((method, req.rank, req.step, req.should_commit, context.time_remaining()))
            if req.step == 13:
                context.abort(grpc.StatusCode.NOT_FOUND, "no such step: 13 é")
            return S.ShouldCommitResponse(should_commit=req.should_commit).SerializeToString()

        def slow(request, context):
            time.sleep(1.0)
            return S.CheckpointMetadataResponse(checkpoint_metadata="late").SerializeToString()

        def big(request, context):
            return S.CheckpointMetadataResponse(checkpoint_metadata="x" * 300_000).SerializeToString()

        table = {"/torchft.LighthouseService/Heartbeat": heartbeat, "/torchft.ManagerService/ShouldCommit": should_commit}
        if method == "/torchft.ManagerService/CheckpointMetadata":
            return grpc.unary_unary_rpc_method_handler(
                lambda request, context: (slow if S.CheckpointMetadataRequest.FromString(request).rank == 9 else big)(request, context))
        if method in table:
            return grpc.unary_unary_rpc_method_handler(table[method])
        return None


_CLIENT_SCRIPT = r"""
import sys, time
from datetime import timedelta
from torchft_b200 import _control as C
C.set_rpc_protocol("grpc")
assert C.rpc_protocol() == "grpc"
addr = sys.argv[1]
m = C.ManagerClient(addr, connect_timeout=timedelta(seconds=5))
assert m.should_commit(2, 5, True, timeout=timedelta(seconds=7)) is True
assert m.should_commit(3, 6, False, timeout=timedelta(seconds=7)) is False
try:
    m.should_commit(0, 13, True, timeout=timedelta(seconds=7))
    raise SystemExit("expected an error")
except RuntimeError as e:
    assert "NotFound" in str(e) or "code: 5" in str(e) or "no such step" in str(e), str(e)
    assert "no such step: 13 é" in str(e), str(e)
big = m.checkpoint_metadata(1, timeout=timedelta(seconds=10))
assert len(big) == 300000 and set(big) == {"x"}
t0 = time.time()
try:
    m.checkpoint_metadata(9, timeout=timedelta(milliseconds=200))
    raise SystemExit("expected a timeout")
except TimeoutError:
    assert time.time() - t0 < 0.9
# the connection survives a cancelled call, and the late response of the old stream is skipped
assert m.should_commit(4, 8, True, timeout=timedelta(seconds=7)) is True
time.sleep(1.0)
assert m.should_commit(4, 9, True, timeout=timedelta(seconds=7)) is True
print("client ok")
"""


def test_our_clients_talk_to_a_grpcio_server():
    S = _schema()
    seen = []
    server = grpc.server(futures.ThreadPoolExecutor(max_workers=4), handlers=[_Generic(S, seen)])
    port = server.add_insecure_port("127.0.0.1:0")
    server.start()
    try:
        # the protocol switch is per process, so the client side runs in a child
        res = subprocess.run([sys.executable, "-c", _CLIENT_SCRIPT, f"http://127.0.0.1:{port}"], capture_output=True,
                             text=True, timeout=120, env=dict(os.environ, PYTHONPATH=ROOT))
        assert res.returncode == 0 and "client ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
        commits = [s for s in seen if s[0].endswith("ShouldCommit")]
        assert [(s[1], s[2], s[3]) for s in commits[:2]] == [(2, 5, True), (3, 6, False)]
        assert 5.0 < commits[0][4] <= 7.0  # grpc-timeout reached the server
    finally:
        server.stop(0)


# ---------------------------------------------------------------- whole path on the gRPC protocol
_E2E_SCRIPT = r"""
import threading
from datetime import timedelta
from torchft_b200 import _control as C
C.set_rpc_protocol("grpc")
C.set_log_enabled(False)
lighthouse = C.Lighthouse(bind="[::]:0", min_replicas=2, join_timeout_ms=200, quorum_tick_ms=10)
managers = [C.Manager(replica_id=f"g{i}", lighthouse_addr=lighthouse.address(), hostname="127.0.0.1", bind="[::]:0",
                      store_addr=f"store{i}", world_size=1, heartbeat_interval=timedelta(milliseconds=100),
                      connect_timeout=timedelta(seconds=5)) for i in range(2)]
out = {}
def run(i):
    c = C.ManagerClient(managers[i].address(), connect_timeout=timedelta(seconds=5))
    for step in range(5):
        q = c.quorum(0, step, f"m{i}", False, timeout=timedelta(seconds=10))
        assert q.replica_world_size == 2 and q.max_step == step, (q.replica_world_size, q.max_step)
        assert c.should_commit(0, step, True, timeout=timedelta(seconds=10))
    out[i] = q.replica_rank
threads = [threading.Thread(target=run, args=(i,)) for i in range(2)]
[t.start() for t in threads]; [t.join(60) for t in threads]
assert sorted(out.values()) == [0, 1], out
for m in managers: m.shutdown()
lighthouse.shutdown()
print("e2e ok")
"""


def test_quorum_and_commit_with_all_clients_on_grpc():
    res = subprocess.run([sys.executable, "-c", _E2E_SCRIPT], capture_output=True, text=True, timeout=180,
                         env=dict(os.environ, PYTHONPATH=ROOT))
    assert res.returncode == 0 and "e2e ok" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_protocol_switch_validation():
    with pytest.raises(ValueError):
        C.set_rpc_protocol("carrier-pigeon")
    assert C.rpc_protocol() in ("framed", "grpc")


# ---------------------------------------------------------------- hand-made frames
def _frame(ftype, flags, stream, payload=b""):
    n = len(payload)
    return bytes([(n >> 16) & 255, (n >> 8) & 255, n & 255, ftype, flags]) + stream.to_bytes(4, "big") + payload


def _read_frames(sock, until_end_of_stream):
    """Reads frames until the given stream carries END_STREAM; returns [(type, flags, stream, payload)]."""
    out, buf = [], b""
    sock.settimeout(10)
    while True:
        while len(buf) < 9:
            chunk = sock.recv(65536)
            assert chunk, "server closed the connection"
            buf += chunk
        n = int.from_bytes(buf[:3], "big")
        while len(buf) < 9 + n:
            chunk = sock.recv(65536)
            assert chunk, "server closed the connection"
            buf += chunk
        ftype, flags, stream = buf[3], buf[4], int.from_bytes(buf[5:9], "big") & 0x7FFFFFFF
        out.append((ftype, flags, stream, buf[9 : 9 + n]))
        buf = buf[9 + n :]
        if stream == until_end_of_stream and ftype in (0, 1) and flags & 0x1:
            return out


def test_continuation_padding_priority_and_split_data():
    """Frame layouts a gRPC library rarely produces: header block in HEADERS + CONTINUATION with
    padding and a priority block, message split over two DATA frames (one padded), PING in between."""
    import socket

    S = _schema()
    lighthouse = C.Lighthouse(bind="[::]:0", min_replicas=1, join_timeout_ms=100, quorum_tick_ms=10)
    try:
        port = int(lighthouse.address().rsplit(":", 1)[1])
        sock = socket.create_connection(("127.0.0.1", port))
        sock.sendall(b"PRI * HTTP/2.0\r\n\r\nSM\r\n\r\n" + _frame(4, 0, 0))
        block = C.hpack_encode([(":method", "POST"), (":scheme", "http"), (":path", "/torchft.LighthouseService/Quorum"),
                                (":authority", "x"), ("te", "trailers"), ("content-type", "application/grpc"),
                                ("grpc-timeout", "5S")], True)
        cut = len(block) // 2
        pad = 7
        headers = bytes([pad]) + b"\x00\x00\x00\x00\x10" + block[:cut] + bytes(pad)  # PADDED | PRIORITY
        sock.sendall(_frame(1, 0x08 | 0x20, 1, headers) + _frame(9, 0x4, 1, block[cut:]))
        member = S.QuorumMember(replica_id="raw", address="a", store_address="s", step=2, world_size=1)
        message = S.LighthouseQuorumRequest(requester=member).SerializeToString()
        body = b"\x00" + len(message).to_bytes(4, "big") + message
        half = len(body) // 2
        sock.sendall(_frame(0, 0x08, 1, bytes([3]) + body[:half] + bytes(3)) + _frame(6, 0, 0, b"12345678") +
                     _frame(0, 0x1, 1, body[half:]))
        frames = _read_frames(sock, until_end_of_stream=1)
        assert any(t == 6 and f & 0x1 and p == b"12345678" for t, f, s, p in frames), "PING was not acknowledged"
        assert any(t == 4 and f & 0x1 for t, f, s, p in frames), "SETTINGS was not acknowledged"
        decoder = C.HpackDecoder()
        blocks = [decoder.decode(p) for t, f, s, p in frames if t == 1 and s == 1]
        assert dict(blocks[0])[b":status"] == b"200" and dict(blocks[0])[b"content-type"] == b"application/grpc"
        assert dict(blocks[-1])[b"grpc-status"] == b"0"
        data = b"".join(p for t, f, s, p in frames if t == 0 and s == 1)
        assert data[0] == 0 and int.from_bytes(data[1:5], "big") == len(data) - 5
        resp = S.LighthouseQuorumResponse.FromString(data[5:])
        assert [p.replica_id for p in resp.quorum.participants] == ["raw"]
        # flow control: the server returned the DATA bytes it consumed to the connection window
        credited = sum(int.from_bytes(p, "big") for t, f, s, p in frames if t == 8 and s == 0)
        assert credited == len(body) + 1 + 3  # both DATA payloads, the pad-length byte and the padding included

        # an even stream id from a client is a protocol error: GOAWAY
        sock.sendall(_frame(1, 0x4 | 0x1, 2, block))
        sock.settimeout(5)
        tail = b""
        try:
            while True:
                chunk = sock.recv(4096)
                if not chunk:
                    break
                tail += chunk
        except OSError:
            pass
        assert len(tail) >= 9 and tail[3] == 7, "expected a GOAWAY frame"
        sock.close()
    finally:
        lighthouse.shutdown()


def test_server_survives_garbage_frames():
    """Random frames after a valid preface must at worst close that connection, never the server."""
    import random
    import socket

    S = _schema()
    lighthouse = C.Lighthouse(bind="[::]:0", min_replicas=1, join_timeout_ms=100, quorum_tick_ms=10)
    try:
        port = int(lighthouse.address().rsplit(":", 1)[1])
        rng = random.Random(1234)
        for conn in range(20):
            sock = socket.create_connection(("127.0.0.1", port))
            sock.settimeout(2)
            try:
                sock.sendall(b"PRI * HTTP/2.0\r\n\r\nSM\r\n\r\n" + _frame(4, 0, 0))
                for _ in range(rng.randint(1, 30)):
                    payload = bytes(rng.getrandbits(8) for _ in range(rng.randint(0, 64)))
                    stream = rng.choice([0, 1, 1, 3, 5, 2, 2**31 - 1])
                    sock.sendall(_frame(rng.randint(0, 11), rng.getrandbits(8), stream, payload))
                if conn % 3 == 0:
                    sock.sendall(bytes(rng.getrandbits(8) for _ in range(100)))  # not even frames
            except OSError:
                pass  # the server hung up on a protocol error: fine
            finally:
                sock.close()
        # truncated preface and a preface with a wrong tail
        for bad in (b"PRI * HT", b"PRI * HTTP/2.0\r\n\r\nXX\r\n\r\n"):
            sock = socket.create_connection(("127.0.0.1", port))
            sock.sendall(bad)
            sock.close()
        with grpc.insecure_channel(f"127.0.0.1:{port}") as ch:
            _unary(ch, "/torchft.LighthouseService/Heartbeat", S.LighthouseHeartbeatRequest(replica_id="after"), S.Empty)
    finally:
        lighthouse.shutdown()


def test_hpack_decoder_on_random_blocks():
    """Random header blocks decode to a list or to None; re-encoding what decoded gives the same headers."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    @settings(max_examples=300, deadline=None)
    @given(block=st.binary(max_size=96))
    def check(block):
        out = C.HpackDecoder().decode(block)
        if out is None:
            return
        headers = [(k.decode("latin-1"), v.decode("latin-1")) for k, v in out]
        if any(ord(ch) > 255 for k, v in headers for ch in k + v):
            return
        # latin-1 text survives the Python <-> C++ string conversion only for ASCII; keep to that
        if not all(k.isascii() and v.isascii() for k, v in headers):
            return
        again = C.HpackDecoder().decode(C.hpack_encode(headers, True))
        assert again == out

    check()

    @settings(max_examples=200, deadline=None)
    @given(data=st.binary(max_size=64))
    def huffman(data):
        assert C.huffman_decode(C.huffman_encode(data)) == data

    huffman()


def test_compressed_request_is_refused_with_unimplemented():
    S = _schema()
    lighthouse = C.Lighthouse(bind="[::]:0", min_replicas=1, join_timeout_ms=100, quorum_tick_ms=10)
    try:
        port = lighthouse.address().rsplit(":", 1)[1]
        with grpc.insecure_channel(f"127.0.0.1:{port}", compression=grpc.Compression.Gzip) as ch:
            with pytest.raises(grpc.RpcError) as err:
                # long enough for the client to bother compressing
                _unary(ch, "/torchft.LighthouseService/Heartbeat", S.LighthouseHeartbeatRequest(replica_id="z" * 4096), S.Empty)
            assert err.value.code() == grpc.StatusCode.UNIMPLEMENTED
        with grpc.insecure_channel(f"127.0.0.1:{port}") as ch:
            _unary(ch, "/torchft.LighthouseService/Heartbeat", S.LighthouseHeartbeatRequest(replica_id="plain"), S.Empty)
    finally:
        lighthouse.shutdown()
