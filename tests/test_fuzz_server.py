"""A server must survive whatever arrives on its port: truncated frames, bodies shorter than the message tail,
random bytes behind a well-formed tail for every request type, counts that point far past the end of the body.
After the barrage the same server still answers a real client correctly. (The reference asserts
`archive().is_exhausted()` after every decode and aborts on a malformed request; a serving process should
answer with an error instead.)"""
import json
import socket
import struct

import numpy as np

from parameter_server_b200 import service as S

DIM = 4


def _frame(payload: bytes, req_id: int = 1, kind: int = 0) -> bytes:
    return struct.pack("<IQB", len(payload), req_id, kind) + payload


def _tail(sid, hid, ver, uver, req_type) -> bytes:
    return struct.pack("<iiiib3x", sid, hid, ver, uver, req_type)   # int8 request type + padding: 20 bytes


def _send(addr, data: bytes, expect_reply: bool):
    host, port = addr.rsplit(":", 1)
    with socket.create_connection((host, int(port)), timeout=5) as s:
        s.sendall(data)
        if expect_reply:
            s.settimeout(5)
            try:
                hdr = s.recv(13)
                if len(hdr) == 13:
                    n = struct.unpack("<I", hdr[:4])[0]
                    while n > 0:
                        chunk = s.recv(min(n, 1 << 16))
                        if not chunk:
                            break
                        n -= len(chunk)
            except socket.timeout:
                pass


def test_server_survives_malformed_requests():
    master = S.Master()
    server = S.Server(master.address())
    client = S.Client(master.address())
    try:
        node = server.node_id()
        cfg = S.storage_config({node: [0, 1, 2]}, dict(dim=DIM, optimizer="sum", init_range=0.0))
        st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", cfg)
        assert st.ok()
        hids = {}
        for key, op, c in [("pull", "SparseTablePullOperator", {}), ("push", "SparseTablePushOperator", {}),
                           ("for_each", "ForEachOperator", {}), ("erase_if", "EraseIfOperator", {}), ("dump", "DumpOperator", {}),
                           ("load", "LoadOperator", {}), ("update_ctx", "ShardUpdateContextOperator", {}), ("sync", "KVSyncOperator", {})]:
            st, hids[key] = client.register_handler(key, S.LIB, op, json.dumps(c), sid)
            assert st.ok()
        keys = np.arange(200, dtype=np.int64)
        vals = np.ones((200, DIM), np.float32) * 3
        assert S.PushHandler(client, sid, hids["push"]).async_push(keys, vals).ok()
        st, ctx_json = client.get_current_ctx(sid)
        ver = json.loads(ctx_json)["version"] if st.ok() else 0
        rng = np.random.default_rng(0)
        for addr in (server.c2s_address(), server.s2s_address()):
            # frames that are not even frames
            _send(addr, b"", False)
            _send(addr, b"\x01\x02\x03", False)
            _send(addr, struct.pack("<IQB", 1000, 7, 0) + b"short", False)          # announces more than it sends
            # bodies shorter than the 20-byte tail
            for n in (0, 1, 19):
                _send(addr, _frame(bytes(rng.integers(0, 256, n, dtype=np.uint8))), True)
            # every request type with a valid tail and garbage / hostile bodies
            for req_type in list(range(0, 26)) + [77, -3]:
                for hid in list(hids.values()) + [-1, 9999]:
                    for body in (b"", bytes(rng.integers(0, 256, 7, dtype=np.uint8)), bytes(rng.integers(0, 256, 200, dtype=np.uint8)),
                                 struct.pack("<iiii", 1, 1, 0, 0x7FFFFFFF) + b"\x00" * 16,        # one shard, one list, count 2^31-1
                                 struct.pack("<iiii", 0x7FFFFFFF, 0x7FFFFFFF, 0, -5),              # absurd shard / merge counts
                                 struct.pack("<q", 1 << 60) + b"abc"):                             # string length 2^60
                        if req_type in (1, 2, 5, 15):   # STORAGE_DELETE / STORAGE_CLEAR / HANDLER_DEREGISTER / EXIT would do what they say
                            continue
                        _send(addr, _frame(body + _tail(sid, hid, ver, -1, req_type)), True)
                        _send(addr, _frame(body + _tail(12345, hid, ver, -1, req_type)), True)  # unknown storage
        # random bodies of random lengths behind a tail that passes every gate (right storage, handler, version)
        by_type = {6: "for_each", 7: "erase_if", 8: "dump", 9: "load", 10: "pull", 11: "push", 12: "push", 13: "push", 16: "update_ctx",
                   17: "update_ctx", 18: "update_ctx", 21: "sync", 23: "pull", 25: "pull"}
        for req_type, key in by_type.items():
            for _ in range(40):
                body = bytes(rng.integers(0, 256, int(rng.integers(0, 300)), dtype=np.uint8))
                if rng.random() < 0.5:      # small plausible counts in front, garbage behind
                    body = struct.pack("<ii", int(rng.integers(0, 4)), int(rng.integers(0, 3))) + body
                _send(server.c2s_address(), _frame(body + _tail(sid, hids[key], ver, -1, req_type)), False)
        # the master gets its share: unknown operations, truncated arguments, absurd lengths, an oversized frame
        maddr = master.address()
        for op in list(range(-2, 24)) + [1000]:
            for body in (b"", bytes(rng.integers(0, 256, 5, dtype=np.uint8)), struct.pack("<q", 1 << 61) + b"xy",
                         struct.pack("<q", 3) + b"abc" + struct.pack("<q", -1)):
                _send(maddr, _frame(struct.pack("<i", op) + body), False)
        _send(maddr, struct.pack("<IQB", 0xFFFFFFF0, 1, 0) + b"x" * 64, False)
        st, nodes = client.get_pserver_list()
        assert st.ok() and node in nodes
        # the server is still there and still right
        st, rows = S.PullHandler(client, sid, hids["pull"]).pull(keys, 10000)
        assert st.ok() and np.array_equal(rows, vals)
        assert client.health_check(node).ok()
    finally:
        server.stop()
        master.stop()


def test_damaged_dump_files_are_reported_not_followed(tmp_path):
    """Truncated and garbled dump files (both codecs) end a load with an error status; nothing hangs or crashes and
    intact files still load."""
    import os
    master = S.Master()
    server = S.Server(master.address())
    client = S.Client(master.address())
    try:
        node = server.node_id()
        cfg = S.storage_config({node: [0, 1]}, dict(dim=DIM, optimizer="sum", init_range=0.0))
        for fmt in ("binary", "archiveline"):
            st, sid = client.create_storage(S.LIB, "SparseTableStorageOperator", cfg)
            assert st.ok()
            h = {}
            for key, op in [("push", "SparseTablePushOperator"), ("pull_ro", "SparseTablePullOperator"), ("dump", "DumpOperator"),
                            ("load", "LoadOperator")]:
                st, h[key] = client.register_handler(key, S.LIB, op, json.dumps({"read_only": True} if key == "pull_ro" else {}), sid)
                assert st.ok()
            keys = np.arange(500, dtype=np.int64)
            assert S.PushHandler(client, sid, h["push"]).async_push(keys, np.ones((500, DIM), np.float32)).ok()
            good = str(tmp_path / f"good_{fmt}")
            assert S.DumpHandler(client, sid, h["dump"]).dump(good + f"?format={fmt}", 1)[0].ok()
            src = os.path.join(good, os.listdir(good)[0])
            raw = open(src, "rb").read()
            rng = np.random.default_rng(1)
            variants = {"truncated": raw[: len(raw) * 2 // 3 + 3], "tail_garbage": raw + bytes(rng.integers(0, 256, 37, dtype=np.uint8)),
                        "garbled": raw[:20] + bytes(rng.integers(0, 256, 300, dtype=np.uint8)) + raw[320:], "empty": b"",
                        "no_newline": raw.rstrip(b"\n")}
            for name, data in variants.items():
                d = tmp_path / f"{fmt}_{name}"
                d.mkdir()
                (d / "model_0_0").write_bytes(data)
                st, n = S.LoadHandler(client, sid, h["load"]).load(str(d) + f"?format={fmt}", 4, 20000)
                if name == "no_newline":
                    assert st.ok() and n == 500, (fmt, name, st, n)       # a missing final newline is not damage
                elif name == "empty" and fmt == "archiveline":
                    assert st.ok() and n == 0
                elif fmt == "binary" and name != "garbled":
                    assert not st.ok(), (fmt, name, st, n)      # a cut record / missing header is noticed
                # garbled bytes of the right length are just other records (the format has no checksum), and text
                # garbage may still parse as numbers: those only have to come back, with whatever status
            st, n = S.LoadHandler(client, sid, h["load"]).load(good + f"?format={fmt}", 4, 20000)
            assert st.ok() and n == 500
            st, rows = S.PullHandler(client, sid, h["pull_ro"]).pull(keys, 10000)
            assert st.ok() and rows.shape == (500, DIM)
    finally:
        server.stop()
        master.stop()


def test_master_refuses_a_damaged_state_file_and_reads_back_its_own(tmp_path):
    import pytest
    from parameter_server_b200 import service as S
    path = tmp_path / "master.state"
    m = S.Master(2, 0, str(path))
    c = S.MasterClient(m.address())
    assert c.generate_id("x")[1] == 0 and c.generate_id("x")[1] == 1
    assert c.set_context("storage/7", '{"a": 1}').ok() and c.tree_node_set("model/m", "{}").ok()
    m.stop()
    again = S.Master(2, 0, str(path), 0)                      # no recovery window: answer at once
    c2 = S.MasterClient(again.address())
    assert c2.generate_id("x")[1] == 2 and c2.get_context("storage/7")[1] == '{"a": 1}' and c2.tree_node_get("model/m")[1] == "{}"
    again.stop()
    good = path.read_bytes()
    rng = np.random.default_rng(3)
    for trial in range(40):
        raw = bytearray(good)
        if trial % 2:
            raw = raw[: int(rng.integers(1, len(raw)))]          # cut short
        else:
            for i in rng.integers(0, len(raw), size=4):
                raw[int(i)] = int(rng.integers(0, 256))          # bytes flipped: lengths and counts go wild
        path.write_bytes(bytes(raw))
        try:
            mm = S.Master(1, 0, str(path), 0)
        except RuntimeError as e:
            assert "master" in str(e)
            continue
        mm.stop()                                                  # damage that still parses is accepted: no crash either way
