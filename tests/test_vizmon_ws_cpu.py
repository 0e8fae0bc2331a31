"""Dashboard store (native) and the live WebSocket feed: summaries, incremental snapshots, handshake and frames."""
import base64
import json
import os
import socket
import struct
import time

from sneppx_alg_b200.utils.net import ws_accept_key
from sneppx_alg_b200.utils.vizmon import VizMon


def _read_frame(sock):
    hdr = sock.recv(2)
    n = hdr[1] & 0x7F
    if n == 126:
        n = struct.unpack(">H", sock.recv(2))[0]
    elif n == 127:
        n = struct.unpack(">Q", sock.recv(8))[0]
    data = b""
    while len(data) < n:
        data += sock.recv(n - len(data))
    return hdr[0] & 0x0F, data


def test_native_store_summaries_and_incremental_reads():
    mon = VizMon(history=100)
    for i in range(250):
        mon.scalar("loss", 10.0 / (i + 1), step=i)
    s = mon.summary("loss")
    assert s["count"] == 100 and s["total"] == 250 and abs(s["last"] - 10 / 250) < 1e-12 and s["min"] == s["last"]
    assert s["max"] == 10 / 151 and s["p50"] <= s["p95"] <= s["max"] and mon.summary("nope") is None
    full = mon.updates_since(0)
    assert len(full["scalars"]["loss"]) == 100 and full["scalars"]["loss"][-1][0] == 249 and full["seq"] == 250
    mon.scalar("lr", 3e-4)
    with mon.span('step "quoted"'):
        pass
    inc = mon.updates_since(full["seq"])
    assert list(inc["scalars"]) == ["lr"] and inc["spans"][0]["name"] == 'step "quoted"' and inc["seq"] == 252
    assert mon.updates_since(inc["seq"]) == {"seq": 252, "scalars": {}, "spans": []}


def test_websocket_feed():
    mon = VizMon()
    mon.scalar("tokens_per_s", 1000.0, step=0)
    port = mon.serve(ws_interval=0.05)
    key = base64.b64encode(os.urandom(16)).decode()
    s = socket.create_connection(("127.0.0.1", port), timeout=5)
    s.sendall((f"GET /ws HTTP/1.1\r\nHost: x\r\nUpgrade: websocket\r\nConnection: Upgrade\r\n"
               f"Sec-WebSocket-Key: {key}\r\nSec-WebSocket-Version: 13\r\n\r\n").encode())
    head = b""
    while b"\r\n\r\n" not in head:
        head += s.recv(1)
    assert b"101" in head.split(b"\r\n")[0] and ws_accept_key(key).encode() in head
    op, data = _read_frame(s)
    first = json.loads(data)
    assert op == 1 and first["scalars"]["tokens_per_s"] == [[0, 1000.0, first["scalars"]["tokens_per_s"][0][2]]]
    mon.scalar("tokens_per_s", 1200.0, step=1)
    op, data = _read_frame(s)
    upd = json.loads(data)
    assert [p[:2] for p in upd["scalars"]["tokens_per_s"]] == [[1, 1200.0]] and upd["seq"] == first["seq"] + 1
    assert mon.ws_clients == 1
    s.close()
    # a plain GET of /ws is refused; the page still serves
    import urllib.request
    import urllib.error
    try:
        urllib.request.urlopen(f"http://127.0.0.1:{port}/ws", timeout=5)
        assert False
    except urllib.error.HTTPError as e:
        assert e.code == 400
    assert b"WebSocket" in urllib.request.urlopen(f"http://127.0.0.1:{port}/", timeout=5).read()
    mon.stop()
    time.sleep(0.1)
