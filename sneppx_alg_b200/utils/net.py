"""Bindings of the C++ network components (``csrc/host/net.cpp``): rank topology and routes, framed TCP messages with
tensor transfer, rendezvous coordinator, Raft cluster core, health checks, WebSocket / MQTT codecs and a service
directory.

Reference counterparts: ``net/topology.c``, ``net/socket/socket_comm.c``, ``net/grpc/grpc_service.c``,
``net/consensus/raft.c``, ``net/monitoring/health_check.c``, ``net/websocket/websocket_client.c``,
``net/mqtt/mqtt_client.c``, ``net/dns/sd_client.c`` and the Python wrapper ``net_bindings.py``. The reference's QUIC and
RDMA shells have no counterpart: between GPUs of a node the transport is NVLink through NCCL and the peer-memory
kernels, and the control plane here is TCP.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Tuple

import numpy as np

from .. import _build

_DTYPES = [np.float32, np.float64, np.float16, np.int32, np.int64, np.uint8, np.int8, np.uint16]


def _L():
    L = _build.load_host()
    if not getattr(L, "_net_ready", False):
        for f in ("sx_topo_ring", "sx_topo_tree", "sx_topo_graph", "sx_coord_server_start", "sx_coord_connect",
                  "sx_raft_cluster_create", "sx_health_create", "sx_sd_create"):
            getattr(L, f).restype = C.c_void_p
        for f in ("sx_topo_destroy", "sx_coord_server_stop", "sx_coord_server_port", "sx_coord_close", "sx_coord_world",
                  "sx_coord_rank", "sx_coord_barrier", "sx_raft_cluster_destroy", "sx_raft_cluster_leader",
                  "sx_health_destroy", "sx_sd_destroy"):
            getattr(L, f).argtypes = [C.c_void_p]
        L.sx_topo_graph.argtypes = [C.c_int, C.c_void_p]
        for f in ("sx_topo_next", "sx_topo_prev", "sx_topo_parent"):
            getattr(L, f).argtypes = [C.c_void_p, C.c_int]
        L.sx_topo_children.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        L.sx_topo_route.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int]
        L.sx_sock_listen.argtypes = [C.c_int, C.c_void_p]
        L.sx_sock_connect.argtypes = [C.c_char_p, C.c_int, C.c_int]
        L.sx_sock_send_message.argtypes = [C.c_int, C.c_void_p, C.c_longlong]
        L.sx_sock_recv_message.argtypes = [C.c_int, C.c_void_p, C.c_longlong]
        L.sx_sock_recv_message.restype = C.c_longlong
        L.sx_sock_send_tensor.argtypes = [C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_longlong]
        L.sx_sock_recv_tensor.argtypes = [C.c_int, C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]
        L.sx_sock_recv_tensor.restype = C.c_longlong
        L.sx_coord_server_start.argtypes = [C.c_int, C.c_int, C.c_char_p]
        L.sx_coord_connect.argtypes = [C.c_char_p, C.c_int, C.c_int]
        L.sx_coord_error.argtypes = [C.c_void_p]
        L.sx_coord_error.restype = C.c_char_p
        L.sx_coord_register.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p]
        L.sx_coord_all_gather.argtypes = [C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]
        L.sx_coord_send.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_longlong]
        L.sx_coord_recv.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_longlong, C.c_int]
        L.sx_coord_recv.restype = C.c_longlong
        L.sx_raft_cluster_create.argtypes = [C.c_int, C.c_int, C.c_int, C.c_ulonglong]
        L.sx_raft_cluster_step.argtypes = [C.c_void_p, C.c_int]
        L.sx_raft_cluster_set_connected.argtypes = [C.c_void_p, C.c_int, C.c_int]
        L.sx_raft_cluster_propose.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_longlong]
        L.sx_raft_cluster_state.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.sx_raft_cluster_entry.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_longlong]
        L.sx_raft_cluster_entry.restype = C.c_longlong
        L.sx_health_create.argtypes = [C.c_double, C.c_int]
        L.sx_health_report.argtypes = [C.c_void_p, C.c_int, C.c_double, C.c_int, C.c_double]
        L.sx_health_status.argtypes = [C.c_void_p, C.c_int, C.c_double]
        L.sx_health_latency.argtypes = [C.c_void_p, C.c_int]
        L.sx_health_latency.restype = C.c_double
        L.sx_sha1.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p]
        L.sx_ws_accept_key.argtypes = [C.c_char_p, C.c_void_p]
        L.sx_ws_encode.argtypes = [C.c_int, C.c_void_p, C.c_longlong, C.c_uint, C.c_void_p, C.c_longlong]
        L.sx_ws_encode.restype = C.c_longlong
        L.sx_ws_decode.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p, C.c_longlong, C.c_void_p]
        L.sx_ws_decode.restype = C.c_longlong
        L.sx_mqtt_connect.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_void_p, C.c_longlong]
        L.sx_mqtt_publish.argtypes = [C.c_char_p, C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_longlong]
        L.sx_mqtt_subscribe.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_void_p, C.c_longlong]
        for f in ("sx_mqtt_connect", "sx_mqtt_publish", "sx_mqtt_subscribe", "sx_mqtt_parse_publish"):
            getattr(L, f).restype = C.c_longlong
        L.sx_mqtt_parse_header.argtypes = [C.c_void_p, C.c_longlong, C.c_void_p, C.c_void_p, C.c_void_p]
        L.sx_mqtt_parse_publish.argtypes = [C.c_void_p, C.c_longlong, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
        L.sx_mqtt_topic_match.argtypes = [C.c_char_p, C.c_char_p]
        L.sx_sd_register.argtypes = [C.c_void_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_int, C.c_char_p, C.c_double, C.c_double]
        L.sx_sd_unregister.argtypes = [C.c_void_p, C.c_char_p]
        L.sx_sd_browse.argtypes = [C.c_void_p, C.c_char_p, C.c_double, C.c_void_p, C.c_int]
        L._net_ready = True
    return L


class Topology:
    """Ring, k-ary tree or arbitrary graph over ranks, with hop routes (breadth-first)."""

    def __init__(self, handle, world):
        if not handle:
            raise ValueError("invalid topology arguments")
        self._h, self.world = handle, world

    @classmethod
    def ring(cls, world: int):
        return cls(_L().sx_topo_ring(world), world)

    @classmethod
    def tree(cls, world: int, branching: int = 2):
        return cls(_L().sx_topo_tree(world, branching), world)

    @classmethod
    def graph(cls, adjacency):
        a = np.ascontiguousarray(adjacency, dtype=np.int32)
        return cls(_L().sx_topo_graph(a.shape[0], a.ctypes.data), a.shape[0])

    def next(self, rank):
        return _L().sx_topo_next(self._h, rank)

    def prev(self, rank):
        return _L().sx_topo_prev(self._h, rank)

    def parent(self, rank):
        return _L().sx_topo_parent(self._h, rank)

    def children(self, rank) -> List[int]:
        out = (C.c_int * 64)()
        n = _L().sx_topo_children(self._h, rank, out, 64)
        return list(out[:max(n, 0)])

    def route(self, src, dst) -> Optional[List[int]]:
        out = (C.c_int * max(self.world, 1))()
        n = _L().sx_topo_route(self._h, src, dst, out, self.world)
        return list(out[:n]) if n > 0 else None

    def __del__(self):
        try:
            _L().sx_topo_destroy(self._h)
        except Exception:
            pass


class FramedSocket:
    """Length-prefixed messages and tensors over one TCP connection (loopback listener)."""

    def __init__(self, fd: int):
        if fd < 0:
            raise ConnectionError("socket not connected")
        self.fd = fd

    @staticmethod
    def listen(port: int = 0) -> Tuple[int, int]:
        bound = C.c_int(0)
        fd = _L().sx_sock_listen(port, C.byref(bound))
        if fd < 0:
            raise OSError("cannot listen")
        return fd, bound.value

    @classmethod
    def accept(cls, listen_fd: int, timeout_ms: int = 5000):
        return cls(_L().sx_sock_accept(listen_fd, timeout_ms))

    @classmethod
    def connect(cls, host: str, port: int, timeout_ms: int = 5000):
        return cls(_L().sx_sock_connect(host.encode(), port, timeout_ms))

    def set_timeout(self, ms: int):
        _L().sx_sock_set_timeout(self.fd, ms)

    def send_message(self, data: bytes):
        if _L().sx_sock_send_message(self.fd, data, len(data)):
            raise ConnectionError("send failed")

    def recv_message(self, cap: int = 1 << 20) -> bytes:
        buf = C.create_string_buffer(cap)
        n = _L().sx_sock_recv_message(self.fd, buf, cap)
        if n == -1:
            raise ConnectionError("peer closed or timed out")
        if n < 0:
            raise BufferError(f"message of {-n - 2} bytes exceeds the {cap}-byte buffer")
        return buf.raw[:n]

    def send_tensor(self, a: np.ndarray):
        a = np.ascontiguousarray(a)
        code = [np.dtype(d) for d in _DTYPES].index(a.dtype)
        dims = (C.c_longlong * max(a.ndim, 1))(*a.shape)
        if _L().sx_sock_send_tensor(self.fd, a.ctypes.data, code, a.ndim, dims, a.nbytes):
            raise ConnectionError("send failed")

    def recv_tensor(self, max_bytes: int = 1 << 28) -> np.ndarray:
        buf = np.empty(max_bytes, dtype=np.uint8)
        dt, nd = C.c_int(0), C.c_int(0)
        dims = (C.c_longlong * 8)()
        n = _L().sx_sock_recv_tensor(self.fd, buf.ctypes.data, max_bytes, C.byref(dt), C.byref(nd), dims, 8)
        if n < 0:
            raise ConnectionError("tensor receive failed")
        return buf[:n].view(_DTYPES[dt.value]).reshape(tuple(dims[: nd.value])).copy()

    def close(self):
        if self.fd >= 0:
            _L().sx_sock_close(self.fd)
            self.fd = -1


def close_listener(fd: int):
    _L().sx_sock_close(fd)


class CoordinatorServer:
    """Rendezvous service for `world` ranks; stops and joins its threads on ``stop()``."""

    def __init__(self, world: int, token: str = "", port: int = 0):
        self._h = _L().sx_coord_server_start(port, world, token.encode())
        if not self._h:
            raise OSError("cannot start coordinator")
        self.port = _L().sx_coord_server_port(self._h)

    def stop(self):
        if self._h:
            _L().sx_coord_server_stop(self._h)
            self._h = None


class CoordinatorClient:
    def __init__(self, host: str, port: int, token: str = "", name: str = "", timeout_ms: int = 5000):
        self._h = _L().sx_coord_connect(host.encode(), port, timeout_ms)
        if not self._h:
            raise ConnectionError(f"cannot reach coordinator {host}:{port}")
        rc = _L().sx_coord_register(self._h, token.encode(), name.encode())
        if rc < 0:
            err = _L().sx_coord_error(self._h).decode()
            self.close()
            raise PermissionError(err) if "unauth" in err else ConnectionError(err)
        self.rank, self.world = rc, _L().sx_coord_world(self._h)

    def _check(self, rc):
        if rc < 0:
            raise ConnectionError(_L().sx_coord_error(self._h).decode() or f"coordinator error {rc}")

    def barrier(self):
        self._check(_L().sx_coord_barrier(self._h))

    def all_gather(self, data: bytes) -> List[bytes]:
        out = C.create_string_buffer(len(data) * self.world)
        self._check(_L().sx_coord_all_gather(self._h, data, len(data), out))
        return [out.raw[i * len(data):(i + 1) * len(data)] for i in range(self.world)]

    def send(self, dst: int, data: bytes):
        self._check(_L().sx_coord_send(self._h, dst, data, len(data)))

    def recv(self, src: int, cap: int = 1 << 20, timeout_ms: int = 5000) -> bytes:
        buf = C.create_string_buffer(cap)
        n = _L().sx_coord_recv(self._h, src, buf, cap, timeout_ms)
        if n == -2 and "timeout" in _L().sx_coord_error(self._h).decode():
            raise TimeoutError(f"nothing from rank {src} within {timeout_ms} ms")
        self._check(n)
        return buf.raw[:n]

    def close(self):
        if self._h:
            _L().sx_coord_close(self._h)
            self._h = None


class RaftCluster:
    """N Raft nodes on an in-memory network. ``step(ms)`` advances every connected node's clock and delivers messages;
    ``set_connected`` cuts a node off (its messages are dropped both ways) to exercise re-election and log repair."""

    ROLES = ("follower", "candidate", "leader")

    def __init__(self, n: int, election_ms: int = 150, heartbeat_ms: int = 50, seed: int = 0):
        self.n = n
        self._h = _L().sx_raft_cluster_create(n, election_ms, heartbeat_ms, seed)

    def step(self, ms: int = 10, times: int = 1):
        for _ in range(times):
            _L().sx_raft_cluster_step(self._h, ms)

    def leader(self) -> int:
        return _L().sx_raft_cluster_leader(self._h)

    def propose(self, node: int, data: bytes) -> int:
        return _L().sx_raft_cluster_propose(self._h, node, data, len(data))

    def set_connected(self, node: int, on: bool):
        _L().sx_raft_cluster_set_connected(self._h, node, int(on))

    def state(self, node: int) -> dict:
        out = (C.c_int * 6)()
        _L().sx_raft_cluster_state(self._h, node, out)
        return {"term": out[0], "commit_index": out[1], "last_applied": out[2], "role": self.ROLES[out[3]],
                "log_length": out[4], "leader": out[5]}

    def entry(self, node: int, index: int) -> Optional[bytes]:
        buf = C.create_string_buffer(4096)
        n = _L().sx_raft_cluster_entry(self._h, node, index, buf, 4096)
        return buf.raw[:n] if n >= 0 else None

    def committed(self, node: int) -> List[bytes]:
        return [self.entry(node, i) for i in range(1, self.state(node)["commit_index"] + 1)]

    def __del__(self):
        try:
            _L().sx_raft_cluster_destroy(self._h)
        except Exception:
            pass


class HealthChecker:
    def __init__(self, timeout_ms: float = 3000.0, max_failures: int = 3):
        self._h = _L().sx_health_create(timeout_ms, max_failures)

    def report(self, node: int, now_ms: float, ok: bool = True, latency_ms: float = 0.0):
        _L().sx_health_report(self._h, node, now_ms, int(ok), latency_ms)

    def status(self, node: int, now_ms: float) -> str:
        return {1: "healthy", 0: "unhealthy", -1: "unknown"}[_L().sx_health_status(self._h, node, now_ms)]

    def latency(self, node: int) -> float:
        return _L().sx_health_latency(self._h, node)

    def __del__(self):
        try:
            _L().sx_health_destroy(self._h)
        except Exception:
            pass


def sha1(data: bytes) -> bytes:
    out = C.create_string_buffer(20)
    _L().sx_sha1(data, len(data), out)
    return out.raw


def ws_accept_key(client_key: str) -> str:
    out = C.create_string_buffer(32)
    _L().sx_ws_accept_key(client_key.encode(), out)
    return out.value.decode()


def ws_encode(payload: bytes, opcode: int = 1, mask_key: int = 0) -> bytes:
    cap = len(payload) + 16
    out = C.create_string_buffer(cap)
    n = _L().sx_ws_encode(opcode, payload, len(payload), mask_key, out, cap)
    return out.raw[:n]


def ws_decode(data: bytes):
    """Returns (consumed, opcode, fin, payload) or None when the frame is incomplete."""
    op, fin, plen = C.c_int(0), C.c_int(0), C.c_longlong(0)
    out = C.create_string_buffer(max(len(data), 1))
    n = _L().sx_ws_decode(data, len(data), C.byref(op), C.byref(fin), out, len(data), C.byref(plen))
    if n == 0:
        return None
    if n < 0:
        raise ValueError("malformed WebSocket frame")
    return n, op.value, bool(fin.value), out.raw[: plen.value]


def mqtt_connect(client_id: str, keepalive_s: int = 60, clean: bool = True) -> bytes:
    out = C.create_string_buffer(512)
    n = _L().sx_mqtt_connect(client_id.encode(), keepalive_s, int(clean), out, 512)
    return out.raw[:n]


def mqtt_publish(topic: str, payload: bytes, qos: int = 0, retain: bool = False, packet_id: int = 0) -> bytes:
    cap = len(payload) + len(topic) + 16
    out = C.create_string_buffer(cap)
    n = _L().sx_mqtt_publish(topic.encode(), payload, len(payload), qos, int(retain), packet_id, out, cap)
    return out.raw[:n]


def mqtt_subscribe(topic_filter: str, qos: int = 0, packet_id: int = 1) -> bytes:
    out = C.create_string_buffer(len(topic_filter) + 16)
    n = _L().sx_mqtt_subscribe(topic_filter.encode(), qos, packet_id, out, len(topic_filter) + 16)
    return out.raw[:n]


def mqtt_parse(packet: bytes) -> dict:
    ty, fl, rem = C.c_int(0), C.c_int(0), C.c_longlong(0)
    h = _L().sx_mqtt_parse_header(packet, len(packet), C.byref(ty), C.byref(fl), C.byref(rem))
    if h <= 0:
        raise ValueError("incomplete or malformed MQTT header")
    d = {"type": ty.value, "flags": fl.value, "remaining": rem.value, "header_len": h}
    if ty.value == 3:
        body = packet[h:h + rem.value]
        topic, pid = C.create_string_buffer(1024), C.c_int(0)
        off = _L().sx_mqtt_parse_publish(body, len(body), fl.value, topic, 1024, C.byref(pid))
        if off < 0:
            raise ValueError("malformed PUBLISH")
        d.update(topic=topic.value.decode(), packet_id=pid.value, payload=body[off:], qos=(fl.value >> 1) & 3)
    return d


def mqtt_topic_match(topic_filter: str, topic: str) -> bool:
    return bool(_L().sx_mqtt_topic_match(topic_filter.encode(), topic.encode()))


class ServiceDirectory:
    """DNS-SD-style records (name, type, host, port, TXT) with a time-to-live."""

    def __init__(self):
        self._h = _L().sx_sd_create()

    def register(self, name, type_, host, port, txt="", now_ms=0.0, ttl_ms=120000.0):
        _L().sx_sd_register(self._h, name.encode(), type_.encode(), host.encode(), port, txt.encode(), now_ms, ttl_ms)

    def unregister(self, name) -> bool:
        return bool(_L().sx_sd_unregister(self._h, name.encode()))

    def browse(self, type_, now_ms=0.0) -> List[dict]:
        buf = C.create_string_buffer(1 << 16)
        _L().sx_sd_browse(self._h, type_.encode(), now_ms, buf, 1 << 16)
        out = []
        for line in buf.value.decode().splitlines():
            name, host, port, txt = line.split("\t")
            out.append({"name": name, "host": host, "port": int(port), "txt": txt})
        return out

    def __del__(self):
        try:
            _L().sx_sd_destroy(self._h)
        except Exception:
            pass


class RDMA:
    """One-sided read / write of registered memory regions between processes of one host, over POSIX shared memory.

    The reference's ``RDMA`` (``net_bindings.py:193-225``) is a shell whose ``read`` / ``write`` return 0. Between GPUs
    the one-sided transport of this framework is NVLink peer memory (``torch.distributed._symmetric_memory`` buffers
    read and written by the fused kernels); this class gives host memory the same shape: a process registers a region
    under a key, any other process attaches by key and reads or writes it at an offset with no involvement of the
    owner. Ordering between writer and reader is the caller's business (a flag word in the region, or the
    coordinator's barrier), as with real RDMA."""

    def __init__(self):
        self._regions = {}
        self._owned = set()
        self._open = False

    def open(self, device_idx: int = 0) -> bool:
        self._open = True
        return True

    def register_memory(self, key: str, nbytes: int = 0, array: Optional[np.ndarray] = None) -> np.ndarray:
        """Creates the shared region `key` (initialised from `array` when given) and returns a NumPy view of it."""
        from multiprocessing import shared_memory
        if not self._open:
            raise RuntimeError("open() first")
        nbytes = int(array.nbytes if array is not None else nbytes)
        shm = shared_memory.SharedMemory(name=key, create=True, size=max(nbytes, 1))
        self._regions[key] = shm
        self._owned.add(key)
        view = np.ndarray((nbytes,), dtype=np.uint8, buffer=shm.buf)
        if array is not None:
            view[:] = np.frombuffer(np.ascontiguousarray(array).tobytes(), dtype=np.uint8)
        return view

    def attach(self, key: str):
        from multiprocessing import shared_memory
        if key not in self._regions:
            self._regions[key] = shared_memory.SharedMemory(name=key)
        return self._regions[key]

    def read(self, key: str, remote_offset: int, local: np.ndarray, length: Optional[int] = None) -> int:
        """Copies `length` bytes at `remote_offset` of region `key` into `local`; returns the byte count."""
        shm = self.attach(key)
        dst = local.reshape(-1).view(np.uint8)
        length = dst.nbytes if length is None else int(length)
        if remote_offset < 0 or remote_offset + length > shm.size or length > dst.nbytes:
            raise ValueError("read outside the registered region or the local buffer")
        dst[:length] = np.frombuffer(shm.buf, dtype=np.uint8, count=length, offset=remote_offset)
        return length

    def write(self, key: str, remote_offset: int, local: np.ndarray, length: Optional[int] = None) -> int:
        shm = self.attach(key)
        src = np.ascontiguousarray(local).reshape(-1).view(np.uint8)
        length = src.nbytes if length is None else int(length)
        if remote_offset < 0 or remote_offset + length > shm.size or length > src.nbytes:
            raise ValueError("write outside the registered region or the local buffer")
        np.frombuffer(shm.buf, dtype=np.uint8, count=length, offset=remote_offset)[:] = src[:length]
        return length

    def deregister_memory(self, key: Optional[str] = None):
        for k in ([key] if key else list(self._regions)):
            shm = self._regions.pop(k, None)
            if shm is None:
                continue
            shm.close()
            if k in self._owned:
                self._owned.discard(k)
                try:
                    shm.unlink()
                except FileNotFoundError:
                    pass

    def close(self):
        self.deregister_memory()
        self._open = False


class SecureStreamConnection:
    """Encrypted connection with independent numbered streams (the reference's QUIC shell, ``net/quic/quic_transport.h``:
    listener / dial / stream_open / stream_send / stream_recv; its body opens no socket).

    Not the QUIC wire protocol: the carrier is one framed TCP connection. What it keeps of QUIC's shape is what callers
    use: a key agreement when the connection opens (ephemeral X25519, optionally combined with ML-KEM-768 so that the
    session keys also resist an attacker with a quantum computer; HKDF-SHA256, one key per direction), every frame
    sealed with ChaCha20-Poly1305 under a per-direction counter nonce (replayed, reordered or altered frames fail
    authentication), and any number of streams multiplexed on the connection so that a large transfer on one stream
    does not have to finish before a message on another is read."""

    def __init__(self, sock: FramedSocket, initiator: bool, psk: bytes = b"", post_quantum: bool = False):
        try:
            self._handshake(sock, initiator, psk, post_quantum)
        except Exception:
            sock.close()                      # the peer must not be left waiting for the rest of a failed handshake
            raise

    def _handshake(self, sock, initiator, psk, post_quantum):
        import os
        from collections import defaultdict, deque
        from ..security import crypto
        self._crypto, self.sock = crypto, sock
        secret = os.urandom(32)
        mine = crypto.x25519(secret)
        kem_secret = b""
        if post_quantum and initiator:
            # hybrid key agreement: the initiator adds an ML-KEM-768 encapsulation key, the acceptor answers with a
            # ciphertext; the session keys depend on both the X25519 and the ML-KEM secrets
            ek, dk = crypto.mlkem_keygen(768)
            sock.send_message(mine + ek)
            reply = sock.recv_message(4096)
            if len(reply) != 32 + crypto.mlkem_sizes(768)[2]:
                raise ConnectionError("bad handshake")
            theirs, kem_secret = reply[:32], crypto.mlkem_decaps(dk, reply[32:], 768)
        elif post_quantum:
            hello = sock.recv_message(4096)
            if len(hello) != 32 + crypto.mlkem_sizes(768)[0]:
                raise ConnectionError("bad handshake")
            theirs = hello[:32]
            try:
                kem_secret, ct = crypto.mlkem_encaps(hello[32:], 768)
            except ValueError as e:
                raise ConnectionError("bad handshake") from e
            sock.send_message(mine + ct)
        else:
            sock.send_message(mine)
            theirs = sock.recv_message(64)
            if len(theirs) != 32:
                raise ConnectionError("bad handshake")
        shared = crypto.x25519(secret, theirs) + kem_secret
        first, second = (mine, theirs) if initiator else (theirs, mine)
        okm = crypto.hkdf_sha256(shared + psk, salt=first + second, info=b"sneppx-stream", length=64)
        self._send_key, self._recv_key = (okm[:32], okm[32:]) if initiator else (okm[32:], okm[:32])
        self._send_ctr = self._recv_ctr = 0
        self._next_stream = 0 if initiator else 1          # initiator opens even ids, acceptor odd ids
        self._queues = defaultdict(deque)
        self._closed = set()
        # key confirmation: a peer with another pre-shared key fails here, not at the first payload
        self._send_frame(0xFFFFFFFF, 2, b"confirm")
        sid, kind, body = self._recv_frame()
        if (sid, kind, body) != (0xFFFFFFFF, 2, b"confirm"):
            raise ConnectionError("key confirmation failed")

    @classmethod
    def dial(cls, host: str, port: int, timeout_ms: int = 5000, psk: bytes = b"", post_quantum: bool = False):
        sock = FramedSocket.connect(host, port, timeout_ms)
        sock.set_timeout(timeout_ms)
        return cls(sock, True, psk, post_quantum)

    @classmethod
    def accept(cls, listen_fd: int, timeout_ms: int = 5000, psk: bytes = b"", post_quantum: bool = False):
        sock = FramedSocket.accept(listen_fd, timeout_ms)
        sock.set_timeout(timeout_ms)
        return cls(sock, False, psk, post_quantum)

    def _send_frame(self, stream_id: int, kind: int, body: bytes):
        nonce = self._send_ctr.to_bytes(12, "little")
        self._send_ctr += 1
        head = stream_id.to_bytes(4, "little") + bytes([kind])
        self.sock.send_message(head + self._crypto.aead_encrypt(self._send_key, nonce, body, head))

    def _recv_frame(self):
        raw = self.sock.recv_message(1 << 24)
        nonce = self._recv_ctr.to_bytes(12, "little")
        self._recv_ctr += 1
        head = raw[:5]
        try:
            body = self._crypto.aead_decrypt(self._recv_key, nonce, raw[5:], head)
        except Exception as e:
            raise ConnectionError("frame failed authentication") from e
        return int.from_bytes(head[:4], "little"), head[4], body

    def stream_open(self) -> int:
        sid = self._next_stream
        self._next_stream += 2
        return sid

    def stream_send(self, stream_id: int, data: bytes, chunk: int = 1 << 20):
        for off in range(0, max(len(data), 1), chunk):
            self._send_frame(stream_id, 0, data[off:off + chunk])

    def stream_close(self, stream_id: int):
        self._send_frame(stream_id, 1, b"")

    def stream_recv(self, stream_id: int, timeout_ms: int = 5000):
        """Next chunk of `stream_id`, or None once the peer closed that stream. Frames of other streams that arrive in
        the meantime are queued for their own readers."""
        self.sock.set_timeout(timeout_ms)
        while not self._queues[stream_id]:
            if stream_id in self._closed:
                return None
            sid, kind, body = self._recv_frame()
            if kind == 1:
                self._closed.add(sid)
            else:
                self._queues[sid].append(body)
        return self._queues[stream_id].popleft()

    def close(self):
        self.sock.close()
