"""Encrypted links between services: a TLS 1.3 echo server on a real socket with a certificate chain made on the spot,
the same connection resumed from its ticket, an external pre-shared key for workers that have no certificates, and a
QUIC handshake (TLS 1.3 inside CRYPTO frames) that survives the loss of the server's first flight."""
from _common import seed  # first: makes the package importable from a checkout
import os
import socket
import threading

from sneppx.security import tls13
from sneppx.utils.quic_tls import QuicTlsConnection


def _echo_server(listener, make_server, count):
    for _ in range(count):
        sock, _ = listener.accept()
        conn = tls13.TlsSocket(sock, make_server()).handshake()
        conn.sendall(conn.recv().upper())
        conn.close()


def main() -> dict:
    seed(12)
    out = {}
    root_seed, node_seed = os.urandom(32), os.urandom(32)
    root = tls13.make_certificate(root_seed, "cluster root", ca=True)
    node = tls13.make_certificate(node_seed, "coordinator", issuer_seed=root_seed, issuer="cluster root", dns_names=["coordinator.svc"])
    tickets, worker_key = tls13.TicketStore(), os.urandom(32)
    make_server = lambda: tls13.TlsServer([node, root], node_seed, tickets=tickets, alpn=["sx/1"],
                                          psk_lookup=lambda ident: worker_key if ident == b"worker-3" else None)
    listener = socket.socket()
    listener.bind(("127.0.0.1", 0))
    listener.listen(4)
    thread = threading.Thread(target=_echo_server, args=(listener, make_server, 3), daemon=True)
    thread.start()
    address = listener.getsockname()

    full = tls13.connect(address, server_name="coordinator.svc", trusted_roots=[root], alpn=["sx/1"])
    full.sendall(b"register rank 0")
    out["certificate"] = {"reply": full.recv(), "alpn": full.conn.alpn, "resumed": full.conn.used_psk}
    while not full.conn.sessions and not full.conn.peer_closed:      # the ticket follows the handshake
        full.recv()
    session = full.conn.sessions[0]
    full.close()

    again = tls13.connect(address, server_name="coordinator.svc", session=session)
    again.sendall(b"back again")
    out["ticket"] = {"reply": again.recv(), "resumed": again.conn.used_psk}
    again.close()

    worker = tls13.connect(address, psk=(b"worker-3", worker_key))
    worker.sendall(b"no certificate needed")
    out["psk"] = {"reply": worker.recv(), "psk": worker.conn.used_psk}
    worker.close()
    thread.join(5)
    listener.close()

    try:
        wrong_root = tls13.TlsClient("coordinator.svc", trusted_roots=[tls13.make_certificate(os.urandom(32), "cluster root", ca=True)])
        server = make_server()
        wrong_root.start()
        server.receive(wrong_root.data_to_send())
        wrong_root.receive(server.data_to_send())
        out["impostor_root"] = "accepted"
    except tls13.TlsError as e:
        out["impostor_root"] = str(e)

    client = QuicTlsConnection.client(["sx/1"], server_name="coordinator.svc", trusted_roots=[root])
    hello = client.datagrams_to_send()
    server = QuicTlsConnection.accept(hello[0], lambda params: tls13.TlsServer([node, root], node_seed, alpn=["sx/1"],
                                                                               quic_transport_parameters=params))
    lost = server.datagrams_to_send()                      # the server's first flight never arrives
    server.on_timeout()
    client.on_timeout()
    for _ in range(4):
        for d in client.datagrams_to_send():
            server.receive_datagram(d)
        for d in server.datagrams_to_send():
            client.receive_datagram(d)
    client.send_stream(0, b"gradient shard", fin=True)
    for d in client.datagrams_to_send():
        server.receive_datagram(d)
    out["quic"] = {"first_datagram": len(hello[0]), "lost": len(lost), "confirmed": client.handshake_confirmed,
                   "stream": bytes(server.streams[0]), "keys_left": [l for l, s in client.spaces.items() if s.protector is not None]}
    for k, v in out.items():
        print(f"{k}: {v}")
    return out


if __name__ == "__main__":
    main()
