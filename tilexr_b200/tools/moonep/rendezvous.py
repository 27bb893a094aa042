"""Completion barrier over TCP with HMAC-framed messages (reference: tools/moonep/rendezvous.py).

Ranks that finished a harness run tell rank 0 and wait for its release, so no rank tears its communicator down
while a peer may still read its memory.  Frames are `length | payload | HMAC-SHA256(key, payload)`; a frame with
a wrong digest is dropped, so a stray connection cannot release the barrier."""
from __future__ import annotations

import hashlib
import hmac
import json
import socket
import struct
import time
from typing import Dict, Optional


def _send(sock: socket.socket, key: bytes, obj: Dict[str, object]) -> None:
    payload = json.dumps(obj, sort_keys=True).encode()
    sock.sendall(struct.pack("!I", len(payload)) + payload + hmac.new(key, payload, hashlib.sha256).digest())


def _recv_exact(sock: socket.socket, n: int) -> Optional[bytes]:
    buf = b""
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            return None
        buf += chunk
    return buf


def _recv(sock: socket.socket, key: bytes) -> Optional[Dict[str, object]]:
    head = _recv_exact(sock, 4)
    if head is None:
        return None
    (n,) = struct.unpack("!I", head)
    if n > 1 << 20:
        return None
    body = _recv_exact(sock, n + 32)
    if body is None:
        return None
    payload, digest = body[:n], body[n:]
    if not hmac.compare_digest(digest, hmac.new(key, payload, hashlib.sha256).digest()):
        return None
    return json.loads(payload)


def completion_barrier(rank: int, world: int, host: str, port: int, key: bytes, tag: str, timeout_s: float = 60.0) -> bool:
    """Returns True when all `world` ranks reached the barrier named `tag` within the timeout."""
    if world == 1:
        return True
    deadline = time.time() + timeout_s
    if rank == 0:
        server = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        server.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        server.bind((host, port))
        server.listen(world)
        peers = {}
        try:
            while len(peers) < world - 1:
                server.settimeout(max(0.05, deadline - time.time()))
                try:
                    conn, _ = server.accept()
                except socket.timeout:
                    return False
                conn.settimeout(max(0.05, deadline - time.time()))
                msg = _recv(conn, key)
                if msg is None or msg.get("tag") != tag or not isinstance(msg.get("rank"), int) or msg["rank"] in peers:
                    conn.close()               # unauthenticated, wrong barrier or duplicate: ignored
                    continue
                peers[msg["rank"]] = conn
            for conn in peers.values():
                _send(conn, key, {"tag": tag, "release": True})
            return True
        finally:
            for conn in peers.values():
                conn.close()
            server.close()
    while time.time() < deadline:
        try:
            with socket.create_connection((host, port), timeout=1.0) as s:
                s.settimeout(max(0.05, deadline - time.time()))
                _send(s, key, {"tag": tag, "rank": rank})
                msg = _recv(s, key)
                return bool(msg and msg.get("tag") == tag and msg.get("release"))
        except (ConnectionRefusedError, socket.timeout, OSError):
            time.sleep(0.05)
    return False
