"""Control-plane wire protocol: framed messages over a stream socket.

Frame = ``u64 BE length | u32 BE kind | body`` (comms/src/codec/sink.rs:37-57, source.rs:34-56);
kind 0 carries a JSON command in serde's externally tagged snake_case form, kinds 5 and 6 carry raw
little-endian f32 payloads (parameters, dataset chunks) as in comms/src/protocol/msg.rs:120-191.
Gradients never travel here: on this runtime they move through NVLink windows (kinds 1-4 are accepted
for completeness and decoded by the C++ codecs).

Handshake (comms/src/connection/{connector.rs:175-196, acceptor.rs:52-74}): the initiator sends
``connect{id,src}``, the acceptor answers ``accept{id,src}``; ``src`` names the sender's entity.
"""
from __future__ import annotations

import json
import socket
import struct
import uuid

import numpy as np

KIND_CONTROL, KIND_PARAMS, KIND_DATACHUNK = 0, 5, 6
ENTITIES = ("Node", "Orchestrator", "ParamServer", "Worker")


class Channel:
    """One framed, bidirectional connection."""

    def __init__(self, sock: socket.socket):
        self.sock = sock
        self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self.peer_entity: str | None = None
        self.peer_id: str | None = None

    # ---- framing ----
    def _send_frame(self, kind: int, body: bytes | memoryview) -> None:
        head = struct.pack(">QI", len(body) + 4, kind)
        self.sock.sendall(head)
        if len(body):
            self.sock.sendall(body)

    def _recv_exact(self, n: int) -> bytearray:
        buf = bytearray(n)
        view = memoryview(buf)
        got = 0
        while got < n:
            k = self.sock.recv_into(view[got:], n - got)
            if k == 0:
                raise ConnectionError("peer closed the connection")
            got += k
        return buf

    def send_command(self, cmd) -> None:
        """``cmd`` is a bare string (unit variant) or a single-key dict (struct variant)."""
        self._send_frame(KIND_CONTROL, json.dumps(cmd).encode())

    def send_floats(self, kind: int, arr: np.ndarray) -> None:
        a = np.ascontiguousarray(arr, dtype="<f4")
        self._send_frame(kind, memoryview(a).cast("B"))

    def recv(self, timeout: float | None = None):
        """Returns ("control", command) or ("params"|"datachunk", float32 array)."""
        self.sock.settimeout(timeout)
        head = self._recv_exact(12)
        length, kind = struct.unpack(">QI", head)
        body = self._recv_exact(length - 4)
        if kind == KIND_CONTROL:
            return "control", json.loads(bytes(body).decode().replace("NaN", "null"))
        if kind == KIND_PARAMS:
            return "params", np.frombuffer(body, dtype="<f4")
        if kind == KIND_DATACHUNK:
            return "datachunk", np.frombuffer(body, dtype="<f4")
        if kind in (1, 2, 3, 4):
            return ("dense_grad" if kind < 3 else "sparse_grad"), (bytes(body), kind % 2 == 0)
        raise ValueError(f"Received an invalid kind byte {kind}")

    # ---- handshake ----
    def connect_as(self, entity: str, my_id: str | None = None) -> str:
        my_id = my_id or str(uuid.uuid4())
        self.send_command({"connect": {"id": my_id, "src": entity}})
        kind, msg = self.recv(timeout=30)
        if kind != "control" or "accept" not in msg:
            raise ConnectionError(f"expected accept, got {msg!r}")
        self.peer_id, self.peer_entity = msg["accept"]["id"], msg["accept"]["src"]
        return my_id

    def accept_as(self, entity: str, my_id: str) -> None:
        kind, msg = self.recv(timeout=30)
        if kind != "control" or "connect" not in msg:
            raise ConnectionError(f"expected connect, got {msg!r}")
        self.peer_id, self.peer_entity = msg["connect"]["id"], msg["connect"]["src"]
        self.send_command({"accept": {"id": my_id, "src": entity}})

    # ---- dataset streaming (comms/src/share_dataset/{send,recv}_dataset.rs) ----
    def send_dataset(self, xs: np.ndarray, ys: np.ndarray, chunk_bytes: int = 1 << 20) -> None:
        for arr in (xs, ys):
            flat = np.ascontiguousarray(arr, dtype="<f4").reshape(-1)
            self.send_command({"share_dataset_size": {"size": int(flat.size)}})
            step = max(1, chunk_bytes // 4)
            for lo in range(0, flat.size, step):
                self.send_floats(KIND_DATACHUNK, flat[lo:lo + step])
            self.send_command("eof")

    def recv_dataset(self) -> tuple[np.ndarray, np.ndarray]:
        out = []
        for _ in range(2):
            kind, msg = self.recv(timeout=300)
            if kind != "control" or "share_dataset_size" not in msg:
                raise ConnectionError(f"expected share_dataset_size, got {msg!r}")
            buf = np.empty(msg["share_dataset_size"]["size"], dtype=np.float32)
            at = 0
            while True:
                kind, payload = self.recv(timeout=300)
                if kind == "control" and payload == "eof":
                    break
                if kind != "datachunk":
                    raise ConnectionError("unexpected message while receiving a dataset")
                buf[at:at + payload.size] = payload
                at += payload.size
            if at != buf.size:
                raise ConnectionError("dataset stream shorter than announced")
            out.append(buf)
        return out[0], out[1]

    def close(self) -> None:
        try:
            self.sock.close()
        except OSError:
            pass


def connect(host: str, port: int, timeout: float = 30.0) -> Channel:
    return Channel(socket.create_connection((host, port), timeout=timeout))


def listen(host: str, port: int) -> socket.socket:
    s = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
    s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
    s.bind((host, port))
    s.listen(64)
    return s


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]
