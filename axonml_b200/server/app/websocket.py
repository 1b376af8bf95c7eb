"""Server side of RFC 6455 WebSockets on a plain socket (the ``http.server`` request handler's
connection after the upgrade), plus a matching minimal client for tests and the CLI.

The reference streams training metrics and a PTY terminal over axum WebSockets
(crates/axonml-server/src/training/websocket.rs, api/terminal.rs).  Text and binary frames, ping /
pong and close are handled; fragmented messages are reassembled; extensions are not negotiated."""
from __future__ import annotations

import base64
import hashlib
import os
import socket
import struct

_GUID = "258EAFA5-E914-47DA-95CA-C5AB0DC85B11"
OP_CONT, OP_TEXT, OP_BIN, OP_CLOSE, OP_PING, OP_PONG = 0x0, 0x1, 0x2, 0x8, 0x9, 0xA


def accept_key(key: str) -> str:
    return base64.b64encode(hashlib.sha1((key + _GUID).encode()).digest()).decode()


class WebSocketClosed(Exception):
    pass


class WebSocket:
    """One end of an established connection.  ``mask_outgoing`` is True for a client."""

    def __init__(self, sock: socket.socket, mask_outgoing: bool = False, pending: bytes = b""):
        self.sock, self.mask_outgoing, self.closed = sock, mask_outgoing, False
        self._pending = pending          # bytes that arrived with the handshake response

    # ------------------------------------------------------------------ sending
    def _send_frame(self, opcode: int, payload: bytes) -> None:
        head = bytes([0x80 | opcode])
        n = len(payload)
        m = 0x80 if self.mask_outgoing else 0
        if n < 126:
            head += bytes([m | n])
        elif n < 1 << 16:
            head += bytes([m | 126]) + struct.pack(">H", n)
        else:
            head += bytes([m | 127]) + struct.pack(">Q", n)
        if self.mask_outgoing:
            key = os.urandom(4)
            payload = bytes(b ^ key[i & 3] for i, b in enumerate(payload))
            head += key
        try:
            self.sock.sendall(head + payload)
        except OSError as e:
            self.closed = True
            raise WebSocketClosed(str(e)) from None

    def send_text(self, text: str) -> None:
        self._send_frame(OP_TEXT, text.encode())

    def send_bytes(self, data: bytes) -> None:
        self._send_frame(OP_BIN, data)

    def send_json(self, obj) -> None:
        import json
        self.send_text(json.dumps(obj))

    def ping(self, data: bytes = b"") -> None:
        self._send_frame(OP_PING, data)

    def close(self, code: int = 1000) -> None:
        if not self.closed:
            try:
                self._send_frame(OP_CLOSE, struct.pack(">H", code))
            except WebSocketClosed:
                pass
            self.closed = True

    # ------------------------------------------------------------------ receiving
    def _read(self, n: int) -> bytes:
        buf, self._pending = self._pending[:n], self._pending[n:]
        while len(buf) < n:
            try:
                chunk = self.sock.recv(n - len(buf))
            except socket.timeout:
                raise
            except OSError as e:
                self.closed = True
                raise WebSocketClosed(str(e)) from None
            if not chunk:
                self.closed = True
                raise WebSocketClosed("peer closed the connection")
            buf += chunk
        return buf

    def recv(self, timeout: float | None = None):
        """Next message: ``str`` for text, ``bytes`` for binary.  Returns None on timeout.  Raises
        ``WebSocketClosed`` when the peer closed."""
        self.sock.settimeout(timeout)
        parts, kind = [], None
        while True:
            try:
                b0, b1 = self._read(2)
            except socket.timeout:
                return None
            fin, opcode, masked, n = b0 & 0x80, b0 & 0x0F, b1 & 0x80, b1 & 0x7F
            self.sock.settimeout(None if timeout is None else max(timeout, 5.0))   # rest of a started frame
            if n == 126:
                n = struct.unpack(">H", self._read(2))[0]
            elif n == 127:
                n = struct.unpack(">Q", self._read(8))[0]
            key = self._read(4) if masked else None
            data = self._read(n) if n else b""
            if key:
                data = bytes(b ^ key[i & 3] for i, b in enumerate(data))
            if opcode == OP_CLOSE:
                self.close()
                raise WebSocketClosed("close frame")
            if opcode == OP_PING:
                self._send_frame(OP_PONG, data)
                continue
            if opcode == OP_PONG:
                continue
            if opcode in (OP_TEXT, OP_BIN):
                kind = opcode
            parts.append(data)
            if fin:
                whole = b"".join(parts)
                return whole.decode("utf-8", "replace") if kind == OP_TEXT else whole


def upgrade(handler) -> WebSocket | None:
    """Completes the opening handshake on a ``BaseHTTPRequestHandler``; None if the request is not
    a WebSocket upgrade (the caller then answers 400)."""
    h = handler.headers
    if h.get("Upgrade", "").lower() != "websocket" or "Sec-WebSocket-Key" not in h:
        return None
    handler.send_response(101, "Switching Protocols")
    handler.send_header("Upgrade", "websocket")
    handler.send_header("Connection", "Upgrade")
    handler.send_header("Sec-WebSocket-Accept", accept_key(h["Sec-WebSocket-Key"]))
    handler.end_headers()
    handler.wfile.flush()
    handler.close_connection = True
    return WebSocket(handler.connection)


def connect(host: str, port: int, path: str, headers: dict | None = None, timeout: float = 10.0) -> WebSocket:
    """Client handshake (tests, ``axonml logs --follow``)."""
    s = socket.create_connection((host, port), timeout=timeout)
    key = base64.b64encode(os.urandom(16)).decode()
    req = [f"GET {path} HTTP/1.1", f"Host: {host}:{port}", "Upgrade: websocket", "Connection: Upgrade",
           f"Sec-WebSocket-Key: {key}", "Sec-WebSocket-Version: 13"]
    req += [f"{k}: {v}" for k, v in (headers or {}).items()]
    s.sendall(("\r\n".join(req) + "\r\n\r\n").encode())
    resp = b""
    while b"\r\n\r\n" not in resp:
        chunk = s.recv(1024)
        if not chunk:
            break
        resp += chunk
    head_b, rest = resp.split(b"\r\n\r\n", 1) if b"\r\n\r\n" in resp else (resp, b"")
    head = head_b.decode("latin1")
    if " 101 " not in head.splitlines()[0]:
        s.close()
        raise ConnectionError(f"upgrade refused: {head.splitlines()[0]}")
    if accept_key(key) not in head:
        s.close()
        raise ConnectionError("bad Sec-WebSocket-Accept")
    return WebSocket(s, mask_outgoing=True, pending=rest)
