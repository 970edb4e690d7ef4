"""Wire format and message types of the fault-tolerance control plane (length-prefixed JSON over TCP).
Message set follows the reference (mindspeed/core/ttp/constants.py:16-31)."""
import json
import socket
import struct

REGISTER, HEARTBEAT, REPORT_FAULT, PAUSE, DUMP_REQUEST, DUMP_DONE, EXIT, ACK, STATUS = (
    "REGISTER", "HEARTBEAT", "REPORT_FAULT", "PAUSE", "DUMP_REQUEST", "DUMP_DONE", "EXIT", "ACK", "STATUS")

DEFAULT_HEARTBEAT_INTERVAL_MS = 1000
DEFAULT_HEARTBEAT_TIMEOUT_MS = 3000
DEFAULT_MAX_MISSED = 3


def send_msg(sock: socket.socket, kind: str, **payload):
    data = json.dumps({"type": kind, **payload}).encode()
    sock.sendall(struct.pack("!I", len(data)) + data)


def _recv_exact(sock, n):
    buf = b""
    while len(buf) < n:
        chunk = sock.recv(n - len(buf))
        if not chunk:
            raise ConnectionError("peer closed the connection")
        buf += chunk
    return buf


def recv_msg(sock: socket.socket) -> dict:
    (n,) = struct.unpack("!I", _recv_exact(sock, 4))
    return json.loads(_recv_exact(sock, n).decode())
