"""Per-rank side of the fault-tolerance control plane: registers with the controller, sends heartbeats, reports its
own faults, and reacts to PAUSE / DUMP_REQUEST / EXIT
(reference: mindspeed/core/ttp/comm/processor.py:138-851, heartbeat.py:14-259).

PAUSE interrupts the training thread by raising ``TTPPause`` in it asynchronously (the reference raises
``RuntimeError("STEP FINISH")`` the same way, processor.py:378-404); on a GPU the host side then stops issuing work
and in-flight NCCL operations are abandoned by aborting the communicator from the watchdog."""
from __future__ import annotations

import ctypes
import socket
import threading
import time
from typing import Callable, List, Optional

from . import protocol as P


class TTPPause(RuntimeError):
    """Raised in the training thread when the controller pauses this rank."""


class TTPProcessor:
    def __init__(self, rank: int, host: str, port: int, replica_groups: Optional[List[List[int]]] = None,
                 heartbeat_interval_ms: int = P.DEFAULT_HEARTBEAT_INTERVAL_MS, dump_fn: Optional[Callable[[List[int]], None]] = None,
                 interrupt_main: bool = False):
        self.rank, self.host, self.port = rank, host, port
        self.replica_groups = replica_groups or []
        self.interval = heartbeat_interval_ms / 1000.0
        self.dump_fn = dump_fn
        self.interrupt_main = interrupt_main
        self.main_thread_id = threading.get_ident()
        self.sock: Optional[socket.socket] = None
        self.paused = threading.Event()
        self.exited = threading.Event()
        self.dumped = threading.Event()
        self.beat_enabled = threading.Event()
        self.beat_enabled.set()
        self.stop_evt = threading.Event()
        self.events: List[str] = []
        self.send_lock = threading.Lock()

    def start(self, connect_timeout_s: float = 10.0):
        deadline = time.time() + connect_timeout_s
        while True:
            try:
                self.sock = socket.create_connection((self.host, self.port), timeout=2.0)
                break
            except OSError:
                if time.time() > deadline:
                    raise
                time.sleep(0.05)
        self.sock.settimeout(None)
        self._send(P.REGISTER, rank=self.rank, replica_groups=self.replica_groups)
        ack = P.recv_msg(self.sock)
        assert ack["type"] == P.ACK
        for fn in (self._heartbeat_loop, self._listen_loop):
            threading.Thread(target=fn, daemon=True).start()
        return self

    def _send(self, kind, **payload):
        with self.send_lock:
            P.send_msg(self.sock, kind, **payload)

    def _heartbeat_loop(self):
        while not self.stop_evt.is_set():
            if self.beat_enabled.is_set():
                try:
                    self._send(P.HEARTBEAT, rank=self.rank, t=time.time())
                except OSError:
                    return
            time.sleep(self.interval)

    def _listen_loop(self):
        try:
            while not self.stop_evt.is_set():
                msg = P.recv_msg(self.sock)
                kind = msg["type"]
                self.events.append(kind)
                if kind == P.PAUSE:
                    self.paused.set()
                    if self.interrupt_main:
                        ctypes.pythonapi.PyThreadState_SetAsyncExc(ctypes.c_ulong(self.main_thread_id), ctypes.py_object(TTPPause))
                elif kind == P.DUMP_REQUEST:
                    try:
                        if self.dump_fn is not None:
                            self.dump_fn(msg["ranks"])
                    finally:
                        self.dumped.set()
                        self._send(P.DUMP_DONE, rank=self.rank)
                elif kind == P.EXIT:
                    self.exited.set()
                    return
        except (ConnectionError, OSError, ValueError):
            self.exited.set()

    # ---- API used by the training loop ----
    def report_fault(self, reason: str):
        try:
            self._send(P.REPORT_FAULT, rank=self.rank, reason=reason[:400])
        except OSError:
            pass

    def stop_heartbeat(self):
        """Test hook: a frozen process stops sending heartbeats but keeps its socket open."""
        self.beat_enabled.clear()

    def close(self):
        self.stop_evt.set()
        try:
            self.sock.shutdown(socket.SHUT_RDWR)
        except OSError:
            pass
        try:
            self.sock.close()
        except OSError:
            pass
