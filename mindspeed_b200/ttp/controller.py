"""Fault-tolerance controller: a TCP server (normally on rank 0) that tracks heartbeats, learns of faults by time-out,
disconnect or self-report, pauses the healthy ranks, chooses one healthy member per replica group, asks them for an
emergency dump checkpoint and finally tells everyone to exit
(reference: mindspeed/core/ttp/comm/controller.py:35-978)."""
from __future__ import annotations

import socket
import threading
import time
from typing import Dict, List, Optional, Set

from . import protocol as P
from .replica import select_dump_ranks


class TTPController:
    def __init__(self, world_size: int, host: str = "127.0.0.1", port: int = 0, heartbeat_timeout_ms: int = P.DEFAULT_HEARTBEAT_TIMEOUT_MS,
                 max_missed: int = P.DEFAULT_MAX_MISSED, dump_timeout_s: float = 60.0):
        self.world_size = world_size
        self.timeout_s = heartbeat_timeout_ms / 1000.0
        self.max_missed = max_missed
        self.dump_timeout_s = dump_timeout_s
        self.sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self.sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self.sock.bind((host, port))
        self.sock.listen(world_size + 8)
        self.port = self.sock.getsockname()[1]
        self.clients: Dict[int, socket.socket] = {}
        self.last_beat: Dict[int, float] = {}
        self.replica_groups: List[List[int]] = []
        self.faulty: Set[int] = set()
        self.fault_reasons: Dict[int, str] = {}
        self.dump_done: Set[int] = set()
        self.state = "RUNNING"
        self.plan: Optional[dict] = None
        self.lock = threading.RLock()
        self.stop_evt = threading.Event()
        self.finished = threading.Event()
        self.threads: List[threading.Thread] = []

    # ---- lifecycle ----
    def start(self):
        for fn in (self._accept_loop, self._monitor_loop):
            t = threading.Thread(target=fn, daemon=True)
            t.start()
            self.threads.append(t)
        return self

    def stop(self):
        self.stop_evt.set()
        try:
            self.sock.close()
        except OSError:
            pass
        for s in list(self.clients.values()):
            try:
                s.close()
            except OSError:
                pass

    # ---- loops ----
    def _accept_loop(self):
        self.sock.settimeout(0.2)
        while not self.stop_evt.is_set():
            try:
                conn, _ = self.sock.accept()
            except (socket.timeout, OSError):
                continue
            t = threading.Thread(target=self._client_loop, args=(conn,), daemon=True)
            t.start()
            self.threads.append(t)

    def _client_loop(self, conn: socket.socket):
        rank = None
        try:
            while not self.stop_evt.is_set():
                msg = P.recv_msg(conn)
                kind = msg["type"]
                if kind == P.REGISTER:
                    rank = int(msg["rank"])
                    with self.lock:
                        self.clients[rank] = conn
                        self.last_beat[rank] = time.time()
                        for g in msg.get("replica_groups", []):
                            if g not in self.replica_groups:
                                self.replica_groups.append(g)
                    P.send_msg(conn, P.ACK)
                elif kind == P.HEARTBEAT:
                    with self.lock:
                        self.last_beat[int(msg["rank"])] = time.time()
                elif kind == P.REPORT_FAULT:
                    self._on_fault(int(msg["rank"]), msg.get("reason", "reported"))
                elif kind == P.DUMP_DONE:
                    with self.lock:
                        self.dump_done.add(int(msg["rank"]))
                    self._maybe_finish()
        except (ConnectionError, OSError, ValueError):
            if rank is not None and not self.stop_evt.is_set() and self.state == "RUNNING":
                self._on_fault(rank, "disconnect")

    def _monitor_loop(self):
        while not self.stop_evt.is_set():
            time.sleep(min(0.05, self.timeout_s / 4))
            now = time.time()
            with self.lock:
                if self.state != "RUNNING":
                    if self.state == "DUMPING" and now - self._dump_started > self.dump_timeout_s:
                        self._finish(timeout=True)
                    continue
                late = [r for r, t in self.last_beat.items() if r not in self.faulty and now - t > self.timeout_s]
            for r in late:
                self._on_fault(r, "heartbeat timeout")

    # ---- fault handling ----
    def _on_fault(self, rank: int, reason: str):
        with self.lock:
            if rank in self.faulty:
                return
            self.faulty.add(rank)
            self.fault_reasons[rank] = reason
            if self.state != "RUNNING":
                return
            self.state = "PAUSING"
            healthy = [r for r in self.clients if r not in self.faulty]
            for r in healthy:
                self._send(r, P.PAUSE, faulty=sorted(self.faulty), reason=reason)
            groups = self.replica_groups or [[r] for r in range(self.world_size)]
            self.plan = select_dump_ranks(groups, self.faulty)
            self.state = "DUMPING"
            self._dump_started = time.time()
            if self.plan["ok"]:
                for r in self.plan["ranks"]:
                    self._send(r, P.DUMP_REQUEST, ranks=self.plan["ranks"])
            else:
                self._finish(timeout=False)

    def _send(self, rank, kind, **payload):
        s = self.clients.get(rank)
        if s is None:
            return
        try:
            P.send_msg(s, kind, **payload)
        except OSError:
            self.faulty.add(rank)

    def _maybe_finish(self):
        with self.lock:
            if self.state == "DUMPING" and self.plan and set(self.plan["ranks"]) <= self.dump_done:
                self._finish(timeout=False)

    def _finish(self, timeout: bool):
        with self.lock:
            if self.state == "EXITING":
                return
            self.state = "EXITING"
            self.dump_timed_out = timeout
            for r in list(self.clients):
                if r not in self.faulty:
                    self._send(r, P.EXIT, dump_ok=bool(self.plan and self.plan["ok"] and not timeout))
            self.finished.set()
