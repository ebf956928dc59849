"""Socket clients for flow end-points and for the daemon.

``send_control`` speaks the reference's one-command-per-connection protocol
(src/tools/cpu_client_control.py:17-20, src/tools/pcie_case_study_controller.py:82-99).
``FabricClient`` keeps one connection to ``fabricd`` and registers flows.
"""
from __future__ import annotations

import mmap
import os
import socket
import struct
import time
from dataclasses import dataclass
from typing import Dict, Optional


def send_control(host: str, port: int, command: str, timeout_s: float = 2.0) -> str:
    """Sends one command, half-closes, returns the one-line reply."""
    with socket.create_connection((host, port), timeout=timeout_s) as sock:
        sock.sendall((command.strip() + "\n").encode())
        sock.shutdown(socket.SHUT_WR)
        chunks = []
        while True:
            data = sock.recv(4096)
            if not data:
                break
            chunks.append(data)
            if data.endswith(b"\n"):
                break
    return b"".join(chunks).decode(errors="replace").strip()


def wait_for_control(host: str, port: int, timeout_s: float, command: str = "STATUS") -> str:
    """Retries ``command`` every 0.5 s until the port answers or ``timeout_s`` passes."""
    deadline = time.time() + timeout_s
    last = "timeout"
    while time.time() < deadline:
        try:
            return send_control(host, port, command, timeout_s=1.0)
        except OSError as exc:
            last = str(exc)
            time.sleep(0.5)
    raise RuntimeError(f"control port {host}:{port} not reachable: {last}")


def parse_reply(reply: str) -> Dict[str, str]:
    """``OK a=1 b=x`` -> {'status': 'OK', 'a': '1', 'b': 'x'}; ERR keeps its reason in 'reason'."""
    out: Dict[str, str] = {}
    parts = reply.split()
    if not parts:
        return {"status": "", "reason": "empty"}
    out["status"] = parts[0]
    rest = parts[1:]
    if parts[0] == "ERR" and rest and "=" not in rest[0]:
        out["reason"] = rest[0]
        rest = rest[1:]
    for tok in rest:
        if "=" in tok:
            k, v = tok.split("=", 1)
            out[k] = v
    return out


# Field offsets of SkyCreditPage (skygdr_b200/csrc/ctl/credit_page.h).
_GRANT = struct.Struct("<QQQQQIIIIIId")      # magic granted epoch window_ns budget mode unlimited stop sleep flow prio target
_USAGE_OFF = 128
_USAGE = struct.Struct("<QQQQQQQQ")          # consumed completed stall busy last_ts chunks yields backlog


@dataclass
class FlowHandle:
    flow_id: int
    name: str
    page_path: Optional[str]
    lease_ms: int
    window_us: int
    _mm: Optional[mmap.mmap] = None

    def grant(self) -> Dict[str, float]:
        f = _GRANT.unpack_from(self._mm, 0)
        keys = ("magic", "granted_bytes", "epoch", "window_ns", "budget_per_window", "mode", "unlimited", "stop",
                "pace_sleep_us", "flow_id", "priority", "target_gbps")
        return dict(zip(keys, f))

    def usage(self) -> Dict[str, int]:
        f = _USAGE.unpack_from(self._mm, _USAGE_OFF)
        keys = ("consumed_bytes", "completed_bytes", "stall_ns", "busy_ns", "last_ts_ns", "chunks", "yields",
                "backlog_bytes")
        return dict(zip(keys, f))

    def report(self, consumed: int, completed: int, backlog: int) -> None:
        """Host-side data paths publish their progress here (kernels write the same fields)."""
        struct.pack_into("<QQ", self._mm, _USAGE_OFF, consumed, completed)
        struct.pack_into("<Q", self._mm, _USAGE_OFF + 56, backlog)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None


class FabricClient:
    """A persistent connection to ``fabricd``: register flows, renew leases, query budgets."""

    def __init__(self, host: str = "127.0.0.1", port: int = 7070, timeout_s: float = 2.0, unix: Optional[str] = None):
        """TCP by default; ``unix`` = path of the daemon's Unix-domain socket (``fabricd --unix PATH``) for clients on its host."""
        self.host, self.port = host, port
        if unix:
            self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            self.sock.settimeout(timeout_s)
            self.sock.connect(unix)
        else:
            self.sock = socket.create_connection((host, port), timeout=timeout_s)
            self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        self._buf = b""

    def request(self, line: str) -> str:
        self.sock.sendall((line.strip() + "\n").encode())
        while b"\n" not in self._buf:
            data = self.sock.recv(4096)
            if not data:
                raise ConnectionError("fabricd closed the connection")
            self._buf += data
        reply, self._buf = self._buf.split(b"\n", 1)
        return reply.decode()

    def link(self, name: str, capacity_gbps: Optional[float] = None) -> Dict[str, str]:
        """Defines a link (one shared capacity with its own policy pass, e.g. ``nvlink:gpu0`` at 700 GB/s), changes its
        capacity, or just reports it. Flows name their link when they register; the default link always exists."""
        rep = parse_reply(self.request(f"LINK {name}" + ("" if capacity_gbps is None else f" {capacity_gbps}")))
        if rep.get("status") != "OK":
            raise RuntimeError(f"LINK failed: {rep}")
        return rep

    def register(self, name: str, priority: str | int, target_gbps: float, kind: Optional[str] = None,
                 link: Optional[str] = None) -> FlowHandle:
        rep = parse_reply(self.request(f"REGISTER {name} {priority} {target_gbps} {kind or name}" + (f" link={link}" if link else "")))
        if rep.get("status") != "OK":
            raise RuntimeError(f"REGISTER failed: {rep}")
        path = rep.get("page")
        h = FlowHandle(int(rep["flow_id"]), name, None if path in (None, "-") else path, int(rep["lease_ms"]),
                       int(rep["window_us"]))
        if h.page_path:
            fd = os.open(h.page_path, os.O_RDWR)
            try:
                h._mm = mmap.mmap(fd, 4096)
            finally:
                os.close(fd)
        return h

    def renew(self, flow: FlowHandle | int) -> bool:
        fid = flow.flow_id if isinstance(flow, FlowHandle) else int(flow)
        return self.request(f"RENEW {fid}").startswith("OK")

    def unregister(self, flow: FlowHandle | int) -> bool:
        fid = flow.flow_id if isinstance(flow, FlowHandle) else int(flow)
        ok = self.request(f"UNREGISTER {fid}").startswith("OK")
        if isinstance(flow, FlowHandle):
            flow.close()
        return ok

    def budget(self, flow: FlowHandle | int) -> Dict[str, str]:
        fid = flow.flow_id if isinstance(flow, FlowHandle) else int(flow)
        return parse_reply(self.request(f"BUDGET {fid}"))

    def flow_command(self, flow: FlowHandle | int, command: str) -> str:
        fid = flow.flow_id if isinstance(flow, FlowHandle) else int(flow)
        return self.request(f"FLOW {fid} {command}")

    def close(self) -> None:
        try:
            self.sock.sendall(b"QUIT\n")
        except OSError:
            pass
        self.sock.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
