"""Launcher for the ``fabricd`` executable."""
from __future__ import annotations

import signal
import socket
import subprocess
from pathlib import Path
from typing import Optional

from .client import wait_for_control


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class FabricDaemon:
    """Starts ``fabricd`` as a child process and stops it with SIGTERM (which writes the snapshot)."""

    def __init__(self, port: Optional[int] = None, policy: str = "target_track", window_us: int = 5000,
                 capacity_gbps: float = 64.0, lease_ms: int = 5000, log: Optional[str] = None,
                 snapshot: Optional[str] = None, restore: Optional[str] = None, extra: Optional[list] = None):
        from skygdr_b200 import build

        exe = Path(build.build_bin()) / "fabricd"
        self.port = port or free_port()
        cmd = [str(exe), "--port", str(self.port), "--policy", policy, "--window_us", str(window_us),
               "--capacity_gbps", str(capacity_gbps), "--lease_ms", str(lease_ms)]
        if log:
            cmd += ["--log", log]
        if snapshot:
            cmd += ["--snapshot", snapshot]
        if restore:
            cmd += ["--restore", restore]
        cmd += list(extra or [])
        self.proc = subprocess.Popen(cmd, stderr=subprocess.PIPE, text=True)
        wait_for_control("127.0.0.1", self.port, 10.0, command="PING")

    def stop(self, timeout_s: float = 5.0) -> int:
        if self.proc.poll() is None:
            self.proc.send_signal(signal.SIGTERM)
            try:
                self.proc.wait(timeout=timeout_s)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                self.proc.wait(timeout=2)
        return self.proc.returncode

    def kill(self) -> None:
        """Ends the daemon without a snapshot: what a crash looks like to its flows."""
        if self.proc.poll() is None:
            self.proc.kill()
            self.proc.wait(timeout=2)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.stop()
