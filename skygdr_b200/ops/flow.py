"""Device-visible flow state: a credit page in mapped host memory plus the
launch status block, shared by the transfer, offload and memhog kernels."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .._ext import load

STATUS_NAMES = {0: "OK", 1: "YIELD_CREDIT", 2: "STOPPED", 3: "TIMEOUT_FLAG", 4: "BAD_INDEX", 5: "TIMEOUT_MBAR", 6: "CONTROL_LOST"}
DEAD_POLICIES = {"stall": 0, "unpaced": 1, "static": 2}


class CreditPage:
    """One flow's credit page in pinned, mapped host memory.

    ``host_ptr`` is what the control side writes; ``dev_ptr`` is what kernels
    read. ``attach`` wraps a page that the daemon created under /dev/shm."""

    def __init__(self, flow_id: int = 0, unlimited: bool = True):
        self._C = load()
        self.host_ptr, self.dev_ptr = self._C.host_alloc_mapped(4096)
        self._owned = True
        self._mm = None
        self._C.credit_page_init(self.host_ptr, flow_id, unlimited)
        self.granted = 0

    @classmethod
    def attach(cls, path: str) -> "CreditPage":
        import ctypes
        import mmap
        import os

        self = cls.__new__(cls)
        self._C = load()
        fd = os.open(path, os.O_RDWR)
        try:
            self._mm = mmap.mmap(fd, 4096)
        finally:
            os.close(fd)
        self.host_ptr = ctypes.addressof(ctypes.c_char.from_buffer(self._mm))
        self.dev_ptr = self._C.host_register(self.host_ptr, 4096)
        self._owned = False
        self.granted = 0
        return self

    def grant(self, granted_bytes: int, unlimited: bool = False, stop: bool = False) -> None:
        self.granted = granted_bytes
        self._C.credit_page_grant(self.host_ptr, granted_bytes, unlimited, stop)

    def set_heartbeat(self, window_ms: float, dead_after_windows: int, policy: str = "stall", fallback_gbps: float = 1.0) -> None:
        """The heartbeat contract of this page: a data path that waits for credit and sees ``epoch`` (bumped by every
        ``grant``) stand still for ``dead_after_windows`` windows takes the control side for dead and follows ``policy``:
        "stall" (give up with CONTROL_LOST once the last grant is used), "unpaced", or "static" (``fallback_gbps``)."""
        window_ns = int(window_ms * 1e6)
        self._C.credit_page_heartbeat(self.host_ptr, window_ns, dead_after_windows, DEAD_POLICIES[policy],
                                      int(fallback_gbps * 1e9 * window_ms * 1e-3))

    def set_unlimited(self) -> None:
        self._C.credit_page_grant(self.host_ptr, self.granted, True, False)

    def read(self) -> Dict[str, int]:
        return dict(self._C.credit_page_read(self.host_ptr))

    def close(self) -> None:
        if self.host_ptr:
            if self._owned:
                self._C.host_free_mapped(self.host_ptr)
            else:
                self._C.host_unregister(self.host_ptr)
                self._mm = None
            self.host_ptr = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class LocalPacer:
    """In-process control side for one page: adds ``rate_gbps`` worth of bytes to the grant every ``window_ms`` (what fabricd
    does for registered flows, without the daemon). The loop is a native thread (csrc/ctl/daemon_core.hpp, PagePacer), so a
    paced flow does not depend on the interpreter lock of the process that also launches the kernels."""

    def __init__(self, page: CreditPage, rate_gbps: float, window_ms: float = 1.0, burst_windows: float = 2.0):
        from ..control import ctl

        self.page = page
        self._native = ctl.PagePacer(page.host_ptr, rate_gbps, int(window_ms * 1e6), burst_windows)

    def start(self, base: int = 0):
        self.page.granted = base
        self._native.start(base)
        return self

    def stop(self):
        self._native.stop()
        self.page.granted = self.page.read()["granted_bytes"]


def new_status(device) -> torch.Tensor:
    return load().new_status(torch.device(device).index or 0)


def read_status(status: torch.Tensor) -> Dict[str, int]:
    d = dict(load().read_status(status))
    d["status_name"] = STATUS_NAMES.get(d["status"], str(d["status"]))
    return d
