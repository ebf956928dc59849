"""Control plane: protocol, flow registry, policies, fabric simulator, daemon.

The heavy lifting is native (``skygdr_b200/csrc/ctl``); this package loads the
bindings, building them on first use, and adds the socket client and the
daemon launcher.
"""
from __future__ import annotations

import importlib


def _load_ctl():
    try:
        return importlib.import_module("skygdr_b200._ctl")
    except ImportError:
        from skygdr_b200 import build

        build.build_ctl()
        importlib.invalidate_caches()
        return importlib.import_module("skygdr_b200._ctl")


ctl = _load_ctl()

from .client import FabricClient, send_control, wait_for_control  # noqa: E402
from .daemon import FabricDaemon  # noqa: E402
from .config1 import Config1, run_config1  # noqa: E402

__all__ = ["ctl", "FabricClient", "send_control", "wait_for_control", "FabricDaemon", "Config1", "run_config1"]
