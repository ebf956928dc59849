"""One typed configuration for a deployment: daemon, policy and flows, as dataclasses that round-trip through JSON,
with command-line style overrides (``policy.enter_ratio=0.7``) and the reference's environment variables honoured.

The reference has no configuration file: it mixes positional arguments, ``--key=value`` flags and ``SKYGDR_*``
environment variables (src/cpu_client.cc:398-534). Those names keep working (``from_env``); this adds one place to
write a whole set-up down.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, fields, is_dataclass
from typing import Any, Dict, List


@dataclass
class PolicySettings:
    name: str = "target_track"
    enter_ratio: float = 0.65
    exit_ratio: float = 0.80
    util_threshold_pct: float = 85.0
    enter_windows: int = 1
    exit_windows: int = 2
    low1_fraction: float = 0.5
    min_be_fraction: float = 0.02


@dataclass
class FlowSettings:
    name: str = "kv_transfer"
    priority: str = "high"
    target_gbps: float = 40.0
    kind: str = "kv_transfer"
    link: str = ""                 # the shared capacity the flow competes on; "" = the daemon's default link


@dataclass
class ControlPortSettings:
    port: int = 0
    bind_ip: str = "0.0.0.0"
    high_sleep_us: int = 0
    low_sleep_us: int = 100
    low2_sleep_us: int = -1
    low3_sleep_us: int = -1
    low4_sleep_us: int = -1


@dataclass
class RuntimeConfig:
    daemon_host: str = "127.0.0.1"
    daemon_port: int = 7070
    window_us: int = 5000
    capacity_gbps: float = 64.0
    lease_ms: int = 5000
    policy: PolicySettings = field(default_factory=PolicySettings)
    control: ControlPortSettings = field(default_factory=ControlPortSettings)
    flows: List[FlowSettings] = field(default_factory=lambda: [FlowSettings(), FlowSettings("kv_offload", "besteffort", 0.0, "kv_offload")])
    links: Dict[str, float] = field(default_factory=dict)     # more links beside the default one: name -> capacity in GB/s

    # ---- JSON ----
    def to_json(self) -> str:
        return json.dumps(asdict(self), indent=1)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RuntimeConfig":
        known = {f.name for f in fields(cls)}
        bad = set(d) - known
        if bad:
            raise KeyError(f"unknown configuration keys: {sorted(bad)}")
        kw = dict(d)
        if "policy" in kw:
            kw["policy"] = PolicySettings(**kw["policy"])
        if "control" in kw:
            kw["control"] = ControlPortSettings(**kw["control"])
        if "flows" in kw:
            kw["flows"] = [FlowSettings(**f) for f in kw["flows"]]
        return cls(**kw)

    @classmethod
    def from_json(cls, text: str) -> "RuntimeConfig":
        return cls.from_dict(json.loads(text))

    # ---- overrides: "window_us=1000", "policy.enter_ratio=0.7" ----
    def override(self, *assignments: str) -> "RuntimeConfig":
        for a in assignments:
            key, _, val = a.partition("=")
            obj: Any = self
            parts = key.split(".")
            for p in parts[:-1]:
                obj = getattr(obj, p)
            if not hasattr(obj, parts[-1]) or is_dataclass(getattr(obj, parts[-1])):
                raise KeyError(f"unknown configuration key: {key}")
            cur = getattr(obj, parts[-1])
            setattr(obj, parts[-1], type(cur)(val) if not isinstance(cur, bool) else val.lower() in ("1", "true", "yes"))
        return self

    # ---- the reference's environment names ----
    def from_env(self, env=os.environ) -> "RuntimeConfig":
        m = {"SKYGDR_CTRL_PORT": "port", "SKYGDR_CTRL_BIND_IP": "bind_ip", "SKYGDR_CTRL_HIGH_SLEEP_US": "high_sleep_us",
             "SKYGDR_CTRL_LOW_SLEEP_US": "low_sleep_us", "SKYGDR_CTRL_LOW2_SLEEP_US": "low2_sleep_us",
             "SKYGDR_CTRL_LOW3_SLEEP_US": "low3_sleep_us", "SKYGDR_CTRL_LOW4_SLEEP_US": "low4_sleep_us"}
        for name, attr in m.items():
            if env.get(name):
                cur = getattr(self.control, attr)
                setattr(self.control, attr, type(cur)(env[name]))
        if env.get("SKYGDR_DAEMON"):
            host, _, port = env["SKYGDR_DAEMON"].rpartition(":")
            self.daemon_host, self.daemon_port = host or self.daemon_host, int(port)
        return self

    def daemon_args(self) -> List[str]:
        p = self.policy
        return ["--port", str(self.daemon_port), "--policy", p.name, "--window_us", str(self.window_us), "--capacity_gbps",
                str(self.capacity_gbps), "--lease_ms", str(self.lease_ms), "--enter_ratio", str(p.enter_ratio), "--exit_ratio",
                str(p.exit_ratio), "--util_threshold_pct", str(p.util_threshold_pct), "--enter_windows", str(p.enter_windows),
                "--exit_windows", str(p.exit_windows), "--low1_fraction", str(p.low1_fraction)] + \
            [x for name, cap in self.links.items() for x in ("--link", f"{name}={cap}")]
