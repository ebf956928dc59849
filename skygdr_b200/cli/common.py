"""Shared bits of the command-line programs: size parsing, environment capture."""
from __future__ import annotations

import json
import os
import platform
import subprocess
import time
from typing import Dict


def parse_size(text: str) -> int:
    from skygdr_b200.control import ctl

    v = ctl.parse_size(str(text))
    if v is None:
        raise ValueError(f"bad size: {text!r}")
    return v


def env_info() -> Dict:
    """What every benchmark result embeds: GPU, driver, clocks, git revision (the reference writes an
    env_info.txt per run, llm_problem_analysis/final_run_vllm_decode_kv_colocation_bench.sh:185-215)."""
    info = {"time_unix": time.time(), "host": platform.node(), "python": platform.python_version()}
    try:
        import torch

        info["torch"] = torch.__version__
        if torch.cuda.is_available():
            p = torch.cuda.get_device_properties(0)
            info.update(gpu=p.name, sms=p.multi_processor_count, hbm_gb=round(p.total_memory / 1e9, 1), n_gpus=torch.cuda.device_count())
    except Exception as exc:  # pragma: no cover
        info["torch_error"] = repr(exc)
    try:
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        info["git"] = subprocess.run(["git", "-C", root, "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5).stdout.strip()
    except Exception:
        pass
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=driver_version,clocks.sm,clocks.max.sm,power.limit", "--format=csv,noheader"],
                             capture_output=True, text=True, timeout=10).stdout.strip().splitlines()
        if out:
            info["nvidia_smi"] = out[0]
    except Exception:
        pass
    try:       # how the GPUs are wired (NVLink / PCIe matrix), read-only
        topo = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=10).stdout
        rows = [ln.rstrip() for ln in topo.splitlines() if ln.startswith(("GPU", "\tGPU", " "))][:10]
        if rows:
            info["topology"] = rows
    except Exception:
        pass
    return info


def dump_json(path: str, obj) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as f:
        json.dump(obj, f, indent=1)


class ResultFile:
    """A benchmark's result JSON that is written after every arm, so that a run that is cut short keeps what it measured,
    and that a later run can continue (``resume=True``): arms already in the file are skipped, not measured again. The
    reference's tools continue result files in the same spirit (``gpu_metrics_logger.py --append``, the sweep's
    append-with-header logic, src/tools/rdma_msgsize_sweep.py:174-187)."""

    def __init__(self, path: str, head: Dict, section: str = "arms", resume: bool = False):
        self.path, self.section = path, section
        self.data = dict(head)
        self.data.setdefault(section, {})
        self.kept: Dict = {}
        if resume and os.path.exists(path):
            try:
                with open(path) as f:
                    self.kept = dict(json.load(f).get(section, {}))
            except (OSError, ValueError):
                self.kept = {}                  # an unreadable file is not a reason to refuse the run
            self.data[section].update(self.kept)

    def done(self, name: str) -> bool:
        return name in self.kept

    def get(self, name: str):
        return self.data[self.section].get(name)

    def put(self, name: str, value) -> None:
        self.data[self.section][name] = value
        self.save()

    def save(self) -> None:
        os.makedirs(os.path.dirname(os.path.abspath(self.path)), exist_ok=True)
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump(self.data, f, indent=1)
        os.replace(tmp, self.path)              # never leaves a half-written file behind
