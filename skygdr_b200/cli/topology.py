"""The links of this machine's GPUs, as `fabricd --link` arguments.

    python -m skygdr_b200.cli.topology [--gpus 0,1,...] [--nvlink_efficiency 0.855] [--signals] [--json]
    skygdr_b200/bin/fabricd --port 7070 $(python -m skygdr_b200.cli.topology)

Per GPU, three shared capacities that flows can register on (`REGISTER ... link=<name>`):
  nvlink:gpuN   NVLink per direction (product table; scaled by --nvlink_efficiency, default the share a peer copy reaches)
  pcie:gpuN     the PCIe link in one direction: lanes x usable rate of the current generation
  hbm:gpuN      device memory bandwidth (product table)
Read from NVML through the same bindings as the signal loggers. The reference has one implicit link, the PCIe link of the
GPU under test (src/tools/gpu_metrics_logger.py:38-67 computes its peak the same way).
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, Optional


def links_of_gpu(index: int, fake: Optional[dict] = None, nvlink_efficiency: float = 0.855) -> Dict[str, float]:
    """name -> GB/s for one GPU; empty when NVML does not answer. ``fake`` is the stand-in NVML of ctl.GpuSignals."""
    from skygdr_b200.control import ctl

    sig = ctl.GpuSignals(index, fake, 0.0)
    if not sig.available:
        return {}
    out: Dict[str, float] = {}
    nv = ctl.nvlink_peak_gbs(sig.name)
    if nv > 0:
        out[f"nvlink:gpu{index}"] = round(nv * nvlink_efficiency, 1)
    pcie = sig.pcie_peak_gib_s * 1.073741824
    if pcie > 0:
        out[f"pcie:gpu{index}"] = round(pcie, 1)
    hbm = ctl.hbm_peak_gbs(sig.name)
    if hbm > 0:
        out[f"hbm:gpu{index}"] = float(hbm)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", default="", help="comma list; default: every GPU that NVML shows")
    ap.add_argument("--nvlink_efficiency", type=float, default=0.855, help="share of nominal NVLink that a peer copy reaches (770 of 900 GB/s measured)")
    ap.add_argument("--signals", action="store_true", help="also bind every NVLink / PCIe link to its GPU's inbound NVML counter (--link_signal)")
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    ids = [int(x) for x in a.gpus.split(",") if x] if a.gpus else range(64)
    links: Dict[str, float] = {}
    for i in ids:
        got = links_of_gpu(i, None, a.nvlink_efficiency)
        if not got:
            if a.gpus:
                print(f"gpu {i}: NVML does not answer", file=sys.stderr)
                return 1
            break
        links.update(got)
    if not links:
        print("NVML is not available on this machine", file=sys.stderr)
        return 1
    args = [f"--link {k}={v}" for k, v in links.items()]
    if a.signals:
        for k in links:
            kind, _, gpu = k.partition(":gpu")
            if kind in ("nvlink", "pcie"):
                args.append(f"--link_signal {k}={gpu}:{kind}_rx")
    print(json.dumps(links, indent=1) if a.json else " ".join(args))
    return 0


if __name__ == "__main__":
    sys.exit(main())
