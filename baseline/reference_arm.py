"""`bench.py --impl reference`: what can be run of the unmodified reference for the headline metric.

The reference is not a Python package (no setup.py / pyproject.toml: `pip install <reference checkout>` ends
with "neither 'setup.py' nor 'pyproject.toml' found"), has no decoder model, no GEMM and no tensor
parallelism, and its scheduled data path needs libibverbs and an RNIC. So the headline configuration
(Qwen3-8B tensor-parallel decode) cannot be produced by it. What does exist is its decode KV-scan
stressor; when `baseline/_ref/` holds that program (built by baseline/build_ref.sh from the untouched
source) it is run here with the Qwen3-8B KV geometry and reported under `nearest`, beside the
`unavailable` line, never in place of the metric.
"""
from __future__ import annotations

import os
import re
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
REF_BIN = os.path.join(HERE, "_ref", "bin")


def run(args, rank: int) -> dict:
    out = {
        "impl": "reference",
        "unavailable": "the reference has no Qwen3 decoder, GEMM or tensor-parallel path and is not a Python package "
                       "(pip install: neither setup.py nor pyproject.toml); its RDMA path needs libibverbs + an RNIC",
    }
    exe = os.path.join(REF_BIN, "decode_vllm_kvcache_hbm_stress")
    if rank != 0 or not os.path.exists(exe):
        return out
    try:
        import torch

        if not torch.cuda.is_available():
            return out
        # the reference's own decode workload: fp32 KV scan, no block table, no weights; one GPU
        ctx = (args.ctx_lo + args.ctx_hi) // 2
        cmd = [exe, "--gpu", "0", "--layers", "36", "--kv-heads", "8", "--head-dim", "128", "--context", str(ctx),
               "--gen", str(args.steps), "--batch", str(args.batch_per_gpu), "--tile-tokens", "128", "--threads", "256",
               "--report-every", str(max(1, args.steps))]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
        text = r.stdout + r.stderr
        m = re.search(r"sequence-throughput:\s*([0-9.]+)", text)
        out["nearest"] = {
            "program": "llm_problem_analysis/decode_vllm_kvcache_hbm_stress.cu (built unmodified, sm_100)",
            "what": "batched KV scan only: fp32 KV, fixed context, no block table, no weights, no sampling",
            "cmd": " ".join(cmd[1:]), "rc": r.returncode,
            "seq_tokens_per_s": float(m.group(1)) if m else None,
            "tail": text.strip().splitlines()[-8:],
        }
    except Exception as exc:  # the unavailable line stands on its own
        out["nearest_error"] = repr(exc)
    return out
