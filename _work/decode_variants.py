"""The decode benchmark under each opt-in engine option, one process per variant, as one table.

    python benchmarks/decode_variants.py [--gpus 1] [--steps 16] [--warmup 3] [--variants default,fuse_norm,...]
                                         [--out results/decode_variants.json] [--resume]

Every variant is `bench.py` with some flags, started as its own process (through torch.distributed.run for more than
one GPU), so a variant that fails or reports a kernel status other than OK does not take the others with it; its row
says what happened. Rows are written to --out as they finish and `--resume` skips the ones already there. The table
gives tokens/s, the ratio to the default engine, the end-to-end figure and the kernels' status word.

Variants (see `bench.py --help`): default; fuse_norm (RMSNorms folded into the GEMM epilogues, one GPU only); tail and
fine (decode attention grid orders that schedule partial chunks last); oneshot (tensor-parallel one-shot all-reduce,
two or more GPUs); chunk512 / chunk2048 (split-KV chunk size); and combinations joined with '+', e.g. fuse_norm+fine.
"""
import argparse
import json
import os
import socket
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from skygdr_b200.cli.common import ResultFile, env_info  # noqa: E402

FLAGS = {
    "default": [],
    "fuse_norm": ["--fuse-norm"],
    "tail": ["--attn-order", "tail"],
    "fine": ["--attn-order", "fine"],
    "oneshot": ["--tp-collective", "oneshot"],
    "chunk512": ["--attn-chunk", "512"],
    "chunk2048": ["--attn-chunk", "2048"],
}


def flags_of(variant: str):
    out = []
    for part in variant.split("+"):
        if part not in FLAGS:
            raise SystemExit(f"unknown variant {part!r}; known: {', '.join(FLAGS)}")
        out += FLAGS[part]
    return out


def applicable(variant: str, gpus: int) -> str:
    parts = variant.split("+")
    if "fuse_norm" in parts and gpus > 1:
        return "one GPU only"
    if "oneshot" in parts and gpus < 2:
        return "needs two or more GPUs"
    return ""


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_variant(variant: str, a) -> dict:
    bench = a.bench_cmd.split() if a.bench_cmd else [sys.executable, os.path.join(ROOT, "bench.py")]
    if a.gpus > 1 and not a.bench_cmd:
        bench = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}", "--master-addr", "127.0.0.1",
                 "--master-port", str(free_port()), os.path.join(ROOT, "bench.py")]
    cmd = bench + ["--gpus", str(a.gpus), "--steps", str(a.steps), "--warmup", str(a.warmup)] + flags_of(variant)
    t0 = time.time()
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=a.timeout_s, cwd=ROOT)
    except subprocess.TimeoutExpired:
        return {"error": f"no result within {a.timeout_s:.0f} s", "wall_s": time.time() - t0}
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    if r.returncode != 0 or not lines:
        return {"error": f"exit code {r.returncode}", "stderr_tail": r.stderr[-600:], "wall_s": time.time() - t0}
    d = json.loads(lines[-1])
    return {"tok_s": d["value"], "ms_per_step": d["ms_per_step"], "e2e_tok_s": d.get("e2e", {}).get("value"),
            "kernel_status": d.get("kernel_status"), "gpu_launches": d.get("gpu_launches"), "clocks": d.get("clocks"),
            "hbm_frac_of_measured": d.get("roofline", {}).get("hbm_frac_of_measured"), "wall_s": time.time() - t0}


def table(rows: dict) -> str:
    base = rows.get("default", {}).get("tok_s")
    out = [f"{'variant':<22}{'tokens/s':>12}{'vs default':>12}{'e2e tok/s':>12}{'ms/step':>10}  status"]
    for name, r in rows.items():
        if "tok_s" in r:
            rel = f"{r['tok_s'] / base:.3f}" if base else "-"
            e2e = f"{r['e2e_tok_s']:.1f}" if r.get("e2e_tok_s") else "-"
            out.append(f"{name:<22}{r['tok_s']:>12.1f}{rel:>12}{e2e:>12}{r['ms_per_step']:>10.3f}  {r.get('kernel_status')}")
        else:
            out.append(f"{name:<22}{'-':>12}{'-':>12}{'-':>12}{'-':>10}  {r.get('skipped') or r.get('error')}")
    return "\n".join(out)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--variants", default="default,fuse_norm,tail,fine,fuse_norm+fine,oneshot")
    ap.add_argument("--timeout-s", type=float, default=600.0)
    ap.add_argument("--out", default="results/decode_variants.json")
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--bench-cmd", default="", help="command to run instead of bench.py (for testing this driver)")
    a = ap.parse_args(argv)
    rf = ResultFile(a.out, {"config": {"gpus": a.gpus, "steps": a.steps, "warmup": a.warmup}, "env": env_info()}, section="variants", resume=a.resume)
    for v in [x for x in a.variants.split(",") if x]:
        flags_of(v)                                   # unknown names stop the run before anything is measured
    for v in [x for x in a.variants.split(",") if x]:
        if rf.done(v) and "tok_s" in (rf.get(v) or {}):
            continue
        why = applicable(v, a.gpus)
        rf.put(v, {"skipped": why} if why else run_variant(v, a))
    print(table(rf.data["variants"]))
    return 0


if __name__ == "__main__":
    sys.exit(main())
