"""Colocation harness: a workload alone, its competitor alone, both overlapped, then a scraped summary.

    python -m skygdr_b200.cli.colocation_bench hbm_kv        # HBM stressor ‖ fixed-size NVLink transfer
    python -m skygdr_b200.cli.colocation_bench trace_decode  # decoder-style stressor (GEMMs + attention) ‖ trace-shaped transfers
    python -m skygdr_b200.cli.colocation_bench vllm_decode   # batched paged decode attention ‖ trace-shaped transfers, repeats, dmon
    python -m skygdr_b200.cli.colocation_bench multi_kv      # HBM stressor ‖ four transfers at once
    options: --preset NAME  --impl ours|reference  --out-dir DIR  --dry-run

One program for the reference's shell harnesses (llm_problem_analysis/run_hbm_kv_overlap_bench.sh:120-191,
run_trace_decode_colocation_bench.sh:208-353, final_run_vllm_decode_kv_colocation_bench.sh:221-419, run_all.sh:3-12).
Parameters come from the same environment variables (SRC_GPU, DST_GPU, HBM_WORKING_SET_MIB, HBM_ITERS,
KV_TRANSFER_MIB, KV_ITERS, LAYERS, KV_HEADS, HEAD_DIM, ELEM_BYTES, DECODE_CONTEXT, DECODE_GEN, DECODE_BATCH,
TILE_TOKENS, FFN_DIM, KV_DISTS, KV_ITERS_COMPUTED/CACHED/INPUT, START_DELAY_SEC, REPEATS, ENABLE_DMON, OUT_DIR);
`--preset` fills in the values of the reference's wrapper scripts (run_all_stress.sh, run_real_trace.sh,
run_real_trace.sh.small, final_run_vllm_real_trace_for_hbm_contention_between_nvlink_and_decoder.sh) plus
B200-sized ones. Every phase is its own process, the overlapped competitor starts START_DELAY_SEC after the
workload, `nvidia-smi dmon -s pucvmt` (read-only) logs each phase, and the result directory holds env_info.txt,
one log per phase, summary.txt and compact_summary.txt with the reference's section titles and grep patterns.
`--impl reference` runs the reference's own binaries (built unmodified under baseline/_ref/bin) through the
same phases, which gives the same-box comparison.
"""
from __future__ import annotations

import argparse
import os
import re
import shutil
import subprocess
import sys
import time
from typing import Dict, List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

DEFAULTS: Dict[str, Dict[str, str]] = {
    "hbm_kv": dict(HBM_WORKING_SET_MIB="8192", HBM_ITERS="1000", KV_TRANSFER_MIB="16384", KV_ITERS="1000"),
    "multi_kv": dict(HBM_WORKING_SET_MIB="32768", HBM_ITERS="1000", KV_TRANSFER_MIB="8192", KV_ITERS="1000", KV_PARALLEL="4"),
    "trace_decode": dict(LAYERS="32", KV_HEADS="8", HEAD_DIM="128", ELEM_BYTES="2", DECODE_CONTEXT="16384", DECODE_GEN="512",
                         FFN_DIM="8192", KV_DISTS="computed cached", KV_ITERS_COMPUTED="10000", KV_ITERS_CACHED="1000",
                         KV_ITERS_INPUT="1000"),
    "vllm_decode": dict(LAYERS="80", KV_HEADS="8", HEAD_DIM="128", ELEM_BYTES="2", DECODE_CONTEXT="65536", DECODE_GEN="128",
                        DECODE_BATCH="16", TILE_TOKENS="128", KV_DISTS="computed cached", KV_ITERS_COMPUTED="10000",
                        KV_ITERS_CACHED="1000", KV_ITERS_INPUT="1000", REPEATS="1"),
}
COMMON = dict(SRC_GPU="0", DST_GPU="1", START_DELAY_SEC="1", ENABLE_DMON="1")

PRESETS: Dict[str, Dict[str, str]] = {
    # the reference's wrapper scripts
    "stress": dict(HBM_WORKING_SET_MIB="32768", HBM_ITERS="1000", KV_TRANSFER_MIB="16384", KV_ITERS="3000"),
    "real_trace": dict(LAYERS="80", DECODE_CONTEXT="32768", DECODE_GEN="256", FFN_DIM="16384", KV_DISTS="computed cached",
                       KV_ITERS_COMPUTED="10000", KV_ITERS_CACHED="2000"),
    "real_trace_small": dict(LAYERS="32", DECODE_CONTEXT="16384", DECODE_GEN="512", FFN_DIM="8192", KV_DISTS="computed cached",
                             KV_ITERS_COMPUTED="10000", KV_ITERS_CACHED="5000"),
    "vllm_real_trace": dict(LAYERS="80", DECODE_CONTEXT="65536", DECODE_GEN="128", DECODE_BATCH="16", TILE_TOKENS="128",
                            KV_DISTS="computed cached input", KV_ITERS_COMPUTED="10000", KV_ITERS_CACHED="1000",
                            KV_ITERS_INPUT="1000", REPEATS="1"),
    # Qwen3-8B geometry, sized to finish in about a minute on a B200 pair
    "qwen3_quick": dict(LAYERS="36", DECODE_CONTEXT="8192", DECODE_GEN="64", DECODE_BATCH="16", FFN_DIM="12288", TILE_TOKENS="1024",
                        KV_DISTS="computed", KV_ITERS_COMPUTED="300", KV_ITERS_CACHED="100", KV_ITERS_INPUT="100",
                        HBM_WORKING_SET_MIB="8192", HBM_ITERS="300", KV_TRANSFER_MIB="4096", KV_ITERS="60"),
}

DECODE_PATTERN = ("GPU:|layers=|context=|batch=|KV cache:|Time:|Generated tokens:|Active decode batch:|Throughput:|"
                  "Effective sequence-throughput:|Approx KV read traffic:|Approx KV append write:|Approx KV write traffic:|"
                  "Approx FFN traffic:|Approx partial write traffic:|Approx total traffic:|Approx bandwidth:")
KV_PATTERN = ("src_gpu=|peer_access|KV geometry:|Trace quantiles:|sampled tokens:|sampled bytes:|max transfer allocation:|"
              "Trace-shaped KV transfer done:|transfers:|total:|time:|bw:")
HBM_KV_PATTERN = "HBM stress done|KV transfer done|src_gpu=|dst_gpu=|gpu=|working_set=|size=|iters=|GiB/s|time|bw"


def log(msg: str) -> None:
    print(f"[{time.strftime('%F %T')}] {msg}", flush=True)


class Harness:
    def __init__(self, kind: str, cfg: Dict[str, str], out_dir: str, impl: str, dry_run: bool):
        self.kind, self.cfg, self.out, self.impl, self.dry = kind, cfg, out_dir, impl, dry_run
        self.ref_bin = os.environ.get("SKYGDR_REF_BIN", os.path.join(ROOT, "baseline", "_ref", "bin"))
        self.env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
        self.commands: List[List[str]] = []

    # ---- the four programs, in either implementation --------------------------------------------------------
    def prog(self, name: str, args: List[str]) -> List[str]:
        if self.impl == "reference":
            return [os.path.join(self.ref_bin, name)] + args
        module = {"decode_hbm_stress": "decode_hbm_stress", "kv_nvlink_transfer": "kv_nvlink_transfer",
                  "kv_nvlink_transfer_trace": "kv_nvlink_transfer_trace",
                  "decode_vllm_kvcache_hbm_stress": "decode_kvcache_stress",
                  "decode_transformer_kvcache_stress": "decode_kvcache_stress"}[name]
        if name == "decode_transformer_kvcache_stress":
            args = args + ["--mode", "model", "--batch", "1"]
        return [sys.executable, "-m", f"skygdr_b200.cli.{module}"] + args

    def hbm(self) -> List[str]:
        c = self.cfg
        return self.prog("decode_hbm_stress", [c["DST_GPU"], c["HBM_WORKING_SET_MIB"], c["HBM_ITERS"]])

    def kv_fixed(self) -> List[str]:
        c = self.cfg
        return self.prog("kv_nvlink_transfer", [c["SRC_GPU"], c["DST_GPU"], c["KV_TRANSFER_MIB"], c["KV_ITERS"]])

    def kv_trace(self, dist: str, iters: Optional[str] = None) -> List[str]:
        c = self.cfg
        return self.prog("kv_nvlink_transfer_trace", ["--src", c["SRC_GPU"], "--dst", c["DST_GPU"], "--dist", dist, "--layers", c["LAYERS"],
                                                      "--kv-heads", c["KV_HEADS"], "--head-dim", c["HEAD_DIM"], "--elem-bytes", c["ELEM_BYTES"],
                                                      "--iters", iters or c[f"KV_ITERS_{dist.upper()}"]])

    def decode(self, small: bool = False) -> List[str]:
        c = self.cfg
        if self.kind == "trace_decode":
            a = ["--gpu", c["DST_GPU"], "--layers", "4" if small else c["LAYERS"], "--kv-heads", c["KV_HEADS"], "--head-dim", c["HEAD_DIM"],
                 "--context", "1024" if small else c["DECODE_CONTEXT"], "--gen", "8" if small else c["DECODE_GEN"], "--ffn-dim", c["FFN_DIM"]]
            return self.prog("decode_transformer_kvcache_stress", a)
        a = ["--gpu", c["DST_GPU"], "--layers", "8" if small else c["LAYERS"], "--kv-heads", c["KV_HEADS"], "--head-dim", c["HEAD_DIM"],
             "--context", "1024" if small else c["DECODE_CONTEXT"], "--gen", "8" if small else c["DECODE_GEN"],
             "--batch", "4" if small else c["DECODE_BATCH"], "--tile-tokens", c["TILE_TOKENS"]]
        return self.prog("decode_vllm_kvcache_hbm_stress", a)

    # ---- process plumbing -----------------------------------------------------------------------------------
    def path(self, name: str) -> str:
        return os.path.join(self.out, name)

    def start(self, cmd: List[str], logname: str) -> Optional[subprocess.Popen]:
        self.commands.append(cmd)
        log("RUN: " + " ".join(cmd) + f" > {logname}")
        if self.dry:
            open(self.path(logname), "w").write("dry run: " + " ".join(cmd) + "\n")
            return None
        return subprocess.Popen(cmd, stdout=open(self.path(logname), "w"), stderr=subprocess.STDOUT, env=self.env, cwd=ROOT)

    def run(self, cmd: List[str], logname: str, must_pass: bool = True) -> None:
        p = self.start(cmd, logname)
        if p is not None and p.wait() != 0 and must_pass:
            raise SystemExit(f"ERROR: {' '.join(cmd)} exited {p.returncode}; see {self.path(logname)}")

    def overlapped(self, first: List[str], first_log: str, others: List[List[str]], other_logs: List[str]) -> None:
        a = self.start(first, first_log)
        if not self.dry:
            time.sleep(float(self.cfg["START_DELAY_SEC"]))        # the workload is already running when the competitor starts
        ps = [self.start(c, l) for c, l in zip(others, other_logs)]
        bad = [p.args for p in ps + [a] if p is not None and p.wait() != 0]
        if bad:
            raise SystemExit(f"ERROR: overlapped phase failed: {bad}")

    def dmon_start(self, tag: str) -> Optional[subprocess.Popen]:
        if self.dry or self.cfg["ENABLE_DMON"] != "1" or shutil.which("nvidia-smi") is None:
            return None
        gpus = ",".join(sorted({self.cfg["SRC_GPU"], self.cfg["DST_GPU"]}))
        return subprocess.Popen(["nvidia-smi", "dmon", "-i", gpus, "-s", "pucvmt"], stdout=open(self.path(f"dmon_{tag}.log"), "w"),
                                stderr=subprocess.STDOUT)

    @staticmethod
    def dmon_stop(p: Optional[subprocess.Popen]) -> None:
        if p is not None:
            p.terminate()
            try:
                p.wait(timeout=5)
            except subprocess.TimeoutExpired:
                p.kill()

    def phase(self, tag: str, fn) -> None:
        d = self.dmon_start(tag)
        try:
            fn()
        finally:
            self.dmon_stop(d)

    # ---- files ----------------------------------------------------------------------------------------------
    def config_lines(self) -> List[str]:
        keys = list(COMMON)[:2] + [k for k in DEFAULTS[self.kind]]
        return [f"{k}={self.cfg[k]}" for k in keys]

    def write_env_info(self) -> None:
        with open(self.path("env_info.txt"), "w") as f:
            f.write("Benchmark configuration\n=======================\n" + "\n".join(self.config_lines()) + f"\nIMPL={self.impl}\n\n")
            f.write("CUDA / GPU information\n======================\n")
            for cmd in (["nvcc", "--version"], ["nvidia-smi"]):
                f.write(self._capture(cmd))
            f.write("\nTopology\n========\n" + self._capture(["nvidia-smi", "topo", "-m"]))

    @staticmethod
    def _capture(cmd: List[str]) -> str:
        if shutil.which(cmd[0]) is None:
            return f"{cmd[0]}: not found\n"
        try:
            return subprocess.run(cmd, capture_output=True, text=True, timeout=30).stdout
        except Exception as exc:
            return f"{' '.join(cmd)}: {exc!r}\n"

    def extract(self, title: str, logname: str, pattern: str) -> str:
        head = f"\n================ {title} ================\n"
        p = self.path(logname)
        if not os.path.exists(p):
            return head + f"missing logfile: {p}\n"
        rx = re.compile(pattern)
        return head + "".join(l for l in open(p, errors="replace") if rx.search(l))

    def compact(self, title: str, prefix: str, pattern: str) -> str:
        rx = re.compile(pattern)
        out = [title, "=" * len(title)]
        for name in sorted(os.listdir(self.out)):
            if name.startswith(prefix) and name.endswith(".log"):
                out += [f"{self.path(name)}:{l.rstrip()}" for l in open(self.path(name), errors="replace") if rx.search(l)]
        return "\n".join(out) + "\n"

    # ---- the four harnesses ---------------------------------------------------------------------------------
    def run_hbm_kv(self) -> str:
        self.run(self.hbm(), "decode_hbm_alone.log")
        self.run(self.kv_fixed(), "kv_transfer_alone.log")
        self.overlapped(self.hbm(), "decode_hbm_overlap.log", [self.kv_fixed()], ["kv_transfer_overlap.log"])
        s = "Benchmark summary\n=================\n\n" + "\n".join(self.config_lines()) + "\n"
        for title, name in (("decode_hbm_stress alone", "decode_hbm_alone.log"), ("kv_nvlink_transfer alone", "kv_transfer_alone.log"),
                            ("decode_hbm_stress overlap", "decode_hbm_overlap.log"), ("kv_nvlink_transfer overlap", "kv_transfer_overlap.log")):
            s += self.extract(title, name, HBM_KV_PATTERN)
        return s

    def run_multi_kv(self) -> str:
        n = int(self.cfg["KV_PARALLEL"])
        self.overlapped(self.hbm(), "hbm_overlap.log", [self.kv_fixed() for _ in range(n)], [f"kv_{i}.log" for i in range(n)])
        s = "Benchmark summary\n=================\n\n" + "\n".join(self.config_lines()) + "\n"
        s += self.extract("decode_hbm_stress overlap", "hbm_overlap.log", HBM_KV_PATTERN)
        for i in range(n):
            s += self.extract(f"kv_nvlink_transfer {i} overlap", f"kv_{i}.log", HBM_KV_PATTERN)
        return s

    def run_decode(self) -> str:
        c = self.cfg
        dists = c["KV_DISTS"].split()
        for d in dists:
            if d not in ("computed", "cached", "input"):
                raise SystemExit(f"ERROR: Unknown KV dist={d}. Use computed, cached, or input.")
        vllm = self.kind == "vllm_decode"
        stem = "decode_vllm" if vllm else "decode"
        name = "decode_vllm_kvcache_hbm_stress" if vllm else "decode_transformer_kvcache_stress"
        log("Warmup: decode")
        self.run(self.decode(small=True), "warmup_decode.log", must_pass=False)
        log("Warmup: trace-shaped KV transfer")
        self.run(self.kv_trace("computed", "8"), "warmup_kv.log", must_pass=False)
        reps = int(c.get("REPEATS", "1"))
        for r in range(1, reps + 1):
            sfx = f"_r{r}" if vllm else ""
            self.phase(f"r{r}_decode_alone", lambda: self.run(self.decode(), f"{stem}_alone{sfx}.log"))
            for d in dists:
                self.phase(f"r{r}_kv_{d}_alone", lambda d=d: self.run(self.kv_trace(d), f"kv_{d}_alone{sfx}.log"))
            for d in dists:
                self.phase(f"r{r}_overlap_{d}", lambda d=d: self.overlapped(self.decode(), f"{stem}_overlap_{d}{sfx}.log",
                                                                           [self.kv_trace(d)], [f"kv_{d}_overlap{sfx}.log"]))
        title = ("Optimized vLLM-like decode + trace-shaped KV transfer benchmark" if vllm
                 else "Transformer-style decode + trace-shaped KV transfer benchmark")
        s = title + "\n" + "=" * len(title) + "\n\nConfiguration\n-------------\n" + "\n".join(self.config_lines()) + "\n"
        for r in range(1, reps + 1):
            sfx = f"_r{r}" if vllm else ""
            s += "\n################################################################\n" + f"Repeat {r}\n" + "#" * 64 + "\n"
            s += self.extract(f"{name} alone, repeat={r}", f"{stem}_alone{sfx}.log", DECODE_PATTERN)
            for d in dists:
                s += self.extract(f"kv_nvlink_transfer_trace alone, dist={d}, repeat={r}", f"kv_{d}_alone{sfx}.log", KV_PATTERN)
            for d in dists:
                s += self.extract(f"{stem} overlap, dist={d}, repeat={r}", f"{stem}_overlap_{d}{sfx}.log", DECODE_PATTERN)
                s += self.extract(f"kv transfer overlap, dist={d}, repeat={r}", f"kv_{d}_overlap{sfx}.log", KV_PATTERN)
        return s

    def main(self) -> int:
        os.makedirs(self.out, exist_ok=True)
        if self.impl == "reference" and not self.dry and not os.path.isdir(self.ref_bin):
            raise SystemExit(f"ERROR: reference binaries not found under {self.ref_bin}. Build them with baseline/build_ref.sh.")
        log(f"Output directory: {self.out}")
        self.write_env_info()
        s = {"hbm_kv": self.run_hbm_kv, "multi_kv": self.run_multi_kv}.get(self.kind, self.run_decode)()
        open(self.path("summary.txt"), "w").write(s)
        print(s)
        if self.kind in ("trace_decode", "vllm_decode"):
            c = self.compact("Compact decode summary", "decode", "Time:|Throughput:|Effective sequence-throughput:|Approx bandwidth:")
            c += "\n" + self.compact("Compact KV transfer summary", "kv_", "total:|time:|bw:")
            open(self.path("compact_summary.txt"), "w").write(c)
            print(c)
        log(f"Done. Results saved to: {self.out}")
        return 0


def resolve_config(kind: str, preset: Optional[str], environ=os.environ) -> Dict[str, str]:
    """Defaults of the harness < the preset < environment variables (the reference's wrappers set the environment)."""
    cfg = dict(COMMON)
    cfg.update(DEFAULTS[kind])
    if preset:
        if preset not in PRESETS:
            raise SystemExit(f"ERROR: unknown preset {preset}; known: {', '.join(sorted(PRESETS))}")
        cfg.update({k: v for k, v in PRESETS[preset].items() if k in cfg})
    for k in list(cfg):
        if environ.get(k):
            cfg[k] = environ[k]
    return cfg


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kind", choices=sorted(DEFAULTS))
    ap.add_argument("--preset", default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--out-dir", default=None)
    ap.add_argument("--dry-run", action="store_true", help="write the plan (commands, file layout, summaries) without starting a program")
    a = ap.parse_args(argv)
    cfg = resolve_config(a.kind, a.preset)
    stamp = time.strftime("%Y%m%d_%H%M%S")
    default_dir = {"hbm_kv": "bench_results_", "multi_kv": "overlap_multi_kv_", "trace_decode": "trace_decode_results_",
                   "vllm_decode": "final_vllm_decode_kv_results_"}[a.kind] + stamp
    out = a.out_dir or os.environ.get("OUT_DIR") or default_dir
    return Harness(a.kind, cfg, out, a.impl, a.dry_run).main()


if __name__ == "__main__":
    raise SystemExit(main())
