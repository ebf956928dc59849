"""Same-box comparison: the reference's own CUDA programs (built unmodified for sm_100 by baseline/build_ref.sh)
next to this runtime's equivalents, on the GPU(s) of this machine.

    python baseline/run_same_box.py [--gpus 1|2] [--out results/same_box.json]

One GPU: HBM stressor, memhog (rw), PCIe copy task (d2h, h2d), decode KV-cache stressor. Two GPUs add the NVLink
transfers (fixed size and trace-shaped). Every reference number is scraped from the program's own summary line.
"""
import argparse
import json
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref", "bin")
sys.path.insert(0, ROOT)
ENV = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))


def run(cmd, timeout=120):
    try:
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=ENV)
        return r.returncode, r.stdout + r.stderr
    except subprocess.TimeoutExpired:
        return 124, "timeout"


def grab(pattern, text, scale=1.0):
    m = re.findall(pattern, text)
    return float(m[-1]) * scale if m else None


def memhog_row(rows, out_path, py):
    """The reference's memhog cannot be read off its own summary line: it records its timing events on the legacy default
    stream while its kernels go to non-blocking streams (src/gpu_be_memhog_task.cu:297-336), so each event pair closes at once,
    the host loop queues launches for `--seconds` of wall time without waiting for any of them, and the GiB/s it prints divides
    by an interval that does not contain the kernels. With the default --iters=100 one launch repeats the pass 100 times and the
    queued launches take minutes to drain. So: the unmodified binary with --iters=1, for 1 s and for 3 s, timed from outside;
    what it processed (its own "processed=... GiB") more in the longer run over the extra wall time is its bandwidth (start-up
    and the drain of the launch queue, the same in both runs, cancel)."""
    import time

    G = 1.073741824
    exe = f"{REF}/gpu_be_memhog_task"
    runs = []
    if os.path.exists(exe):
        for seconds in (1, 3):
            cmd = [exe, "--gb=8", f"--seconds={seconds}", "--op=rw", "--iters=1"]
            t0 = time.perf_counter()
            rc, out = run(cmd, timeout=110)
            runs.append({"cmd": " ".join(cmd[1:]), "rc": rc, "wall_s": time.perf_counter() - t0, "processed_gib": grab(r"processed=([0-9.]+) GiB", out),
                         "launches": grab(r"launches=([0-9]+)", out), "its_own_avg_bw_gib_s": grab(r"avg BW=([0-9.]+) GiB/s", out)})
    ref = None
    if len(runs) == 2 and all(r["rc"] == 0 and r["processed_gib"] for r in runs) and runs[1]["wall_s"] > runs[0]["wall_s"]:
        ref = (runs[1]["processed_gib"] - runs[0]["processed_gib"]) / (runs[1]["wall_s"] - runs[0]["wall_s"]) * G
    rc_o, out_o = run(py + ["skygdr_b200.cli.gpu_memhog", "--gb=8", "--seconds=2", "--op=rw"])
    ours = grab(r"bw_gib_s=([0-9.]+)", out_o, G)
    rows.append({"what": "memhog rw, 8 GiB (reference: --iters=1, timed from outside over two run lengths)", "unit": "GB/s", "reference": ref, "ours": ours,
                 "reference_runs": runs, "ours_cmd": "skygdr_b200.cli.gpu_memhog --gb=8 --seconds=2 --op=rw", "rc": [runs[-1]["rc"] if runs else 127, rc_o],
                 "ours_tail": out_o.strip().splitlines()[-3:]})
    print(f"{rows[-1]['what'][:70]:70s} ref={ref} ours={ours} GB/s ratio={(ours / ref) if ours and ref else None}", flush=True)
    os.makedirs(os.path.dirname(os.path.abspath(out_path)), exist_ok=True)
    json.dump(rows, open(out_path, "w"), indent=1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--out", default="results/same_box.json")
    a = ap.parse_args()
    py = [sys.executable, "-m"]
    G = 1.073741824
    rows = []

    def add(name, ref_cmd, ref_pat, our_cmd, our_pat, unit="GB/s", ref_scale=G, our_scale=G):
        rc_r, out_r = run(ref_cmd) if os.path.exists(ref_cmd[0]) else (127, "reference program not built")
        rc_o, out_o = run(our_cmd)
        rows.append({"what": name, "unit": unit, "reference": grab(ref_pat, out_r, ref_scale), "ours": grab(our_pat, out_o, our_scale),
                     "reference_cmd": " ".join(ref_cmd[1:]), "ours_cmd": " ".join(our_cmd[2:]), "rc": [rc_r, rc_o],
                     "reference_tail": out_r.strip().splitlines()[-3:], "ours_tail": out_o.strip().splitlines()[-3:]})
        r = rows[-1]
        ratio = (r["ours"] / r["reference"]) if r["ours"] and r["reference"] else None
        print(f"{r['what'][:70]:70s} ref={r['reference']} ours={r['ours']} {r['unit']} ratio={ratio} rc={r['rc']}", flush=True)
        os.makedirs(os.path.dirname(os.path.abspath(a.out)), exist_ok=True)
        json.dump(rows, open(a.out, "w"), indent=1)          # after every row: a cut-off run keeps what it measured

    add("HBM stressor b += a*alpha, 8 GiB working set", [f"{REF}/decode_hbm_stress", "0", "8192", "300"], r"=\s*([0-9.]+) GiB/s",
        py + ["skygdr_b200.cli.decode_hbm_stress", "0", "8192", "300"], r"=\s*([0-9.]+) GiB/s")
    memhog_row(rows, a.out, py)
    for d in ("d2h", "h2d"):
        add(f"PCIe copy task {d}, 128 MiB chunks, 3 s", [f"{REF}/gpu_be_pcie_memcpy_task", "--seconds=3", f"--dir={d}", "--report_ms=500"],
            r"bw_gib_s=([0-9.]+)", py + ["skygdr_b200.cli.gpu_pcie_memcpy", "--seconds=3", f"--dir={d}", "--report_ms=500"], r"avg_bw_gib_s=([0-9.]+)")
    add("decode KV scan, 36 layers x 8 kv heads x 128, batch 16, context 8192, 16 steps (reference: fp32 KV, no block table; ours: bf16 paged GQA attention)",
        [f"{REF}/decode_vllm_kvcache_hbm_stress", "--gpu", "0", "--layers", "36", "--kv-heads", "8", "--head-dim", "128", "--context", "8192", "--gen", "16",
         "--batch", "16", "--report-every", "16"], r"sequence-throughput:\s*([0-9.]+)",
        py + ["skygdr_b200.cli.decode_kvcache_stress", "--layers", "36", "--kv-heads", "8", "--context", "8192", "--gen", "16", "--batch", "16"],
        r"sequence-throughput:\s*([0-9.]+)", unit="sequence-tokens/s", ref_scale=1.0, our_scale=1.0)
    if a.gpus >= 2:
        add("NVLink KV transfer GPU0->GPU1, 4 GiB x 30 (reference: contiguous cudaMemcpyPeerAsync; ours: paged gather + layout change kernel)",
            [f"{REF}/kv_nvlink_transfer", "0", "1", "4096", "30"], r"=\s*([0-9.]+) GiB/s",
            py + ["skygdr_b200.cli.kv_nvlink_transfer", "0", "1", "4096", "30"], r"=\s*([0-9.]+) GiB/s")
        add("NVLink KV transfer, trace-shaped (computed dist, 36 layers, <= 64k tokens), 200 transfers",
            [f"{REF}/kv_nvlink_transfer_trace", "--src", "0", "--dst", "1", "--iters", "200", "--dist", "computed", "--layers", "36", "--kv-heads", "8",
             "--head-dim", "128", "--elem-bytes", "2", "--max-tokens", "65536", "--seed", "1"], r"bw:\s+([0-9.]+) GiB/s",
            py + ["skygdr_b200.cli.kv_nvlink_transfer_trace", "--src", "0", "--dst", "1", "--iters", "200", "--dist", "computed", "--layers", "36",
                  "--max-tokens", "65536", "--seed", "1"], r"bw:\s+([0-9.]+) GiB/s")
    print(f"wrote {a.out}")


if __name__ == "__main__":
    main()
