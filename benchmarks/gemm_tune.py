"""Tunes the decode GEMM's tile, split and split form per shape, and writes the table the chooser consults first.

    python benchmarks/gemm_tune.py [--tps 1,2,4,8] [--batch-per-gpu 16] [--out skygdr_b200/ops/gemm_tuned.json]

For every projection of one rank of Qwen3-8B at the given tensor-parallel degrees (QKV, O, gate/up, down, lm_head; batch
16 x tp tokens) every candidate (token tile 16-128, 1-16 splits through the workspace, 2-8 splits inside a thread-block
cluster) is timed the way a decode step runs it: a CUDA graph of L launches back to back with programmatic dependent launch
between them, each launch on its own copy of the weights so that they come from HBM, not L2. Time per launch = replay
time / L. The fastest candidate per shape goes into the table as "M,N,K,gated": [token tile, splits, cluster]; shapes
that are not in the table keep the cost model's choice (ops/gemm.py, pick_config).
"""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import skygdr_b200.ops as ops  # noqa: E402
from skygdr_b200.ops.gemm import GemmWorkspace, pick_config  # noqa: E402


def time_chain(launch, weights, replays=5):
    for w in weights[:2]:
        launch(w)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        with torch.cuda.graph(g, stream=st):
            for w in weights:
                launch(w)
    torch.cuda.synchronize()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (replays * len(weights))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tps", default="1,2,4,8")
    ap.add_argument("--batch-per-gpu", type=int, default=16)
    ap.add_argument("--out", default=os.path.join(ROOT, "skygdr_b200", "ops", "gemm_tuned.json"))
    ap.add_argument("--report", default="", help="optional JSON with every candidate's time")
    a = ap.parse_args()
    dev = torch.device("cuda", 0)
    table, report = {}, {}
    for tp in [int(t) for t in a.tps.split(",")]:
        M = a.batch_per_gpu * tp
        vocab = (151936 + tp - 1) // tp
        shapes = [("qkv", 6144 // tp, 4096, False), ("o", 4096, 4096 // tp, False), ("gate_up", 12288 // tp, 4096, True),
                  ("down", 4096, 12288 // tp, False), ("lm_head", vocab, 4096, False)]
        for name, N, K, gated in shapes:
            wbytes = (2 * N if gated else N) * K * 2
            L = max(3, min(36, (400 << 20) // wbytes))
            ws_ = [torch.randn((2 * N if gated else N), K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(L)]
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            wsp = GemmWorkspace(dev)
            cands = {}
            for ntok in (16, 32, 64, 128):
                if (ntok > 2 * M and ntok != 16) or (gated and ntok > 128):
                    continue
                for cluster in (False, True):
                    for s in ((2, 3, 4, 5, 6, 7, 8) if cluster else (1, 2, 3, 4, 5, 6, 8, 10, 12, 16)):
                        if s > 1 and (K // 64) // s < 2:
                            continue
                        try:
                            us = time_chain(lambda w: ops.gemm(x, w, out=out, gated=gated, splits=s, ntok=ntok, ws=wsp, cluster=cluster), ws_)
                        except Exception as exc:                       # a candidate the launcher refuses is just not a candidate
                            cands[f"{ntok}x{s}{'c' if cluster else ''}"] = "refused: " + str(exc)[:60]
                            continue
                        cands[f"{ntok}x{s}{'c' if cluster else ''}"] = round(us, 2)
            timed = {k: v for k, v in cands.items() if isinstance(v, float)}
            best = min(timed, key=timed.get)
            ntok, rest = best.split("x")
            cluster = rest.endswith("c")
            splits = int(rest.rstrip("c"))
            model = pick_config(M, N, K, 148, gated)
            key = f"{M},{N},{K},{int(gated)}"
            table[key] = [int(ntok), splits, int(cluster)]
            report[key] = {"name": f"tp{tp} {name}", "best": best, "best_us": timed[best], "model_choice": f"{model[0]}x{model[1]}",
                           "model_us": timed.get(f"{model[0]}x{model[1]}"), "ideal_us_at_6.46TBs": round(wbytes / 6.46e6, 2), "all": cands}
            print(key, json.dumps({k: v for k, v in report[key].items() if k != "all"}), flush=True)
            del ws_
            torch.cuda.empty_cache()
    json.dump({"how": "benchmarks/gemm_tune.py on B200: CUDA-graph chain of launches, weights cold in HBM; [token tile, splits, cluster]",
               "table": table}, open(a.out, "w"), indent=1, sort_keys=True)
    if a.report:
        os.makedirs(os.path.dirname(os.path.abspath(a.report)), exist_ok=True)
        json.dump(report, open(a.report, "w"), indent=1)


if __name__ == "__main__":
    main()
