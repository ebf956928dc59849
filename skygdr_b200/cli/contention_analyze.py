"""Figures and tables of the contention studies from hand-editable summary CSVs.

    python -m skygdr_b200.cli.contention_analyze --partA partA_memcpy_impact.csv --partB partB_size_impact.csv --out_dir figs

The reference's figure script (src/tools/contention2_v2_analyze.py:814-815) reads two summary tables,
`partA_memcpy_impact.csv` (latency/throughput of the protected flow with and without a competing copy) and
`partB_size_impact.csv` (the same against message size), and draws the paper's figures. This does the same from
CSV: it always writes text tables (`*_table.txt`, the numbers behind each figure) and draws PNGs when matplotlib
is importable. Columns are taken by name; any numeric column is summarised as mean/min/max per value of the first column.
"""
from __future__ import annotations

import argparse
import csv
import os
import sys
from collections import defaultdict


def summarise(path: str):
    rows = list(csv.DictReader(open(path)))
    if not rows:
        return [], []
    key = list(rows[0].keys())[0]
    groups = defaultdict(list)
    for r in rows:
        groups[r[key]].append(r)
    numeric = [c for c in rows[0] if c != key and all(_isnum(r[c]) for r in rows if r[c] != "")]
    table = []
    for k, rs in groups.items():
        line = {key: k}
        for c in numeric:
            v = [float(r[c]) for r in rs if r[c] != ""]
            if v:
                line[f"{c}_mean"], line[f"{c}_min"], line[f"{c}_max"] = sum(v) / len(v), min(v), max(v)
        table.append(line)
    return table, numeric


def _isnum(s: str) -> bool:
    try:
        float(s)
        return True
    except ValueError:
        return False


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--partA", default="")
    ap.add_argument("--partB", default="")
    ap.add_argument("--out_dir", required=True)
    a = ap.parse_args(argv)
    os.makedirs(a.out_dir, exist_ok=True)
    for name, path in (("partA", a.partA), ("partB", a.partB)):
        if not path:
            continue
        table, numeric = summarise(path)
        if not table:
            continue
        cols = list(table[0].keys())
        with open(os.path.join(a.out_dir, f"{name}_table.txt"), "w") as fp:
            fp.write("\t".join(cols) + "\n")
            for line in table:
                fp.write("\t".join(f"{line.get(c, ''):.4g}" if isinstance(line.get(c), float) else str(line.get(c, "")) for c in cols) + "\n")
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt

            fig, ax = plt.subplots(figsize=(7, 4))
            xs = [line[cols[0]] for line in table]
            for c in numeric[:4]:
                ax.plot(xs, [line.get(f"{c}_mean", float("nan")) for line in table], marker="o", label=c)
            ax.set_xlabel(cols[0]); ax.legend(); fig.tight_layout()
            fig.savefig(os.path.join(a.out_dir, f"{name}.png"), dpi=120)
        except Exception as exc:
            print(f"plot skipped: {exc}", file=sys.stderr)
        print(f"{name}: {len(table)} groups -> {a.out_dir}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
