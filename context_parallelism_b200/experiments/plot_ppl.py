"""Offline plots (matplotlib ``Agg`` backend, as Tests/bluscriptcp/plot_ppl_sweep.py:14): perplexity versus
position from ``CP_EVAL_OUT`` CSVs, and throughput / loss curves from trainer CSV logs."""
from __future__ import annotations

import argparse
import csv


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("csv", nargs="+", help="label=path pairs")
    ap.add_argument("--kind", default="ppl", choices=["ppl", "loss", "tok"])
    ap.add_argument("--out", default="plot.png")
    ap.add_argument("--smooth", type=int, default=64)
    a = ap.parse_args(argv)
    import matplotlib
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt
    fig, ax = plt.subplots(figsize=(9, 5))
    for item in a.csv:
        label, path = item.split("=", 1) if "=" in item else (item, item)
        rows = [r for r in csv.DictReader(l for l in open(path) if not l.startswith("#"))]
        if a.kind == "ppl":
            x, y = [int(r["pos"]) for r in rows], [float(r["ppl"]) for r in rows]
            k = max(1, a.smooth)
            y = [sum(y[max(0, i - k + 1):i + 1]) / len(y[max(0, i - k + 1):i + 1]) for i in range(len(y))]
            ax.set_xlabel("position"); ax.set_ylabel("perplexity"); ax.set_yscale("log")
        else:
            col = "loss" if a.kind == "loss" else "tok_per_sec"
            x, y = [int(r["step"]) for r in rows], [float(r[col]) for r in rows]
            ax.set_xlabel("step"); ax.set_ylabel(col)
        ax.plot(x, y, label=label)
    ax.legend(); ax.grid(alpha=0.3)
    fig.savefig(a.out, dpi=120, bbox_inches="tight")
    print(a.out)


if __name__ == "__main__":
    main()
