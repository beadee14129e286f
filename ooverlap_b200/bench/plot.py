"""Plots from benchmark JSON lines (needs matplotlib; prints a table instead when it is not installed).

    python -m ooverlap_b200.bench.plot sweep_8.jsonl --kind sweep --out sweep_8.png
    python -m ooverlap_b200.bench.plot overlap_8.jsonl --kind overlap --out overlap_8.png

Capability parity: test/plot_external_p2p_collective.py, test/plot_eval_sm90.py and test/plot_vllm_sweeps.py of
the reference.
"""
from __future__ import annotations

import argparse
import sys
from collections import defaultdict

from .aggregate import read_lines


def sweep_series(rows):
    """{collective: {label: [(bytes, bus_gbs)]}} with the best CTA budget per algorithm and size."""
    best = defaultdict(dict)
    for r in rows:
        label = "nccl" if r["impl"] == "nccl" else r["algo"]
        k = (r["collective"], label, r["bytes"])
        if k not in best or r["bus_gbs"] > best[k]:
            best[k] = r["bus_gbs"]
    series = defaultdict(lambda: defaultdict(list))
    for (coll, label, nbytes), bw in sorted(best.items()):
        series[coll][label].append((nbytes, bw))
    return series


def overlap_series(rows):
    """{(op, M): {impl label: best us}}"""
    out = defaultdict(dict)
    for r in rows:
        label = r["impl"]
        if label == "ours_fused":
            label = f"ours_fused(nvls={r.get('nvls')})"
        k = (r["op"], r["M"])
        if label not in out[k] or r["us"] < out[k][label]:
            out[k][label] = r["us"]
    return out


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("file")
    p.add_argument("--kind", default="sweep", choices=["sweep", "overlap"])
    p.add_argument("--out", default="")
    args = p.parse_args(argv)
    rows = read_lines([args.file])
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        plt = None
    if args.kind == "sweep":
        series = sweep_series(rows)
        if plt is None or not args.out:
            for coll, by_label in series.items():
                for label, pts in by_label.items():
                    print(coll, label, " ".join(f"{b}:{bw}" for b, bw in pts))
            return 0
        fig, axes = plt.subplots(1, len(series), figsize=(6 * len(series), 4))
        axes = [axes] if len(series) == 1 else list(axes)
        for ax, (coll, by_label) in zip(axes, series.items()):
            for label, pts in by_label.items():
                ax.plot([b for b, _ in pts], [bw for _, bw in pts], marker="o", label=label)
            ax.set_xscale("log", base=2)
            ax.set_xlabel("message bytes")
            ax.set_ylabel("bus GB/s")
            ax.set_title(coll)
            ax.legend(fontsize=7)
        fig.tight_layout()
        fig.savefig(args.out, dpi=120)
    else:
        series = overlap_series(rows)
        if plt is None or not args.out:
            for k, by_label in series.items():
                print(k, by_label)
            return 0
        fig, ax = plt.subplots(figsize=(10, 4))
        labels = sorted({lb for v in series.values() for lb in v})
        keys = sorted(series)
        width = 0.8 / max(1, len(labels))
        for i, lb in enumerate(labels):
            ax.bar([j + i * width for j in range(len(keys))], [series[k].get(lb, 0) for k in keys], width, label=lb)
        ax.set_xticks([j + 0.4 for j in range(len(keys))])
        ax.set_xticklabels([f"{op}\\nM={m}" for op, m in keys], fontsize=7)
        ax.set_ylabel("us")
        ax.legend(fontsize=7)
        fig.tight_layout()
        fig.savefig(args.out, dpi=120)
    return 0


if __name__ == "__main__":
    sys.exit(main())
