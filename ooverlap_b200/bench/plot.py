"""Plots from benchmark JSON lines.

    python -m ooverlap_b200.bench.plot sweep_8.jsonl --kind sweep --out sweep_8.svg          # bus GB/s over message size
    python -m ooverlap_b200.bench.plot sweep_8.jsonl --kind latency --out latency_8.svg      # microseconds over size
    python -m ooverlap_b200.bench.plot sweep_8.jsonl --kind efficiency --out eff_8.svg       # fraction of the best per size
    python -m ooverlap_b200.bench.plot overlap_8.jsonl --kind overlap --out overlap_8.svg    # us per (op, M) and arm
    python -m ooverlap_b200.bench.plot vllm_*.jsonl --kind serving --out serving.svg         # output tok/s per backend, batch

With matplotlib installed and an ``--out`` that does not end in ``.svg`` the figure is drawn by matplotlib (PNG, PDF,
...); otherwise by the small SVG writer in this file, which needs nothing but the standard library.  Without
``--out`` the series are printed as text.

Capability parity: test/plot_external_p2p_collective.py (bandwidth and latency curves), test/plot_tma_efficiency_vs_best.py,
test/plot_eval_sm90.py (overlap speed-ups) and test/plot_vllm_sweeps.py (throughput per backend) of the reference.
"""
from __future__ import annotations

import argparse
import math
import sys
from collections import defaultdict
from xml.sax.saxutils import escape

from .aggregate import aggregate, read_lines

COLOURS = ["#1f77b4", "#d62728", "#2ca02c", "#ff7f0e", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#bcbd22", "#17becf"]


# ---------------------------------------------------------------------------------------------------------------------
# series
# ---------------------------------------------------------------------------------------------------------------------
def _sweep_best(rows, field, better):
    best = {}
    for r in rows:
        if field not in r or "bytes" not in r or "collective" not in r or "impl" not in r:
            continue
        label = "nccl" if r["impl"] == "nccl" else (r.get("algo") or r["impl"])
        k = (r["collective"], label, r["bytes"])
        if k not in best or better(r[field], best[k]):
            best[k] = r[field]
    series = defaultdict(lambda: defaultdict(list))
    for (coll, label, nbytes), v in sorted(best.items()):
        series[coll][label].append((nbytes, v))
    return series


def sweep_series(rows):
    """{collective: {label: [(bytes, bus_gbs)]}} with the best CTA budget per algorithm and size."""
    return _sweep_best(rows, "bus_gbs", lambda a, b: a > b)


def latency_series(rows):
    """{collective: {label: [(bytes, us)]}} with the best CTA budget per algorithm and size."""
    return _sweep_best(rows, "us", lambda a, b: a < b)


def efficiency_series(rows):
    """{collective: {label: [(bytes, fraction)]}}: every algorithm's time relative to the fastest entry of that size
    (1.0 = it is the fastest), NCCL included."""
    lat = latency_series(rows)
    out = defaultdict(lambda: defaultdict(list))
    for coll, by_label in lat.items():
        fastest = {}
        for pts in by_label.values():
            for b, us in pts:
                fastest[b] = min(us, fastest.get(b, us))
        for label, pts in by_label.items():
            out[coll][label] = [(b, fastest[b] / us if us > 0 else 0.0) for b, us in pts]
    return out


def overlap_series(rows):
    """{(op, M): {impl label: best us}}"""
    out = defaultdict(dict)
    for r in rows:
        if "op" not in r or "M" not in r or "us" not in r or "impl" not in r:
            continue
        label = r["impl"]
        if label == "ours_fused":
            label = f"ours_fused(nvls={r.get('nvls')})"
        k = (r["op"], r["M"])
        if label not in out[k] or r["us"] < out[k][label]:
            out[k][label] = r["us"]
    return out


def serving_series(rows, metric="output_tok_s"):
    """{(model, tp, batch): {backend: median of the metric over all runs and backend orders}}"""
    out = {}
    for rec in aggregate(rows, metric, ["model", "tp", "batch"], "backend"):
        out[(rec["model"], rec["tp"], rec["batch"])] = {b: s["median"] for b, s in rec["stats"].items()}
    return out


# ---------------------------------------------------------------------------------------------------------------------
# SVG writer (standard library only)
# ---------------------------------------------------------------------------------------------------------------------
def _ticks(lo, hi, log):
    if log:
        a, b = math.floor(math.log2(lo)), math.ceil(math.log2(hi))
        step = max(1, (b - a) // 8)
        return [2.0 ** e for e in range(a, b + 1, step)]
    if hi <= lo:
        return [lo]
    raw = (hi - lo) / 5
    mag = 10 ** math.floor(math.log10(raw))
    step = min((s * mag for s in (1, 2, 5, 10) if s * mag >= raw), default=raw)
    first = math.ceil(lo / step) * step
    return [first + i * step for i in range(int((hi - first) / step) + 1)]


def _fmt(v):
    if v >= 1 << 30 and v % (1 << 30) == 0:
        return f"{int(v) >> 30}Gi"
    if v >= 1 << 20 and v % (1 << 20) == 0:
        return f"{int(v) >> 20}Mi"
    if v >= 1 << 10 and v % (1 << 10) == 0:
        return f"{int(v) >> 10}Ki"
    return f"{v:g}"


def svg_lines(panels, xlabel, ylabel, logx=True, logy=False, width=520, height=340) -> str:
    """One panel per entry of ``panels`` ({title: {label: [(x, y)]}}), side by side, as an SVG document."""
    n = max(1, len(panels))
    ml, mr, mt, mb = 62, 150, 30, 46
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{n * width}" height="{height}" font-family="sans-serif" font-size="11">',
             f'<rect width="{n * width}" height="{height}" fill="white"/>']
    for pi, (title, by_label) in enumerate(panels.items()):
        pts = [p for v in by_label.values() for p in v if (not logx or p[0] > 0) and (not logy or p[1] > 0)]
        if not pts:
            continue
        x0, x1 = min(p[0] for p in pts), max(p[0] for p in pts)
        y0, y1 = (min(p[1] for p in pts) if logy else 0.0), max(p[1] for p in pts) * 1.05
        if x1 == x0:
            x1 = x0 * 2 if x0 > 0 else 1.0
        if y1 <= y0:
            y1 = y0 + 1.0
        ox, pw, ph = pi * width + ml, width - ml - mr, height - mt - mb

        def sx(x):
            f = (math.log2(x) - math.log2(x0)) / (math.log2(x1) - math.log2(x0)) if logx else (x - x0) / (x1 - x0)
            return ox + f * pw

        def sy(y):
            f = (math.log2(y) - math.log2(y0)) / (math.log2(y1) - math.log2(y0)) if logy else (y - y0) / (y1 - y0)
            return mt + ph - f * ph

        parts.append(f'<rect x="{ox}" y="{mt}" width="{pw}" height="{ph}" fill="none" stroke="#444"/>')
        parts.append(f'<text x="{ox + pw / 2}" y="{mt - 10}" text-anchor="middle" font-size="13">{escape(str(title))}</text>')
        for t in _ticks(x0, x1, logx):
            if x0 <= t <= x1:
                parts.append(f'<line x1="{sx(t):.1f}" y1="{mt + ph}" x2="{sx(t):.1f}" y2="{mt + ph + 4}" stroke="#444"/>')
                parts.append(f'<text x="{sx(t):.1f}" y="{mt + ph + 16}" text-anchor="middle">{_fmt(t)}</text>')
        for t in _ticks(y0 if logy else 0.0, y1, logy):
            if y0 <= t <= y1:
                parts.append(f'<line x1="{ox}" y1="{sy(t):.1f}" x2="{ox + pw}" y2="{sy(t):.1f}" stroke="#ddd"/>')
                parts.append(f'<text x="{ox - 6}" y="{sy(t) + 4:.1f}" text-anchor="end">{_fmt(t)}</text>')
        parts.append(f'<text x="{ox + pw / 2}" y="{height - 8}" text-anchor="middle">{escape(xlabel)}</text>')
        parts.append(f'<text x="{pi * width + 14}" y="{mt + ph / 2}" text-anchor="middle" '
                     f'transform="rotate(-90 {pi * width + 14} {mt + ph / 2})">{escape(ylabel)}</text>')
        for li, (label, series) in enumerate(sorted(by_label.items())):
            c = COLOURS[li % len(COLOURS)]
            good = [(x, y) for x, y in series if (not logx or x > 0) and (not logy or y > 0)]
            if good:
                path = " ".join(f"{sx(x):.1f},{sy(y):.1f}" for x, y in good)
                parts.append(f'<polyline points="{path}" fill="none" stroke="{c}" stroke-width="1.6"/>')
                parts.extend(f'<circle cx="{sx(x):.1f}" cy="{sy(y):.1f}" r="2.2" fill="{c}"/>' for x, y in good)
            ly = mt + 12 + li * 15
            parts.append(f'<line x1="{ox + pw + 8}" y1="{ly - 4}" x2="{ox + pw + 26}" y2="{ly - 4}" stroke="{c}" stroke-width="2"/>')
            parts.append(f'<text x="{ox + pw + 30}" y="{ly}">{escape(str(label))}</text>')
    parts.append("</svg>")
    return "\n".join(parts)


def svg_bars(groups, ylabel, width=900, height=360) -> str:
    """Grouped bars: ``groups`` is {group label: {series label: value}}."""
    ml, mr, mt, mb = 62, 170, 20, 58
    labels = sorted({lb for v in groups.values() for lb in v})
    keys = list(groups)
    top = max((v for g in groups.values() for v in g.values()), default=1.0) * 1.08 or 1.0
    pw, ph = width - ml - mr, height - mt - mb
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="11">',
             f'<rect width="{width}" height="{height}" fill="white"/>',
             f'<rect x="{ml}" y="{mt}" width="{pw}" height="{ph}" fill="none" stroke="#444"/>']
    for t in _ticks(0.0, top, False):
        y = mt + ph - t / top * ph
        parts.append(f'<line x1="{ml}" y1="{y:.1f}" x2="{ml + pw}" y2="{y:.1f}" stroke="#ddd"/>')
        parts.append(f'<text x="{ml - 6}" y="{y + 4:.1f}" text-anchor="end">{_fmt(t)}</text>')
    parts.append(f'<text x="14" y="{mt + ph / 2}" text-anchor="middle" transform="rotate(-90 14 {mt + ph / 2})">{escape(ylabel)}</text>')
    gw = pw / max(1, len(keys))
    bw = gw * 0.8 / max(1, len(labels))
    for gi, k in enumerate(keys):
        for li, lb in enumerate(labels):
            v = groups[k].get(lb)
            if v is None:
                continue
            h = v / top * ph
            x = ml + gi * gw + gw * 0.1 + li * bw
            parts.append(f'<rect x="{x:.1f}" y="{mt + ph - h:.1f}" width="{bw:.1f}" height="{h:.1f}" fill="{COLOURS[li % len(COLOURS)]}"/>')
        for j, line in enumerate(str(k).split("\n")):
            parts.append(f'<text x="{ml + gi * gw + gw / 2:.1f}" y="{mt + ph + 16 + 13 * j}" text-anchor="middle">{escape(line)}</text>')
    for li, lb in enumerate(labels):
        ly = mt + 12 + li * 15
        parts.append(f'<rect x="{ml + pw + 10}" y="{ly - 9}" width="12" height="10" fill="{COLOURS[li % len(COLOURS)]}"/>')
        parts.append(f'<text x="{ml + pw + 28}" y="{ly}">{escape(str(lb))}</text>')
    parts.append("</svg>")
    return "\n".join(parts)


# ---------------------------------------------------------------------------------------------------------------------
# command line
# ---------------------------------------------------------------------------------------------------------------------
LINE_KINDS = {"sweep": (sweep_series, "bus GB/s", False), "latency": (latency_series, "us", True),
              "efficiency": (efficiency_series, "fraction of the fastest", False)}


def _matplotlib(out: str):
    if not out or out.endswith(".svg"):
        return None
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        return plt
    except ImportError:
        return None


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("files", nargs="+")
    p.add_argument("--kind", default="sweep", choices=["sweep", "latency", "efficiency", "overlap", "serving"])
    p.add_argument("--metric", default="output_tok_s", help="serving: the field to plot")
    p.add_argument("--out", default="", help="figure file; .svg (or no matplotlib) uses the built-in SVG writer")
    args = p.parse_args(argv)
    rows = read_lines(args.files)
    plt = _matplotlib(args.out)
    out = args.out
    if out and plt is None and not out.endswith(".svg"):
        out = out.rsplit(".", 1)[0] + ".svg"
        print(f"matplotlib is not installed: writing {out}", file=sys.stderr)
    if args.kind in LINE_KINDS:
        fn, ylabel, logy = LINE_KINDS[args.kind]
        series = fn(rows)
        if not out:
            for coll, by_label in series.items():
                for label, pts in by_label.items():
                    print(coll, label, " ".join(f"{b}:{v:.4g}" for b, v in pts))
            return 0
        if plt is None:
            with open(out, "w") as f:
                f.write(svg_lines(series, "message bytes", ylabel, logx=True, logy=logy))
            return 0
        fig, axes = plt.subplots(1, max(1, len(series)), figsize=(6 * max(1, len(series)), 4))
        axes = [axes] if len(series) <= 1 else list(axes)
        for ax, (coll, by_label) in zip(axes, series.items()):
            for label, pts in by_label.items():
                ax.plot([b for b, _ in pts], [v for _, v in pts], marker="o", label=label)
            ax.set_xscale("log", base=2)
            if logy:
                ax.set_yscale("log")
            ax.set_xlabel("message bytes")
            ax.set_ylabel(ylabel)
            ax.set_title(coll)
            ax.legend(fontsize=7)
        fig.tight_layout()
        fig.savefig(out, dpi=120)
        return 0
    if args.kind == "overlap":
        series = overlap_series(rows)
        groups = {f"{op}\nM={m}": v for (op, m), v in sorted(series.items())}
        ylabel = "us"
    else:
        series = serving_series(rows, args.metric)
        groups = {f"{model} tp{tp}\nbatch {batch}": v for (model, tp, batch), v in sorted(series.items(), key=lambda kv: str(kv[0]))}
        ylabel = args.metric
    if not out:
        for k, by_label in series.items():
            print(k, by_label)
        return 0
    if plt is None:
        with open(out, "w") as f:
            f.write(svg_bars(groups, ylabel))
        return 0
    fig, ax = plt.subplots(figsize=(10, 4))
    labels = sorted({lb for v in groups.values() for lb in v})
    keys = list(groups)
    width = 0.8 / max(1, len(labels))
    for i, lb in enumerate(labels):
        ax.bar([j + i * width for j in range(len(keys))], [groups[k].get(lb, 0) for k in keys], width, label=lb)
    ax.set_xticks([j + 0.4 for j in range(len(keys))])
    ax.set_xticklabels(keys, fontsize=7)
    ax.set_ylabel(ylabel)
    ax.legend(fontsize=7)
    fig.tight_layout()
    fig.savefig(out, dpi=120)
    return 0


if __name__ == "__main__":
    sys.exit(main())
