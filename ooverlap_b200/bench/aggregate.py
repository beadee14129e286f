"""Aggregates benchmark JSON lines over repeated runs and backend orders.

Input: one or more ``.jsonl`` files produced by ``serving_bench`` / ``overlap_bench`` / ``collective_sweep``
(possibly one file per permutation of the backend order, as the reference's paper-like protocol runs them).
Output: per configuration the mean, median, standard deviation and count of the chosen metric for every
backend, and the speed-up of each backend over a named base.

    python -m ooverlap_b200.bench.aggregate serving_*.jsonl --metric output_tok_s --group model,tp,batch \
        --by backend --base nccl

Capability parity: test/aggregate_vllm_backend_orders.py and its unit test
(test/test_aggregate_vllm_backend_orders.py:45+) in the reference.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
from collections import defaultdict
from typing import Iterable


def read_lines(paths: Iterable[str]) -> list:
    rows = []
    for path in paths:
        with open(path) as f:
            for line in f:
                line = line.strip()
                if line.startswith("{"):
                    rows.append(json.loads(line))
    return rows


def aggregate(rows: list, metric: str, group: list, by: str, base: str = "", higher_is_better: bool = True) -> list:
    cells = defaultdict(lambda: defaultdict(list))
    for r in rows:
        if metric not in r or by not in r:
            continue
        cells[tuple(r.get(g) for g in group)][r[by]].append(float(r[metric]))
    out = []
    for gkey in sorted(cells, key=lambda k: tuple(str(v) for v in k)):
        rec = {g: v for g, v in zip(group, gkey)}
        stats = {}
        for name, vals in sorted(cells[gkey].items()):
            stats[name] = {"mean": statistics.fmean(vals), "median": statistics.median(vals),
                           "stdev": statistics.stdev(vals) if len(vals) > 1 else 0.0, "n": len(vals)}
        rec["stats"] = stats
        if base and base in stats and stats[base]["median"] > 0:
            ref = stats[base]["median"]
            rec["speedup_vs_" + base] = {
                name: (s["median"] / ref if higher_is_better else ref / s["median"]) for name, s in stats.items() if s["median"] > 0}
        out.append(rec)
    return out


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("files", nargs="+")
    p.add_argument("--metric", default="output_tok_s")
    p.add_argument("--group", default="model,tp,batch")
    p.add_argument("--by", default="backend")
    p.add_argument("--base", default="nccl")
    p.add_argument("--lower-is-better", action="store_true")
    args = p.parse_args(argv)
    for rec in aggregate(read_lines(args.files), args.metric, args.group.split(","), args.by, args.base,
                         not args.lower_is_better):
        print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
