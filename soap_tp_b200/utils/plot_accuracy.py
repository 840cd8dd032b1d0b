#!/usr/bin/env python3
"""Summarise (and, when matplotlib is installed, plot) accuracy-sweep logs.

Consumes the per-step accuracy lines printed by the accuracy sweep and by the trajectory tests,

    "{rows}x{cols} dim{d} basis={impl} | step {k} | SOAP relL2={e} ... | PARAM relL2={e}"

(the format of the reference's ``tests/unit/test_soap.py:775-790``, parsed there by
``scripts/plot_soap_accuracy.py:14-22``).  For every (size, shard dimension, basis) it reports the
maximum, the step-1 and the final update error; ``--png`` writes a log-log figure with the headless
Agg backend, ``--csv`` a table.
"""
from __future__ import annotations

import argparse
import csv
import re
import sys
from collections import defaultdict
from typing import Dict, List, Tuple

LINE = re.compile(
    r"(?P<rows>\d+)x(?P<cols>\d+)\s+dim(?P<dim>[01])\s+basis=(?P<basis>\w+)\s*\|\s*step\s+(?P<step>\d+)\s*\|\s*"
    r"SOAP relL2=(?P<update>[0-9.eE+-]+).*?\|\s*PARAM relL2=(?P<param>[0-9.eE+-]+)")


def parse(lines) -> Dict[Tuple[int, int, int, str], List[Tuple[int, float, float]]]:
    series: Dict[Tuple[int, int, int, str], List[Tuple[int, float, float]]] = defaultdict(list)
    for line in lines:
        match = LINE.search(line)
        if match:
            key = (int(match["rows"]), int(match["cols"]), int(match["dim"]), match["basis"])
            series[key].append((int(match["step"]), float(match["update"]), float(match["param"])))
    return series


def summarise(series):
    rows = []
    for (r, c, dim, basis), points in sorted(series.items()):
        points.sort()
        updates = [u for _, u, _ in points]
        rows.append(dict(rows=r, cols=c, shard_dim=dim, basis=basis, steps=len(points), max_update_error=max(updates),
                         first_update_error=updates[0], final_update_error=updates[-1],
                         final_parameter_error=points[-1][2]))
    return rows


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("logs", nargs="+")
    parser.add_argument("--png", default=None)
    parser.add_argument("--csv", default=None)
    args = parser.parse_args(argv)
    lines: List[str] = []
    for path in args.logs:
        with (sys.stdin if path == "-" else open(path)) as stream:
            lines.extend(stream)
    table = summarise(parse(lines))
    if not table:
        print("no accuracy lines found", file=sys.stderr)
        return 1
    header = list(table[0])
    print(" ".join(f"{h:>22s}" for h in header))
    for row in table:
        print(" ".join(f"{row[h]:>22.3e}" if isinstance(row[h], float) else f"{str(row[h]):>22s}" for h in header))
    if args.csv:
        with open(args.csv, "w", newline="") as stream:
            writer = csv.DictWriter(stream, fieldnames=header)
            writer.writeheader()
            writer.writerows(table)
    if args.png:
        try:
            import matplotlib

            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
        except ImportError:
            print("matplotlib is not installed; skipping the figure", file=sys.stderr)
            return 0
        figure, axis = plt.subplots(figsize=(7, 4.5))
        for label, key in (("max", "max_update_error"), ("step 1", "first_update_error"), ("final", "final_update_error")):
            for basis in sorted({row["basis"] for row in table}):
                points = sorted((max(row["rows"], row["cols"]), row[key]) for row in table if row["basis"] == basis)
                axis.loglog([p[0] for p in points], [p[1] for p in points], marker="o", label=f"{label} ({basis})")
        axis.set_xlabel("matrix size")
        axis.set_ylabel("relative L2 error of the update")
        axis.grid(True, which="both", alpha=0.3)
        axis.legend(fontsize=7)
        figure.tight_layout()
        figure.savefig(args.png, dpi=150)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
