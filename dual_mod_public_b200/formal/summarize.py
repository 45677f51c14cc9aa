"""Tables from the result files of the formal-language runs (`analysis/statetrack_<tag>_<arch>.json`).

  python -m dual_mod_public_b200.formal.summarize analysis                    # one line per run
  python -m dual_mod_public_b200.formal.summarize analysis --grid a5          # accuracy over length x layers per arch,
                                                                              # and the shallowest depth that solves each length
  python -m dual_mod_public_b200.formal.summarize analysis --by k             # accuracy by difficulty side-car (depth, register, hop)

The reference draws these as figures (figures/render/*.py: depth x length heat map with the minimum-depth
frontier, accuracy by circuit depth, length-generalisation curves); here they are text tables computed from the
same FINAL records, so they can be read on a machine without a plotting stack.
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import re


def load(folder):
    runs = []
    for p in sorted(glob.glob(os.path.join(folder, "statetrack_*.json"))):
        d = json.load(open(p))
        d["file"] = os.path.basename(p)
        runs.append(d)
    return runs


def factors_line(run):
    fin = run["final"]
    return "  ".join(f"x{f}={fin[str(f)]:.3f}" for f in run.get("factors", [1]) if str(f) in fin)


def listing(runs):
    lines = [f"{'run':58s} {'arch':9s} {'params':>8s}  accuracy by length factor"]
    for r in runs:
        lines.append(f"{r['task'][:58]:58s} {r['arch']:9s} {r['params'] / 1e6:7.1f}M  {factors_line(r)}")
    return lines


def depth_grid(runs, needle, solved=0.95):
    """Best in-distribution accuracy per (arch, n_ops, layers) over seeds, plus `solved/seeds`, for runs whose tag
    contains `needle`; then per arch and length the shallowest depth at which any seed reaches `solved`."""
    cells = {}
    for r in runs:
        if needle not in r["task"]:
            continue
        m = re.search(r"_L(\d+)", r["task"] + "_" + r.get("file", ""))
        layers = int(m.group(1)) if m else int(r.get("layers", 0))
        cells.setdefault((r["arch"], r["n_ops"], layers), []).append(float(r["final"].get("1", 0.0)))
    lines = []
    for arch in sorted({k[0] for k in cells}):
        Ts = sorted({k[1] for k in cells if k[0] == arch})
        Ls = sorted({k[2] for k in cells if k[0] == arch})
        lines.append(f"{arch}: rows = length, columns = layers {Ls} (best accuracy, solved/seeds)")
        for T in Ts:
            row = []
            for L in Ls:
                v = cells.get((arch, T, L))
                row.append(f"{max(v):.2f} {sum(x >= solved for x in v)}/{len(v)}" if v else "   -    ")
            lines.append(f"  T={T:<5d} " + " | ".join(row))
        frontier = {T: next((L for L in Ls if cells.get((arch, T, L)) and max(cells[(arch, T, L)]) >= solved), None)
                    for T in Ts}
        lines.append(f"  shallowest solving depth: {frontier}")
    return lines


def by_sidecar(runs, key="k"):
    lines = []
    for r in runs:
        for name, val in r["final"].items():
            if name.endswith(f"_by_{key}") and isinstance(val, (dict, list)):
                items = sorted(val.items(), key=lambda kv: float(kv[0])) if isinstance(val, dict) else enumerate(val)
                cells = "  ".join(f"{k}:{v:.2f}" for k, v in items)
                lines.append(f"{r['task'][:48]:48s} {r['arch']:9s} {name:10s} {cells}")
    return lines


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("folder")
    ap.add_argument("--grid", default="", help="substring of the run tags to tabulate over length x layers")
    ap.add_argument("--by", default="", help="side-car to break accuracy down by (k or pos8)")
    ap.add_argument("--solved", type=float, default=0.95)
    a = ap.parse_args(argv)
    runs = load(a.folder)
    lines = depth_grid(runs, a.grid, a.solved) if a.grid else by_sidecar(runs, a.by) if a.by else listing(runs)
    print("\n".join(lines))
    return lines


if __name__ == "__main__":
    main()
