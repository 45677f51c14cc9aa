"""The eight figures of the reference's `figures/render/*.py`, drawn from this repository's result files as SVG.

  python -m dual_mod_public_b200.figures.render a5_heatmap      --data analysis --out a5_depth_heatmap.svg
  python -m dual_mod_public_b200.figures.render a5_position     --data analysis --out a5_T64_position_curves.svg
  python -m dual_mod_public_b200.figures.render lengthgen       --data analysis --out crasp_lengthgen.svg
  python -m dual_mod_public_b200.figures.render cvp_by_depth    --data analysis --out cvp_by_depth.svg
  python -m dual_mod_public_b200.figures.render cvp_minlayers   --data analysis --out cvp_minlayers.svg
  python -m dual_mod_public_b200.figures.render headline        --data analysis --out headline_right_keyed_cvp.svg
  python -m dual_mod_public_b200.figures.render fixedpoints     --data traces   --out loop_fixedpoints_3x3.svg
  python -m dual_mod_public_b200.figures.render tinystories     --data out      --out tinystories_ablation.svg

Inputs are what the trainers of this repository write: `statetrack_<tag>_<arch>.json` (formal-language harness:
`task`, `arch`, `n_ops`, `params`, `final` with the length factors and the `*_by_k` / `*_by_pos8` side-cars),
`metrics.jsonl` of the TinyStories runs (`tokens`, `val/loss`), and the rows printed by
`formal/loop_fixed_point.py` (`k change accuracy`) saved as `<row>_<col>_{in,ood}.txt`.  Where the reference's
scripts hard-code numbers read off its own runs (minimum depth per circuit size, deepest exact depth), the
functions here compute them from the result files.

Reference parity: figures/render/render_a5_heatmap.py, render_a5_position.py, render_crasp_lengthgen.py,
render_cvp_by_depth.py, render_cvp_minlayers.py, render_headline_right.py, render_loop_fixedpoints_3x3.py,
render_tinystories.py (matplotlib, PNG); same panels, axes and series, as SVG without a plotting library.
"""

from __future__ import annotations

import argparse
import glob
import json
import math
import os
import re

from .svg import Figure

ARCH_COLOR = {"dualmod": "#d62728", "dm": "#d62728", "vanilla": "#000000", "tpp": "#000000", "lstm": "#1f77b4",
              "gdn": "#2ca02c", "fbt": "#ff7f0e", "looped": "#9467bd", "rdepth": "#8c564b", "ematch": "#7f7f7f"}
SOLVED = 0.95


def load_runs(folder):
    runs = []
    for p in sorted(glob.glob(os.path.join(folder, "**", "statetrack_*.json"), recursive=True)):
        d = json.load(open(p))
        d["file"] = os.path.basename(p)
        runs.append(d)
    return runs


def _layers(run):
    m = re.search(r"_L(\d+)", run.get("task", "") + "_" + run.get("file", ""))
    return int(m.group(1)) if m else int(run.get("layers", 0) or 0)


def _sidecar(final, suffix):
    """The `*<suffix>` entry of a FINAL record as sorted (key, value) pairs; looped runs keep one per eval K
    (`K<k>_...`): the one with the deepest solved prefix is taken."""
    best = None
    for name, val in final.items():
        if not str(name).endswith(suffix) or not isinstance(val, (dict, list)):
            continue
        items = sorted(((float(k), float(v)) for k, v in val.items()), key=lambda kv: kv[0]) if isinstance(val, dict) \
            else [(float(i + 1), float(v)) for i, v in enumerate(val)]
        depth = 0
        for k, v in items:
            if v < SOLVED:
                break
            depth = k
        if best is None or depth > best[0]:
            best = (depth, items)
    return best[1] if best else []


def deepest_solved(items):
    d = 0
    for k, v in items:
        if v < SOLVED:
            break
        d = k
    return d


# ---- 1. A5 word problem: accuracy over depth x length, one panel per architecture --------------------------
def a5_heatmap(data, out, needle="a5"):
    cells = {}
    for r in load_runs(data):
        if needle in r["task"]:
            cells.setdefault((r["arch"], int(r["n_ops"]), _layers(r)), []).append(float(r["final"].get("1", 0.0)))
    archs = sorted({k[0] for k in cells})
    fig = Figure(80 + 380 * max(1, len(archs)), 330, "A5 word problem: accuracy over depth x length")
    for a_i, arch in enumerate(archs):
        Ts = sorted({k[1] for k in cells if k[0] == arch})
        Ls = sorted({k[2] for k in cells if k[0] == arch})
        M = [[(max(cells[(arch, T, L)]) if (arch, T, L) in cells else None) for L in Ls] for T in Ts]
        notes = [[(f"{sum(x >= SOLVED for x in cells[(arch, T, L)])}/{len(cells[(arch, T, L)])}"
                   if (arch, T, L) in cells and len(cells[(arch, T, L)]) > 1 else "") for L in Ls] for T in Ts]
        ax = fig.add(70 + 380 * a_i, 50, 300, 220, (0, len(Ls)), (0, len(Ts)), title=arch, xlabel="layers L",
                     ylabel="sequence length T")
        ax.heat(M, Ls, Ts, notes=notes)
        # frontier: the shallowest depth at which some seed solves each length
        pts = [(j + 0.5, i + 0.5) for i, T in enumerate(Ts)
               for j in [next((j for j, L in enumerate(Ls) if M[i][j] is not None and M[i][j] >= SOLVED), None)] if j is not None]
        if pts:
            ax.line([p[0] for p in pts], [p[1] for p in pts], color="#ff0000", width=2.2, marker="o")
    return fig.save(out)


# ---- 2. A5 accuracy by position (training range and extrapolation) -----------------------------------------
def a5_position(data, out, needle="a5", train_T=64):
    fig = Figure(1000, 330, "A5: accuracy by position (bin end = number of products composed)")
    ax = fig.add(60, 60, 900, 200, (0, 4 * train_T + 2), (-0.02, 1.08), xlabel="position", ylabel="accuracy")
    ax.span(0, train_T)
    ax.text(2, 1.03, f"training range (T={train_T})", size=9, color="#555", anchor="start")
    ax.hline(1 / 60, text="chance")
    for r in load_runs(data):
        if needle not in r["task"]:
            continue
        xs, ys = [], []
        for f in (1, 2, 4):                               # the length factors evaluated, 8 position bins each
            it = _sidecar({k: v for k, v in r["final"].items() if str(k).endswith(f"x{f}_by_pos8")}, "_by_pos8")
            n = int(r["n_ops"]) * f
            for i, (_, v) in enumerate(it):
                p = (i + 1) * n // 8
                if not xs or p > xs[-1]:
                    xs.append(p)
                    ys.append(v)
        if xs:
            ax.line(xs, ys, color=ARCH_COLOR.get(r["arch"], "#555"), marker="o",
                    label=f"{r['arch']}, {_layers(r) or '?'} layers, {r.get('params', 0) / 1e6:.0f}M")
    fig.legend(70, 290, cols=4)
    return fig.save(out)


# ---- 3. length generalisation of DFA state prediction, one panel per language ---------------------------------
def lengthgen(data, out, factors=(1, 2, 4, 6, 8, 10, 16, 20, 32)):
    runs = [r for r in load_runs(data) if r["task"].startswith("dfa") or "dfa" in r["task"]]
    langs = sorted({r["task"] for r in runs})
    cols = max(1, min(3, len(langs)))
    rows_n = max(1, math.ceil(len(langs) / cols))
    fig = Figure(60 + 330 * cols, 70 + 230 * rows_n, "DFA state prediction: accuracy at x times the training length")
    for i, lang in enumerate(langs):
        ax = fig.add(60 + 330 * (i % cols), 50 + 230 * (i // cols), 270, 150, (1, 32), (0.0, 1.05), xlog=True,
                     title=lang, xlabel="length factor", ylabel="accuracy")
        best = {}
        for r in runs:
            if r["task"] != lang:
                continue
            cur = {f: max([float(v) for k, v in r["final"].items()
                           if str(k) == str(f) or re.fullmatch(rf"K\d+_{f}", str(k))] or [float("nan")]) for f in factors}
            if r["arch"] not in best or cur.get(10, 0) > best[r["arch"]].get(10, 0):
                best[r["arch"]] = cur                      # best seed at 10x per arm
        for arch, cur in best.items():
            fs = [f for f in factors if not math.isnan(cur[f])]
            ax.line(fs, [cur[f] for f in fs], color=ARCH_COLOR.get(arch, "#555"), marker="o", label=arch)
    fig.legend(70, 60 + 230 * rows_n, cols=5, col_w=120)
    return fig.save(out)


# ---- 4. circuit value problem: accuracy by circuit depth ----------------------------------------------------------
def cvp_by_depth(data, out):
    fig = Figure(1000, 360, "CVP: accuracy by circuit depth, each arm at the largest circuit it was trained on")
    ax = fig.add(60, 50, 900, 220, (1, 1200), (0.4, 1.02), xlog=True, xlabel="circuit depth (gate index)",
                 ylabel="accuracy at that depth")
    ax.hline(SOLVED, text="exact (0.95)")
    ax.hline(0.5, text="chance")
    largest = {}
    for r in load_runs(data):
        if "cvp" in r["task"] and (r["arch"] not in largest or int(r["n_ops"]) > int(largest[r["arch"]]["n_ops"])):
            largest[r["arch"]] = r
    for arch, r in sorted(largest.items()):
        it = _sidecar(r["final"], "x1_by_k")
        if it:
            ax.line([k for k, _ in it], [v for _, v in it], color=ARCH_COLOR.get(arch, "#555"),
                    label=f"{arch}, {_layers(r) or '?'} layers, n={r['n_ops']}")
    fig.legend(70, 310, cols=4)
    return fig.save(out)


# ---- 5. CVP: minimum layers that solve a circuit size ---------------------------------------------------------------
def cvp_minlayers(data, out):
    solved, tried = {}, {}
    for r in load_runs(data):
        if "cvp" not in r["task"]:
            continue
        key, L = (r["arch"], int(r["n_ops"])), _layers(r) or 1
        tried[key] = max(tried.get(key, 0), L)
        if float(r["final"].get("1", 0.0)) >= SOLVED:
            solved[key] = min(solved.get(key, 1 << 30), L)
    fig = Figure(640, 380, "CVP: minimum depth vs circuit size")
    ax = fig.add(70, 50, 520, 250, (13, 1200), (0.8, 30), xlog=True, ylog=True, xlabel="circuit size n (gates)",
                 ylabel="min. layers to solve (acc >= 0.95)")
    for arch in sorted({k[0] for k in tried}):
        ns = sorted(n for a, n in tried if a == arch)
        ok = [(n, solved[(arch, n)]) for n in ns if (arch, n) in solved]
        if ok:
            ax.line([n for n, _ in ok], [L for _, L in ok], color=ARCH_COLOR.get(arch, "#555"), marker="o", label=arch)
        miss = [(n, tried[(arch, n)]) for n in ns if (arch, n) not in solved]      # open marker: not solved up to L
        if miss:
            ax.line([n for n, _ in miss], [L for _, L in miss], color=ARCH_COLOR.get(arch, "#555"), dash="2,3", marker="open")
    fig.legend(80, 345, cols=4, col_w=130)
    return fig.save(out)


# ---- 6. headline, right column: CVP deepest exact depth vs n over keyed A5 deepest solved depth vs registers --------
def headline(data, out):
    runs = load_runs(data)
    fig = Figure(560, 780)
    top = fig.add(70, 40, 440, 280, (12, 1400), (0.6, 1500), xlog=True, ylog=True, xlabel="circuit size n (gates)",
                  ylabel="deepest exact depth", title="Circuit value problem (P-complete)")
    top.line([8, 1200], [8, 1200], color="#999", width=0.8, dash="4,3")
    bot = fig.add(70, 400, 440, 250, (1.6, 1300), (0.5, 8.8), xlog=True, xlabel="interleaved registers K",
                  ylabel="deepest solved depth", title="Keyed A5: K registers, circuit depth 8")
    bot.hline(8, text="full circuit (depth 8)")
    series = {}
    for r in runs:
        if "cvp" in r["task"]:
            d = deepest_solved(_sidecar(r["final"], "x1_by_k"))
            series.setdefault(("cvp", r["arch"]), {})[int(r["n_ops"])] = max(d, series.get(("cvp", r["arch"]), {}).get(int(r["n_ops"]), 0))
        elif "keyed" in r["task"]:
            m = re.search(r"[_-]K(\d+)", r["task"])
            if m:
                d = deepest_solved(_sidecar(r["final"], "x1_by_k"))
                K = int(m.group(1))
                series.setdefault(("keyed", r["arch"]), {})[K] = max(d, series.get(("keyed", r["arch"]), {}).get(K, 0))
    for (kind, arch), pts in sorted(series.items()):
        xs = sorted(pts)
        (top if kind == "cvp" else bot).line(xs, [max(pts[x], 0.7) for x in xs], color=ARCH_COLOR.get(arch, "#555"),
                                             marker="o", label=arch)
    fig.legend(80, 700, cols=3, col_w=150)
    return fig.save(out)


# ---- 7. loop iterate dynamics, in- vs out-of-distribution (3 x 3) -----------------------------------------------------
def fixedpoints(data, out):
    def load(path):
        if not os.path.exists(path):
            return None
        rows = [l.split() for l in open(path) if l.strip() and l.strip()[0].isdigit()]
        return ([int(r[0]) for r in rows], [float(r[1]) if r[1] != "nan" else float("nan") for r in rows],
                [float(r[2]) for r in rows])
    rows = [("A5", "a5", 1 / 60), ("keyed A5", "keyed", 1 / 60), ("CVP", "cvp", 0.5)]
    cols = [("iteration-agnostic", "ag", "#7f7f7f"), ("K prop. to length", "kt", "#9467bd"), ("recurrent-depth", "hug", "#ff7f0e")]
    fig = Figure(1000, 760, "Loop iterate dynamics: solid = relative state change (log), dashed = accuracy; dark = in-distribution")
    for i, (rname, rk, chance) in enumerate(rows):
        for j, (cname, ck, color) in enumerate(cols):
            x0, y0 = 70 + 310 * j, 50 + 230 * i
            ax = fig.add(x0, y0, 250, 160, (0.9, 140), (2e-3, 1.5), xlog=True, ylog=True, title=cname if i == 0 else "",
                         xlabel="iteration k" if i == 2 else "", ylabel=f"{rname}: rel. state change" if j == 0 else "")
            acc = fig.add(x0, y0, 250, 160, (0.9, 140), (-0.03, 1.05), xlog=True)
            acc.xticks, acc.yticks = [], []
            acc.hline(chance)
            for tag, alpha in (("in", 1.0), ("ood", 0.45)):
                d = load(os.path.join(data, f"{rk}_{ck}_{tag}.txt"))
                if d is None:
                    continue
                k, ch, a = d
                ax.line(k[1:], ch[1:], color=color, alpha=alpha)
                acc.line(k, a, color=color, alpha=alpha, dash="5,3")
    return fig.save(out)


# ---- 8. TinyStories ablation: validation loss vs tokens --------------------------------------------------------------------
def tinystories(data, out):
    fig = Figure(760, 470, "TinyStories ablation: validation loss vs tokens")
    ax = fig.add(70, 40, 640, 320, (0, 305), (1.6, 3.3), xlabel="tokens (M)", ylabel="validation loss")
    palette = ["#000000", "#7f7f7f", "#1f77b4", "#2ca02c", "#d62728", "#9467bd", "#ff7f0e", "#8c564b", "#17becf"]
    for i, p in enumerate(sorted(glob.glob(os.path.join(data, "*", "metrics.jsonl")))):
        rows = [json.loads(l) for l in open(p) if l.strip()]
        pts = [(r["tokens"] / 1e6, r["val/loss"]) for r in rows if "val/loss" in r and "tokens" in r]
        if pts:
            name = os.path.basename(os.path.dirname(p))
            ax.line([a for a, _ in pts], [b for _, b in pts], color=palette[i % len(palette)], marker="o", width=1.8,
                    label=f"{name}  ({pts[-1][1]:.3f})")
    fig.legend(80, 410, cols=3)
    return fig.save(out)


FIGURES = {"a5_heatmap": a5_heatmap, "a5_position": a5_position, "lengthgen": lengthgen, "cvp_by_depth": cvp_by_depth,
           "cvp_minlayers": cvp_minlayers, "headline": headline, "fixedpoints": fixedpoints, "tinystories": tinystories}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("figure", choices=sorted(FIGURES) + ["all"])
    ap.add_argument("--data", required=True, help="folder with the result files of the runs")
    ap.add_argument("--out", default="", help="output .svg (for `all`: an output folder)")
    a = ap.parse_args(argv)
    if a.figure == "all":
        os.makedirs(a.out or "figures_out", exist_ok=True)
        return [f(a.data, os.path.join(a.out or "figures_out", f"{n}.svg")) for n, f in FIGURES.items()]
    return FIGURES[a.figure](a.data, a.out or f"{a.figure}.svg")


if __name__ == "__main__":
    print(main())
