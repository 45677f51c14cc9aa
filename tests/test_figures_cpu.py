"""The eight figure renderers on small synthetic result files: every figure is written as well-formed SVG with
its series in it."""

import json
import os
import xml.etree.ElementTree as ET

from dual_mod_public_b200.figures import render as R


def _run(folder, tag, arch, n_ops, final, params=12e6):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, f"statetrack_{tag}_{arch}.json"), "w") as f:
        json.dump({"task": tag, "arch": arch, "n_ops": n_ops, "params": params, "final": final, "factors": [1, 2, 4]}, f)


def _svg(path):
    root = ET.parse(path).getroot()
    assert root.tag.endswith("svg")
    return open(path).read()


def test_all_figures_render(tmp_path):
    a = str(tmp_path / "analysis")
    for arch, accs in (("dualmod", {1: 0.99, 2: 1.0}), ("vanilla", {1: 0.3, 2: 0.6, 4: 0.97})):
        for L, acc in accs.items():
            for T in (5, 10):
                by_pos = {f"x{f}_by_pos8": [max(0.0, acc - 0.05 * i * (f - 1)) for i in range(8)] for f in (1, 2, 4)}
                _run(a, f"group_a5T{T}_L{L}_s1", arch, T, {"1": acc - 0.01 * T, "2": acc / 2, "4": acc / 4, **by_pos})
    for arch in ("dualmod", "lstm"):
        for n in (16, 32):
            solved = n if arch == "dualmod" else 10
            _run(a, f"cvp_n{n}_L1", arch, n, {"1": 0.99 if arch == "dualmod" else 0.7,
                                             "x1_by_k": {str(k): (1.0 if k <= solved else 0.6) for k in range(1, n + 1)}})
        for K in (2, 8):
            _run(a, f"keyed_a5-K{K}_L1", arch, 64, {"1": 0.9, "x1_by_k": {str(k): (1.0 if k <= (8 if arch == "dualmod" else 2) else 0.1)
                                                                          for k in range(1, 9)}})
        _run(a, "dfa_z2", arch, 50, {str(f): (1.0 if arch == "dualmod" else 1.0 / f) for f in (1, 2, 4, 6, 8, 10, 16, 20, 32)})
    tr = tmp_path / "traces"
    tr.mkdir()
    for rk in ("a5", "keyed", "cvp"):
        for ck in ("ag", "kt", "hug"):
            for tag in ("in", "ood"):
                with open(tr / f"{rk}_{ck}_{tag}.txt", "w") as f:
                    for k in range(1, 33):
                        f.write(f"{k} {'nan' if k == 1 else 1.0 / k:} {min(1.0, k / 16):.3f}\n")
    ts = tmp_path / "out"
    for name, last in (("A-vanilla", 1.74), ("B-dm", 1.68)):
        (ts / name).mkdir(parents=True)
        with open(ts / name / "metrics.jsonl", "w") as f:
            for i in range(1, 11):
                f.write(json.dumps({"tokens": i * 30e6, "val/loss": last + 1.5 / i}) + "\n")
    out = tmp_path / "figs"
    out.mkdir()
    data_of = {"fixedpoints": str(tr), "tinystories": str(ts)}
    for name, fn in R.FIGURES.items():
        path = fn(data_of.get(name, a), str(out / f"{name}.svg"))
        text = _svg(path)
        assert "polyline" in text or "rect" in text, name
    heat = open(out / "a5_heatmap.svg").read()
    assert "dualmod" in heat and "vanilla" in heat and "0.9" in heat
    assert "B-dm  (1.830)" in open(out / "tinystories.svg").read()
    assert R.main(["cvp_minlayers", "--data", a, "--out", str(out / "again.svg")]).endswith("again.svg")
    # deepest exact depth of the synthetic CVP runs: the Dual-Mod arm solves every depth, the LSTM arm ten gates
    assert R.deepest_solved(R._sidecar(json.load(open(os.path.join(a, "statetrack_cvp_n32_L1_lstm.json")))["final"], "x1_by_k")) == 10
