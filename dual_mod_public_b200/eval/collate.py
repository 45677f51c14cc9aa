"""Pool sharded evaluation outputs and tabulate the result files of a run.

  python -m dual_mod_public_b200.eval.collate pool analysis/lmeval_run_100_ab12cd_s*of4_jrt_fda_TEXT.jsonl
  python -m dual_mod_public_b200.eval.collate table analysis run [--targets targets.json]

`pool`: per-file and pooled "contains" over the generation dumps of a sharded recall task (shards differ
in size by at most one document, but pooling counts documents, not shard means).  `table`: reads every
`lmeval_<run>_*.json` in the folder, groups the results by the engine K they were scored at (none = exact
operator), and prints the language-modelling / common-sense table (accuracies x 100, the average over the
nine accuracy columns when all are present), the recall tasks and the needle tasks; `--targets` adds rows
of published numbers to compare with ({"row name": {"column": value}}).

Reference parity: lm/eval/merge_shards.py, lm/eval/gdn2_collate.py.
"""

from __future__ import annotations

import glob
import json
import os
import sys

COLUMNS = [("Wiki ppl", "wikitext", "word_perplexity"), ("LMB ppl", "lambada_openai", "perplexity"),
           ("LMB acc", "lambada_openai", "acc"), ("PIQA", "piqa", "acc"), ("Hella(n)", "hellaswag", "acc_norm"),
           ("Wino", "winogrande", "acc"), ("ARC-e", "arc_easy", "acc"), ("ARC-c", "arc_challenge", "acc"),
           ("OBQA", "openbookqa", "acc"), ("SIQA", "social_iqa_pq", "acc"), ("BoolQ", "boolq", "acc")]
RECALL_ROWS = ["jrt_swde", "jrt_squad", "jrt_fda", "jrt_triviaqa", "jrt_nq", "jrt_drop"]


def pool(paths):
    hits = n = 0
    lines = []
    for p in paths:
        rows = [json.loads(l) for l in open(p) if l.strip()]
        h = sum(r["metric"].get("contains", 0) >= 0.5 for r in rows)
        lines.append(f"{p}: {h}/{len(rows)} = {100 * h / max(1, len(rows)):.2f}")
        hits, n = hits + h, n + len(rows)
    lines.append(f"POOLED contains = {100 * hits / max(1, n):.2f}  ({hits}/{n})")
    return hits, n, lines


def metric(res, task, name):
    r = res.get(task, {})
    for key in (name, f"{name},none"):
        if key in r:
            return float(r[key])
    return None


def table(folder, run, targets=None):
    files = sorted(glob.glob(os.path.join(folder, f"lmeval_{run}_*.json")), key=os.path.getmtime)
    by_k = {}
    for f in files:
        d = json.load(open(f))
        if "results" in d:
            by_k.setdefault(d.get("engine_K"), {}).update(d["results"])
    lines = [f"== {run}: {len(files)} result files",
             " | ".join(f"{h:>9s}" for h in ["model"] + [c for c, _, _ in COLUMNS] + ["Avg"])]
    for k, res in sorted(by_k.items(), key=lambda kv: (kv[0] is None, kv[0] or 0)):
        if not any(t in res for _, t, _ in COLUMNS):
            continue
        cells, accs = [], []
        for col, task, name in COLUMNS:
            v = metric(res, task, name)
            if v is None:
                cells.append(f"{'-':>9s}")
                continue
            if "ppl" not in col:
                v *= 100
                accs.append(v)
            cells.append(f"{v:9.2f}")
        avg = sum(accs) / 9 if len(accs) == 9 else float("nan")
        lines.append(" | ".join([f"{('K' + str(k)) if k else 'exact':>9s}"] + cells + [f"{avg:9.2f}"]))
    for name, row in (targets or {}).items():
        lines.append(" | ".join([f"{name[:9]:>9s}"] + [f"{row[c]:9.2f}" if c in row else f"{'-':>9s}"
                                                         for c in [c for c, _, _ in COLUMNS] + ["Avg"]]))
    merged = {}
    for k in sorted(by_k, key=lambda kk: (kk is not None, kk or 0)):      # exact first, engine results override
        merged.update(by_k[k])
    nums = lambda r: "  ".join(f"{a}={float(b):.4f}" for a, b in r.items()
                               if isinstance(b, (int, float)) and "stderr" not in a)
    lines.append("recall")
    lines += [f"  {t:14s} {nums(merged[t])}" for t in RECALL_ROWS if t in merged]
    lines.append("needles")
    lines += [f"  {t:28s} {nums(r)}" for t, r in sorted(merged.items()) if t.startswith("niah") or "niah" in t]
    return lines


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] not in ("pool", "table"):
        print(__doc__)
        return 2
    if argv[0] == "pool":
        print("\n".join(pool(argv[1:])[2]))
    else:
        targets = None
        if "--targets" in argv:
            i = argv.index("--targets")
            targets = json.load(open(argv[i + 1]))
            del argv[i:i + 2]
        print("\n".join(table(argv[1], argv[2], targets)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
