"""Post-hoc analysis of a formal-language checkpoint (`{"model", "args"}` written by `--eval_dump`).

  python -m dual_mod_public_b200.formal.analysis reeval run.pt [--factor 2] [--rows 128]
      rebuild the model from the saved options, draw a fresh evaluation batch and score it eagerly (no
      engine): accuracy overall, by difficulty (depth / register / hop side-car) and by position octile
  python -m dual_mod_public_b200.formal.analysis composition run.pt [--factor 1]
      group word problems only: HOW wrong the wrong answers are.  Per position octile: top-1/5/10 accuracy
      and the mean / median rank of the gold state (a graded decay shows a rank that drifts up, a wall shows
      a rank near n/2); and for wrong arg-max answers the correction c = predicted^-1 * gold: its word length
      under a small generating set (P(len <= 2): the model dropped few factors), its entropy relative to
      uniform and the mass of its five commonest values (concentrated = systematic slip, uniform = state lost)

Reference parity: formal_language/harness/eval_cvp_ckpt.py (eager re-evaluation of an engine-trained
checkpoint), formal_language/harness/statetrack_composition_analysis.py (rank and correction statistics).
"""

from __future__ import annotations

import argparse
import json
from types import SimpleNamespace

import numpy as np
import torch

from . import harness as H
from . import tasks as T
from .tasks import step_rng


def load_run(path, device="cpu"):
    """(model, kind, args namespace, mul, n_elem) of a harness checkpoint."""
    ck = torch.load(path, map_location="cpu", weights_only=False)
    a = dict(H.DEFAULTS)
    a.update(ck["args"])
    args = SimpleNamespace(**a)
    if args.task == "cvp":
        T.CVP_GATE[0] = a.get("cvp_gate", "xormaj")
    mul, n_elem = H.task_tables(args)
    sd = ck["model"]
    vocab = sd["tok_emb.weight"].shape[0] if "tok_emb.weight" in sd else H.vocab_of(args, n_elem)
    max_len = max(512, int(a.get("n_ops", 64)) * 8 + 64)
    model, kind = H.build_model(a.get("arch", "dualmod"), vocab, max_len, scale=a.get("scale", "5m"),
                                deq_sweeps=a.get("deq_sweeps", 4), ctx_mod=a.get("ctx_mod", "linear"),
                                n_layers=a.get("n_layers", 0), nope=a.get("nope", False),
                                loop_layers=a.get("loop_layers", 2), loop_k=a.get("loop_k", 64),
                                key_mod=not a.get("no_key_mod", False), logn_ref=a.get("logn_ref", 0),
                                fbt_sched=a.get("fbt_sched", ""), loop_emb_scale=a.get("loop_emb_scale", False),
                                loop_huginn=a.get("loop_huginn", False), loop_bp=a.get("loop_bp", 0))
    missing, unexpected = model.load_state_dict(sd, strict=False)
    return model.to(device).eval(), kind, args, mul, n_elem, (len(missing), len(unexpected))


def fresh_batch(args, mul, n_elem, rows, factor, seed=7):
    return H.make_batch(args, mul, n_elem, step_rng(H.TASK_ID[args.task], seed, 0, 1000 + factor), rows,
                        args.n_ops * factor, evaluating=True)


def reeval(path, factor=1, rows=128, device="cpu", loop_k=None):
    model, kind, args, mul, n_elem, mism = load_run(path, device)
    x, tg, m, d = fresh_batch(args, mul, n_elem, rows, factor)
    evals = {factor: (x.to(device), None if tg is None else tg.to(device), m.to(device), d)}
    amp = torch.autocast(torch.device(device).type, dtype=torch.bfloat16, enabled=torch.device(device).type == "cuda")
    with torch.no_grad(), amp:
        res = H.evaluate(lambda xb: H.logits_of(kind, model, xb, K=loop_k or getattr(args, "loop_k", None)), evals)
    res["state_dict_mismatch"] = {"missing": mism[0], "unexpected": mism[1]}
    return res


# ---- composition analysis ----------------------------------------------------------------------------------
def inverse_table(mul):
    n = mul.shape[0]
    return np.array([int(np.where(mul[g] == 0)[0][0]) for g in range(n)])       # g * g^-1 = identity (index 0)


def word_lengths(mul, gens):
    """Breadth-first distance from the identity in the Cayley graph of `gens` (right multiplication)."""
    n = mul.shape[0]
    dist = np.full(n, -1, dtype=np.int64)
    dist[0], frontier, d = 0, [0], 0
    while frontier:
        d += 1
        nxt = []
        for s in frontier:
            for g in gens:
                v = int(mul[s, g])
                if dist[v] < 0:
                    dist[v] = d
                    nxt.append(v)
        frontier = nxt
    return dist


def small_generators(mul):
    """The first elements (and their inverses) that together generate the group."""
    n, inv = mul.shape[0], inverse_table(mul)
    gens = []
    for g in range(1, n):
        if (word_lengths(mul, gens) >= 0).all():
            break
        if word_lengths(mul, gens)[g] < 0:
            gens += [g] + ([int(inv[g])] if inv[g] != g else [])
    return gens


def composition_stats(state_logits, gold, pos, width, mul):
    """state_logits [N, n] over the group's states, gold [N] state index, pos [N] position in a row of
    `width` tokens.  Returns {"octiles": [...], "all": {...}} of the statistics in the module docstring."""
    n, inv = mul.shape[0], inverse_table(mul)
    wl = word_lengths(mul, small_generators(mul))
    order = np.argsort(-state_logits, axis=1)
    rank = np.argmax(order == gold[:, None], axis=1)                            # 0 = correct
    pred = order[:, 0]

    def summarise(sel):
        r = rank[sel]
        out = {"n": int(sel.sum())}
        if not out["n"]:
            return out
        out.update(top1=float((r < 1).mean()), top5=float((r < 5).mean()), top10=float((r < 10).mean()),
                   mean_rank=float(r.mean()), median_rank=float(np.median(r)))
        wrong = sel & (rank > 0)
        if wrong.any():
            c = mul[inv[pred[wrong]], gold[wrong]]                               # predicted^-1 * gold
            hist = np.bincount(c, minlength=n).astype(np.float64)
            p = hist / hist.sum()
            nz = p[p > 0]
            out.update(wrong=int(wrong.sum()), p_wordlen_le2=float((wl[c] <= 2).mean()),
                       entropy_ratio=float(-(nz * np.log(nz)).sum() / np.log(n)),
                       top5_mass=float(np.sort(p)[-5:].sum()))
        return out

    octile = np.minimum(7, pos * 8 // max(1, width))
    return {"all": summarise(np.ones(len(gold), dtype=bool)),
            "octiles": [summarise(octile == o) for o in range(8)], "n_states": int(n),
            "uniform_p_wordlen_le2": float((wl <= 2).mean())}


def composition(path, factor=1, rows=128, device="cpu"):
    model, kind, args, mul, n_elem, _ = load_run(path, device)
    assert args.task == "group", "the composition analysis reads group word problems"
    x, tg, m, _ = fresh_batch(args, mul, n_elem, rows, factor)
    with torch.no_grad():
        logits = H.logits_of(kind, model, x.to(device), K=getattr(args, "loop_k", None)).float().cpu()
    b, p = m.nonzero(as_tuple=True)
    base = T.BASE + n_elem                                                        # state tokens follow the op tokens
    if tg is not None:
        lg, gold = logits[b, p, base:base + n_elem], tg[b, p] - base
    else:                                                                         # next-token convention
        lg, gold = logits[b, p - 1, base:base + n_elem], x[b, p] - base
    return composition_stats(lg.numpy(), gold.numpy(), p.numpy(), x.shape[1], np.asarray(mul))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("mode", choices=["reeval", "composition"])
    ap.add_argument("ckpt")
    ap.add_argument("--factor", type=int, default=1)
    ap.add_argument("--rows", type=int, default=128)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    args = ap.parse_args(argv)
    fn = reeval if args.mode == "reeval" else composition
    out = fn(args.ckpt, factor=args.factor, rows=args.rows, device=args.device)
    print(json.dumps(out, indent=1, default=str))
    return out


if __name__ == "__main__":
    main()
