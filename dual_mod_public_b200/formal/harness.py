"""Shared pieces of the formal-language trainers: task -> batch dispatch, vocab sizes,
model construction per architecture and scale, the two loss conventions and the
stratified evaluation.

Loss conventions: a tagged batch (tgt given) is scored AT the masked position,
CE(logits[pos], tgt[pos]); an interleaved batch (tgt None) is scored next-token,
CE(logits[pos-1], tok[pos]).  Evaluation reports accuracy per length factor plus
accuracy by difficulty (k / depth side-car) and by position octile.

Reference parity: formal_language/harness/train_statetrack.py (TASK_ID 39-41,
make_batch 50-142, vocab_of 145-168, SCALES 171-183, build_model 189-225,
logits_of 231-236, evaluation 604-647).
"""

from __future__ import annotations

import math
from types import SimpleNamespace

import numpy as np
import torch
import torch.nn.functional as F

from ..config import DualModConfig
from ..models import DualModLM
from ..models.baselines import FBTLM, LSTMLM, LoopedLM, RecurrentDepthLM, build_gdn
from . import tasks as T

TASK_ID = {"group": 11, "khop": 12, "parity": 13, "match3": 14, "niah": 15, "mix": 16,
           "keyed": 17, "ca": 18, "matinv": 19, "dfa": 20, "cvp": 21}

SCALES = {"5m": dict(d=256, L=4, h=4), "63m": dict(d=768, L=9, h=12),
          "w1024": dict(d=1024, L=9, h=16), "w1280": dict(d=1280, L=9, h=20),
          "w1536": dict(d=1536, L=9, h=24), "w2048": dict(d=2048, L=9, h=32),
          "w3072": dict(d=3072, L=9, h=48), "w4096": dict(d=4096, L=9, h=64)}

DEFAULTS = dict(task="group", group="a5", format="tagged", n_ops=64, max_ops=256, K=4, K_max=0, D=8,
                rho=0.0, queries=8, k_max=8, sorted_pairs=False, ablate_pairs=False, v_len=4,
                m3_mod=151, m3_win=16, ca_rule=110, ca_w=16, ca_format="silent", ca_think=False,
                ca_gap=1, dfa="z2", dfa_sep=False, mi_p=2, mi_out="inv", mi_think=False,
                cvp_inputs=32, cvp_format="tagged", cvp_pad=0, cvp_chain=1.0, cvp_queries=4,
                cvp_window=0, cvp_leak_every=0, cvp_addr="abs", key_shuffle=False)


def task_args(**kw):
    """Namespace of task options with the harness defaults filled in."""
    d = dict(DEFAULTS)
    d.update(kw)
    return SimpleNamespace(**d)


def task_tables(args):
    """(mul, n_elem) for the group-like tasks; for `mix` a pair of each; prepares `args._dfa`."""
    if args.task == "mix":
        (ma, na), (mb, nb) = T.cayley("z10"), T.cayley("a5")
        return (ma, mb), (na, nb)
    if args.task == "dfa":
        args._dfa = T.dfa_lib(args.dfa)
        return None, args._dfa[1]
    if args.task in ("group", "keyed"):
        return T.cayley(args.group)
    return None, 0


def cvp_full_len(args, n_ops):
    leak = n_ops // args.cvp_leak_every if args.cvp_leak_every else 0
    return (1 + 2 * args.cvp_inputs + T.CVP_TOK_PER_GATE * n_ops
            + (args.cvp_pad if args.cvp_format == "silent" else 0) + 2 * min(args.cvp_queries, n_ops) + leak)


def vocab_of(args, n_elem):
    t = args.task
    if t == "keyed":
        return T.BASE + (args.K_max or args.K) + 2 * n_elem
    if t == "group":
        return T.BASE + 2 * n_elem
    if t == "khop":
        return T.BASE + args.k_max + args.max_ops
    if t == "parity":
        return 12
    if t == "cvp":
        return T.cvp_vocab(args.max_ops, args.cvp_inputs)
    if t == "ca":
        return T.BASE + 4 + args.max_ops + 1
    if t == "dfa":
        return T.BASE + args._dfa[2] + args._dfa[1]
    if t == "matinv":
        return T.mi_vocab(args.mi_p, args.max_ops)
    if t == "niah":
        return T.BASE + 512 + 64
    if t == "mix":
        return T.BASE + 2 * 10 + 2 * 60
    return T.BASE + args.m3_mod + 2


def make_batch(args, mul, n_elem, rng, B, n_ops, eval_fixed_k=None, D_override=None, evaluating=False):
    """(tok, tgt or None, msk, diff or None) as torch / numpy.  `n_ops` is the task's size
    axis (ops, symbols, CA depth, matrix size, gates).  `D_override`: train-time depth
    (keyed) or ramp fraction (cvp) of a curriculum."""
    t = args.task
    tt = lambda a: None if a is None else torch.from_numpy(a)
    tgt = diff = None
    if t == "keyed":
        km = args.K_max or args.K
        tok, tgt, msk, diff = T.make_keyed_group_batch(rng, B, mul, n_elem, getattr(args, "_K_t", None) or args.K,
                                                       D_override or args.D, args.rho, K_max=km)
        if args.key_shuffle and not evaluating:
            perm = rng.permutation(km)
            is_key = (tok >= T.BASE) & (tok < T.BASE + km)
            tok = np.where(is_key, T.BASE + perm[np.clip(tok - T.BASE, 0, km - 1)], tok)
    elif t == "mix":
        tok, tgt, msk, _ = T.make_mixed_tagged_batch(rng, B, n_ops, mul[0], n_elem[0], mul[1], n_elem[1],
                                                     force=eval_fixed_k)
    elif t == "group" and args.format == "tagged":
        tok, tgt, msk = T.make_group_tagged_batch(rng, B, n_ops, mul, n_elem, op_pool=getattr(args, "_op_pool", None))
    elif t == "group" and args.format == "final":
        if eval_fixed_k is not None:
            k = eval_fixed_k
            width = 1 + max(1, (args.n_ops * 2) // (k + 2)) * (k + 2)
            tok, msk, diff = T.make_group_final_batch(rng, B, width, mul, n_elem, k_max=k, k_min=k)
        else:
            tok, msk, diff = T.make_group_final_batch(rng, B, 1 + 2 * n_ops, mul, n_elem, k_max=args.n_ops)
    elif t == "group":
        tok, msk = T.make_group_batch(rng, B, n_ops, mul, n_elem)
    elif t == "khop":
        tok, msk, diff = T.make_khop_batch(rng, B, n_ops, args.queries, args.k_max,
                                           sorted_pairs=args.sorted_pairs, ablate_pairs=args.ablate_pairs)
    elif t == "ca":
        tok, tgt, msk = T.make_ca_batch(rng, B, args.ca_w, n_ops, args.ca_rule, args.ca_format,
                                        pad=n_ops if args.ca_think else 0, gap=args.ca_gap)
    elif t == "dfa":
        trans, n_st, n_sym, _ = args._dfa
        tok, tgt, msk = T.make_dfa_batch(rng, B, n_ops, trans, n_st, n_sym, sep=args.dfa_sep)
    elif t == "matinv":
        tok, tgt, msk = T.make_matinv_batch(rng, B, n_ops, args.mi_p, args.mi_out,
                                            pad=n_ops * n_ops if args.mi_think else 0)
    elif t == "cvp":
        frac = D_override if (D_override is not None and not evaluating) else 1.0
        m_t = max(4, int(round(4 + frac * (args.cvp_inputs - 4)))) if frac < 1.0 else args.cvp_inputs
        n_t = max(4, int(round(4 + frac * (n_ops - 4)))) if frac < 1.0 else n_ops
        tok, tgt, msk, diff = T.make_cvp_batch(rng, B, n_t, m=m_t, fmt=args.cvp_format, pad=args.cvp_pad,
                                               chain=args.cvp_chain, n_queries=args.cvp_queries, n_max=args.max_ops,
                                               m_max=args.cvp_inputs, n_topo=16 if evaluating else 1,
                                               window=args.cvp_window, leak_every=args.cvp_leak_every, addr=args.cvp_addr)
        full = cvp_full_len(args, n_ops)
        if tok.shape[1] < full:                       # curriculum batches are padded (masked) to the full length
            w = ((0, 0), (0, full - tok.shape[1]))
            tok, tgt, msk, diff = (np.pad(a, w) for a in (tok, tgt, msk, diff))
    elif t == "parity":
        tok, msk = T.make_parity_batch(rng, B, n_ops)
    elif t == "niah":
        tok, msk, diff = T.make_niah_batch(rng, B, n_ops, args.v_len, args.queries,
                                           pairs_min=2 if eval_fixed_k is None else None)
    else:
        tok, msk = T.make_match3_batch(rng, B, n_ops, M=args.m3_mod, W=args.m3_win)
    return tt(tok), tt(tgt), tt(msk), diff


# ---- models -------------------------------------------------------------------------------------
def build_model(arch, vocab, max_seq_len, scale="5m", deq_sweeps=4, ctx_mod="linear", n_layers=0, nope=False,
                loop_layers=2, loop_k=64, key_mod=True, logn_ref=0, fbt_sched="", loop_emb_scale=False,
                loop_huginn=False, loop_bp=0, **cfg_overrides):
    """(model, kind).  kind selects how logits are obtained: "dualmod" (model(x)[0]),
    "looped" / "fbtp" (model(x, K=...)[0]) or "fla" (HF-style output)."""
    s = dict(SCALES[scale])
    if n_layers:
        s["L"] = n_layers
    base = dict(d_model=s["d"], n_heads=s["h"], max_seq_len=max_seq_len, vocab_size=vocab, gate_bias_init=0.0,
                checkpoint_chunk=0, use_rope=not nope)
    if arch == "lstm":
        return LSTMLM(vocab, s["d"], n_layers or max(2, s["L"] // 2)), "dualmod"
    if arch == "looped":
        cfg = DualModConfig(attn_mode="vanilla", n_layers=1, **base)
        if loop_huginn:
            return RecurrentDepthLM(cfg, n_unique=loop_layers, k_max=loop_k, bp_iters=loop_bp,
                                    emb_scale=loop_emb_scale), "looped"
        return LoopedLM(cfg, n_unique=loop_layers, k_max=loop_k), "looped"
    if arch == "fbt":
        return FBTLM(DualModConfig(attn_mode="vanilla", n_layers=s["L"], **base)), ("fbtp" if fbt_sched else "dualmod")
    if arch in ("dualmod", "vanilla"):
        cfg = DualModConfig(attn_mode="vanilla" if arch == "vanilla" else "sequential", n_layers=s["L"],
                            deq_sweeps=deq_sweeps, ctx_mod=ctx_mod, enable_key_mod=key_mod,
                            attn_logn_ref=logn_ref, **{**base, **cfg_overrides})
        return DualModLM(cfg), "dualmod"
    if arch == "gdn":
        return build_gdn(vocab, s["d"], s["L"], s["h"]), "dualmod"
    raise ValueError(arch)


def logits_of(kind, model, x, K=None):
    if kind in ("looped", "fbtp"):
        return model(x, K=K)[0]
    if kind == "fla":
        return model(input_ids=x).logits
    return model(x)[0]


# ---- loss / accuracy --------------------------------------------------------------------------------
def masked_loss(logits, tok, tgt, msk):
    """CE over the masked positions in the batch's convention."""
    b, p = msk.nonzero(as_tuple=True)
    if tgt is not None:
        return F.cross_entropy(logits[b, p].float(), tgt[b, p])
    return F.cross_entropy(logits[b, p - 1].float(), tok[b, p])


def masked_dlogits(logits, tok, tgt, msk):
    """(loss, d loss / d logits) of `masked_loss`, computed by hand so an engine that takes an
    explicit d_logits can be driven (formal_language/harness/train_statetrack_ws.py:300-312)."""
    b, p = msk.nonzero(as_tuple=True)
    if tgt is not None:
        rows, gold = (b, p), tgt[b, p]
    else:
        rows, gold = (b, p - 1), tok[b, p]
    lg = logits[rows].float()
    logp = torch.log_softmax(lg, dim=-1)
    n = max(1, gold.numel())
    loss = -logp.gather(1, gold[:, None]).mean()
    g = torch.exp(logp)
    g[torch.arange(gold.numel(), device=g.device), gold] -= 1.0
    d = torch.zeros_like(logits, dtype=torch.float32)
    d[rows] = g / n
    return loss, d.to(logits.dtype)


@torch.no_grad()
def evaluate(predict, evals, chunk=32):
    """predict(x) -> logits.  evals: {factor: (tok, tgt|None, msk, diff|None)} on the model's
    device.  Returns {factor: acc, "x<f>_by_k": {...}, "x<f>_by_pos8": [...]}"""
    out = {}
    for f, (xe, tge, me, de) in evals.items():
        hit = tot = 0
        by_k, by_pos = {}, {}
        width = xe.shape[1]
        for r0 in range(0, xe.shape[0], chunk):
            xb, mb = xe[r0:r0 + chunk], me[r0:r0 + chunk]
            pred = predict(xb).argmax(-1)
            b, p = mb.nonzero(as_tuple=True)
            if tge is not None:
                ok = pred[b, p] == tge[r0:r0 + chunk][b, p]
                for pos, o in zip(p.tolist(), ok.tolist()):
                    cell = by_pos.setdefault(min(7, pos * 8 // width), [0, 0])
                    cell[0] += o
                    cell[1] += 1
            else:
                ok = pred[b, p - 1] == xb[b, p]
            hit += int(ok.sum())
            tot += int(mb.sum())
            if de is not None:
                side = de[r0:r0 + chunk]
                ks = side[mb.cpu().numpy()] if side.shape[1] == width else side.reshape(-1)
                for k, o in zip(ks.tolist(), ok.tolist()):
                    cell = by_k.setdefault(k, [0, 0])
                    cell[0] += o
                    cell[1] += 1
        out[f] = round(hit / max(1, tot), 4)
        if by_k:
            out[f"x{f}_by_k"] = {k: round(a / c, 3) for k, (a, c) in sorted(by_k.items())}
        if by_pos:
            out[f"x{f}_by_pos8"] = [round(a / c, 3) for _, (a, c) in sorted(by_pos.items())]
    return out


def cosine(step, steps, lr):
    return lr * 0.5 * (1 + math.cos(math.pi * step / steps))
