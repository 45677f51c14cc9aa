"""MQAR (multi-query associative recall) evaluation of a checkpoint: N key = value pairs shown once, then M
queries "? key =" whose next token must be the value; score = fraction of queried values predicted
exactly by greedy arg-max.  Keys and values are single token ids drawn without replacement from a
mid-vocabulary range, so the score is recall, not tokenisation.  Deterministic per (seed, configuration).

  python -m dual_mod_public_b200.eval.mqar --ckpt out/run/ckpt_latest.pt --pairs 8,16,32,64 --seq_len 2048

Writes `mqar_<run>_<step>.json` beside the checkpoint.  `--finetune_steps N` first trains on freshly drawn
MQAR sequences (the post-training variant), with the loss only on the queried positions.

Reference parity: lm/eval/mqar.py:1-120 (format, scoring, JSON), lm/eval/posttrain_mqar.py:1-139 (fine-tune
then evaluate).
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.nn.functional as F

from ..utils.checkpoint import load_checkpoint, model_from_checkpoint


def markers(vocab):
    """(BOS, SEP, EQ, Q) ids: the word pieces ", = ?" of the 32k vocabulary when it is that large, else
    the top of the vocabulary."""
    return (1, 29892, 29922, 29973) if vocab >= 30000 else (1, vocab - 1, vocab - 2, vocab - 3)


def build_batch(n_pairs, n_queries, seq_len, n_seq, seed, vocab=32000):
    bos, SEP, EQ, Q = markers(vocab)
    lo, hi = (3000, 28000) if vocab >= 30000 else (2, vocab - 3)
    assert hi - lo >= 2 * n_pairs, "vocabulary too small for this many pairs"
    g = torch.Generator().manual_seed(seed)
    xs, tgt_pos, tgt_tok = [], [], []
    for _ in range(n_seq):
        ids = torch.randperm(hi - lo, generator=g)[:2 * n_pairs] + lo
        keys, vals = ids[:n_pairs].tolist(), ids[n_pairs:].tolist()
        seq = [bos]
        for k, v in zip(keys, vals):
            seq += [k, EQ, v, SEP]
        pos, toks = [], []
        for q in torch.randperm(n_pairs, generator=g)[:n_queries].tolist():
            seq += [Q, keys[q], EQ]
            pos.append(len(seq) - 1)                       # the value is predicted AT this position
            toks.append(vals[q])
            seq += [vals[q], SEP]
        assert len(seq) <= seq_len, "configuration too large for seq_len"
        xs.append(seq + [SEP] * (seq_len - len(seq)))       # causal-safe tail padding
        tgt_pos.append(pos)
        tgt_tok.append(toks)
    return torch.tensor(xs, dtype=torch.long), torch.tensor(tgt_pos), torch.tensor(tgt_tok)


@torch.no_grad()
def run(model, n_pairs, n_queries, seq_len, n_seq, seed, device, rows=32):
    x, pos, tok = build_batch(n_pairs, n_queries, seq_len, n_seq, seed, model.cfg.vocab_size)
    hit = tot = 0
    amp = torch.autocast(torch.device(device).type, dtype=torch.bfloat16, enabled=torch.device(device).type == "cuda")
    for r0 in range(0, n_seq, rows):
        xb = x[r0:r0 + rows].to(device)
        with amp:
            pred = model(xb)[0].argmax(-1).cpu()
        p, t = pos[r0:r0 + rows], tok[r0:r0 + rows]
        hit += (pred.gather(1, p) == t).sum().item()
        tot += t.numel()
    return hit / max(1, tot)


def finetune(model, steps, n_pairs, n_queries, seq_len, batch, lr, device, seed=0):
    opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=(0.9, 0.95), weight_decay=0.0)
    model.train()
    for s in range(steps):
        x, pos, tok = build_batch(n_pairs, n_queries, seq_len, batch, seed + 1000 + s, model.cfg.vocab_size)
        x, pos, tok = x.to(device), pos.to(device), tok.to(device)
        logits = model(x)[0].float()
        sel = logits.gather(1, pos.unsqueeze(-1).expand(-1, -1, logits.shape[-1]))
        loss = F.cross_entropy(sel.flatten(0, 1), tok.flatten())
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
    model.eval()
    return loss.item() if steps else float("nan")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--pairs", default="8,16,32,64")
    ap.add_argument("--queries", type=int, default=0, help="queries per sequence (0 = min(pairs, 16))")
    ap.add_argument("--seq_len", type=int, default=2048)
    ap.add_argument("--n_seq", type=int, default=64)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--finetune_steps", type=int, default=0)
    ap.add_argument("--finetune_lr", type=float, default=1e-4)
    ap.add_argument("--device", default="")
    args = ap.parse_args(argv)
    dev = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    ck = load_checkpoint(args.ckpt)
    model = model_from_checkpoint(ck, device=dev, ctx_len=args.seq_len).eval()
    if model.cfg.attn_mode not in ("vanilla", "static"):
        model.cfg.attn_mode = "sequential"
    res = {}
    for n in [int(p) for p in args.pairs.split(",")]:
        m = args.queries or min(n, 16)
        if args.finetune_steps:
            res[f"ft_loss_{n}"] = finetune(model, args.finetune_steps, n, m, args.seq_len, 8, args.finetune_lr, dev)
        res[str(n)] = run(model, n, m, args.seq_len, args.n_seq, args.seed, dev)
        print(f"pairs {n:4d} queries {m:3d}: recall {res[str(n)]:.4f}", flush=True)
    run_name = os.path.basename(os.path.dirname(os.path.abspath(args.ckpt)))
    out = os.path.join(os.path.dirname(os.path.abspath(args.ckpt)), f"mqar_{run_name}_{ck.get('step', -1)}.json")
    json.dump({"ckpt": args.ckpt, "step": ck.get("step", -1), "seq_len": args.seq_len, "recall": res}, open(out, "w"), indent=1)
    print("wrote", out, flush=True)
    return res


if __name__ == "__main__":
    main()
