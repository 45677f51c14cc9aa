"""Fixed-point diagnostic for the looped baseline: run a trained `LoopedLM` for K iterations and print, per
iteration k, the relative state change ||x_k - x_{k-1}|| / ||x_k|| (mean over tokens) and the masked
accuracy of the readout applied to x_k.  A collapse to a fixed point shows as the change going to zero
while the accuracy stays flat.

  python -m dual_mod_public_b200.formal.loop_fixed_point run.pt --K 64 [--n_ops 128] [--every]

The checkpoint is the harness's `{"model", "args"}` file; task and sizes are read from `args`.

Reference parity: formal_language/loop_fixed_point/loop_fixed_point.py:1-60.
"""

from __future__ import annotations

import argparse

import numpy as np
import torch

from . import harness as H


def analyse(model, x, tgt, msk, K, every=False, out=print):
    """Rows of (k, relative change, accuracy).  x, tgt [B,T] long, msk [B,T] bool."""
    rows, prev = [], None
    with torch.no_grad():
        _, _, states = model(x, K=K, return_all=True)
        T = x.shape[1]
        for k, xk in enumerate(states, 1):
            xk = xk.float()
            ch = float("nan") if prev is None else ((xk - prev).norm(dim=-1) / (xk.norm(dim=-1) + 1e-6)).mean().item()
            xr = model.coda(xk.to(states[0].dtype), model.rope_cos[:T], model.rope_sin[:T]).float() if model.huginn else xk
            pred = model.lm_head(model.norm_f(xr)).argmax(-1)
            acc = (pred[msk] == tgt[msk]).float().mean().item()
            rows.append((k, ch, acc))
            if every or k <= 8 or k % 8 == 0 or k == K:
                out(f"{k:3d} {ch:11.3e} {acc:7.3f}")
            prev = xk
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("ckpt")
    ap.add_argument("--K", type=int, default=64)
    ap.add_argument("--B", type=int, default=128)
    ap.add_argument("--n_ops", type=int, default=0, help="override the sequence size (0 = the training size)")
    ap.add_argument("--every", action="store_true")
    ap.add_argument("--device", default="")
    a = ap.parse_args(argv)
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    ck = torch.load(a.ckpt, map_location="cpu", weights_only=False)
    args = H.task_args(**ck["args"])
    mul, n_elem = H.task_tables(args)
    vocab = ck["model"]["tok_emb.weight"].shape[0]
    model, kind = H.build_model("looped", vocab, 4096, scale=args.scale, loop_layers=args.loop_layers,
                                loop_k=args.loop_k, loop_huginn=bool(getattr(args, "loop_huginn", False)),
                                loop_bp=int(getattr(args, "loop_bp", 0)),
                                loop_emb_scale=bool(getattr(args, "loop_emb_scale", False)))
    missing, unexpected = model.load_state_dict(ck["model"], strict=False)
    print("load: missing", len(missing), "unexpected", len(unexpected))
    model = model.to(dev).eval()
    rng = np.random.default_rng(0)
    tok, tgt, msk, _ = H.make_batch(args, mul, n_elem, rng, a.B, a.n_ops or args.n_ops, evaluating=True)
    if tgt is None:                                                 # next-token convention
        tgt = torch.roll(tok, -1, 1)
    print(f"{'k':>3s} {'rel_change':>11s} {'acc':>7s}")
    return analyse(model, tok.long().to(dev), tgt.long().to(dev), msk.bool().to(dev), a.K, a.every)


if __name__ == "__main__":
    main()
