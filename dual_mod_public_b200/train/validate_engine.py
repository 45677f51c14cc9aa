"""Validate an engine against the model's exact sequential scan.

  python -m dual_mod_public_b200.train.validate_engine --engine wavescan --T 256 --B 2 --L 2 --W 96
  python -m dual_mod_public_b200.train.validate_engine --engine wave3d --T 128 --C 16 --fp32

  R1  engine at its exact setting vs `model(idx, targets)` (exact scan): loss, logits, per-group gradients.
      Cell engine: K = c.  Wavefront engine: K = T - T/C + 1 (K = C is an approximation for that operator).
  R2  the same with a sliding window W (cell engine only).
  R4  info: loss at every K of `--ladder` against the exact loss (the approximation ladder).

In bf16 the thresholds are the reference's (loss 3e-3, logits 0.25 absolute, gradient groups 5e-2
relative) or, with `--floor`, twice the bf16 noise floor measured as exact-scan-bf16 vs exact-scan-fp32.
In fp32 (`--fp32`, or on CPU): loss 1e-5, logits 1e-4, gradients 1e-4.

Reference parity: lm/train_1p3b/validate_rawdiag.py:1-150 (R1-R4 protocol, group tables, noise floor).
"""

from __future__ import annotations

import argparse
from collections import defaultdict

import torch
import torch.nn.functional as F

from ..config import DualModConfig
from ..engines.schedule import uniform_chunks
from ..engines.wave3d import Wave3DEngine
from ..engines.wavescan import WaveScanEngine
from ..models import DualModLM


def group_name(n):
    p = n.split(".")
    return p[0] if p[0] != "blocks" else ".".join(p[:1] + p[2:3])


def group_rel(g_ref, g_new):
    acc = defaultdict(lambda: [0.0, 0.0])
    for n, gr in g_ref.items():
        gn = g_new.get(n)
        if gr is None or gn is None:
            continue
        acc[group_name(n)][0] += (gr.float() - gn.float()).pow(2).sum().item()
        acc[group_name(n)][1] += gr.float().pow(2).sum().item()
    return {g: (v[0] ** 0.5) / max(v[1] ** 0.5, 1e-30) for g, v in acc.items()}


def scan_ref(model, idx, tgt, amp):
    model.zero_grad(set_to_none=True)
    mode, model.cfg.attn_mode = model.cfg.attn_mode, "sequential"
    model.train()
    with torch.autocast(idx.device.type, dtype=torch.bfloat16, enabled=amp):
        lg, loss = model(idx, targets=tgt)
    loss.backward()
    model.eval()
    model.cfg.attn_mode = mode
    g = {n: None if p.grad is None else p.grad.detach().float().clone() for n, p in model.named_parameters()}
    model.zero_grad(set_to_none=True)
    return loss.item(), lg.detach().float(), g


def engine_run(model, eng, idx, tgt, sid=0):
    eng.zero_grads()
    eng.pack()
    loss = eng.train_step(idx, tgt, sid=sid).item()
    g = {n: eng.grads.get(p).detach().float().clone() for n, p in model.named_parameters()}
    return loss, eng.logits.detach().float().clone() if eng.keep_logits else None, g


def compare(tag, ref, got, tol_loss, tol_lg, tol_g, floor=None, out=print):
    lr, lgr, gr = ref
    lw, lgw, gw = got
    d = abs(lr - lw)
    mad = (lgw - lgr).abs().max().item() if lgw is not None else 0.0
    rels = group_rel(gr, gw)
    ok = d < tol_loss and mad < tol_lg
    out(f"  [{tag}] loss ref={lr:.6f} eng={lw:.6f} |d|={d:.3e} (tol {tol_loss:.0e}); logits max|d|={mad:.3e} (tol {tol_lg})")
    worst = 0.0
    for g in sorted(rels):
        tol = max(tol_g, 2.0 * floor[g]) if floor and g in floor else tol_g
        good = rels[g] < tol
        ok &= good
        worst = max(worst, rels[g])
        out(f"    {g:28} rel={rels[g]:.3e} (tol {tol:.1e}){'' if good else '   <-- FAIL'}")
    out(f"  [{'PASS' if ok else 'FAIL'}] {tag}: worst gradient group rel={worst:.3e}")
    return ok


def main(argv=None, out=print):
    ap = argparse.ArgumentParser()
    a = ap.add_argument
    a("--engine", default="wavescan", choices=["wavescan", "wave3d"])
    a("--T", type=int, default=256)
    a("--B", type=int, default=2)
    a("--L", type=int, default=2)
    a("--d", type=int, default=256)
    a("--heads", type=int, default=4)
    a("--C", type=int, default=64)
    a("--W", type=int, default=0, help="also run R2 with this sliding window (cell engine)")
    a("--ladder", default="", help="R4: comma-separated K values")
    a("--fp32", action="store_true")
    a("--floor", action="store_true", help="bf16: gradient tolerance = max(5e-2, 2 x measured noise floor)")
    a("--device", default="")
    a("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    dev = torch.device(args.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    amp = dev.type == "cuda" and not args.fp32
    tl, tg_, tgr = (3e-3, 0.25, 5e-2) if amp else (1e-5, 1e-4, 1e-4)
    results = {}

    def build(window):
        torch.manual_seed(args.seed)
        cfg = DualModConfig(d_model=args.d, n_layers=args.L, n_heads=args.heads, vocab_size=512, max_seq_len=args.T,
                            gate_bias_init=0.0, ctx_proj_init_std=0.02, local_window=window or None,
                            checkpoint_chunk=0)
        m = DualModLM(cfg).to(dev).eval()
        with torch.no_grad():                                   # leave the near-vanilla init: live gates and ctx branch
            for blk in m.blocks:
                for name in ("w_gk", "w_gv", "w_kctx", "w_vctx"):
                    for p in getattr(blk.attn, name).parameters():
                        if p.dim() >= 2:
                            p.normal_(0, 0.05)
        return cfg, m

    def make(model, ks, window):
        T, C = args.T, args.C
        kw = dict(device=dev, autocast_bf16=amp, keep_logits=True)
        if args.engine == "wave3d":
            return Wave3DEngine(model, ks, args.B, T, C=C, **kw)
        return WaveScanEngine(model, [uniform_chunks(T, C, min(C, k)) for k in ks], args.B, T, **kw)

    g = torch.Generator().manual_seed(1)
    idx = torch.randint(0, 512, (args.B, args.T), generator=g).to(dev)
    tgt = torch.randint(0, 512, (args.B, args.T), generator=g).to(dev)
    k_exact = args.C if args.engine == "wavescan" else args.T - args.T // args.C + 1
    ladder = [int(k) for k in args.ladder.split(",") if k]
    for tag, window in (("R1 full causal", 0),) + ((("R2 window %d" % args.W, args.W),) if args.W and args.engine == "wavescan" else ()):
        cfg, m = build(window)
        ref = scan_ref(m, idx, tgt, amp)
        floor = None
        if amp and args.floor:
            floor = group_rel(scan_ref(m, idx, tgt, False)[2], ref[2])
        eng = make(m, [k_exact] + ladder, window)
        out(f"{tag}: {args.engine} K={k_exact} C={args.C} T={args.T} {'bf16' if amp else 'fp32'}")
        results[tag] = compare(tag, ref, engine_run(m, eng, idx, tgt, 0), tl, tg_, tgr, floor, out)
        if ladder and not window:
            for i, k in enumerate(ladder):
                with torch.no_grad():
                    l = eng.forward(idx, tgt, sid=i + 1).item()
                out(f"  [R4] K={k:3d} loss={l:.6f}  minus exact={l - ref[0]:+.3e}")
                results[f"R4 K={k}"] = l - ref[0]
    return results


if __name__ == "__main__":
    ok = main()
    raise SystemExit(0 if all(v is not False for v in ok.values()) else 1)
