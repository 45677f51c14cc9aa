"""Held-out loss of a checkpoint: mean cross-entropy of the exact operator on a fixed validation set.

  python -m dual_mod_public_b200.eval.heldout_loss --ckpt out/run/snap_007000.pt --val data/val.bin --n_batches 8

The Dual-Mod model is scored with the exact operator: on a GPU through the cell engine at K = c (exact,
and far faster than the eager scan), otherwise through the eager sequential scan.  Baseline checkpoints
(`arch` = vanilla / ematch / gdn / ...) are scored through their own forward.  The validation set is a
`.pt` tensor [n_batches, rows, T+1] or a flat uint16 `.bin` token file cut into rows of T+1.  Writes
`heldout_<run>_<step>_<split>.json` beside the checkpoint.

Reference parity: lm/eval/heldout_loss.py:1-78 (row-chunked fp32 CE, per-batch and mean, JSON record).
"""

from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch
import torch.nn.functional as F

from ..engines.schedule import uniform_chunks
from ..utils.checkpoint import load_checkpoint, model_from_checkpoint


def load_val(path, T, rows, n_batches):
    if path.endswith(".pt"):
        return torch.load(path)[:n_batches]
    arr = np.memmap(path, dtype=np.uint16, mode="r")
    n = min(n_batches, len(arr) // ((T + 1) * rows))
    return torch.from_numpy(np.asarray(arr[:n * rows * (T + 1)]).astype(np.int64)).view(n, rows, T + 1)


@torch.no_grad()
def score(model, val, device, chunk=64, use_engine=None):
    """Mean CE per batch.  val [n, rows, T+1]."""
    cfg = getattr(model, "cfg", None)
    T = val.shape[2] - 1
    dual = cfg is not None and hasattr(cfg, "dual_mod_active") and cfg.dual_mod_active and cfg.attn_mode != "vanilla"
    use_engine = (torch.device(device).type == "cuda" and dual and T % chunk == 0) if use_engine is None else use_engine
    out, eng = [], None
    if use_engine:
        from ..engines.wavescan import WaveScanEngine
        eng = WaveScanEngine(model, [uniform_chunks(T, chunk, chunk)], val.shape[1], T, device=device,
                             autocast_bf16=torch.device(device).type == "cuda")
        eng.pack()
    elif dual:
        cfg.attn_mode = "sequential"
    amp = torch.autocast(torch.device(device).type, dtype=torch.bfloat16, enabled=torch.device(device).type == "cuda")
    for i in range(val.shape[0]):
        blk = val[i].to(device)
        x, y = blk[:, :-1], blk[:, 1:]
        if eng is not None:
            out.append(eng.forward(x, y, sid=0).item())
            continue
        tot, cnt = 0.0, 0
        with amp:
            o = model(x)
            logits = o[0] if isinstance(o, tuple) else getattr(o, "logits", o)
        for r0 in range(0, x.shape[0], 8):
            yc = y[r0:r0 + 8]
            tot += F.cross_entropy(logits[r0:r0 + 8].float().flatten(0, 1), yc.reshape(-1), reduction="sum").item()
            cnt += yc.numel()
        out.append(tot / cnt)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--ckpt", required=True)
    ap.add_argument("--val", required=True)
    ap.add_argument("--n_batches", type=int, default=8)
    ap.add_argument("--rows", type=int, default=8)
    ap.add_argument("--seq_len", type=int, default=0)
    ap.add_argument("--device", default="")
    args = ap.parse_args(argv)
    dev = args.device or ("cuda" if torch.cuda.is_available() else "cpu")
    ck = load_checkpoint(args.ckpt)
    arch = ck.get("arch", "dualmod")
    if arch in ("dualmod", "vanilla", "ematch"):
        model = model_from_checkpoint(ck, device=dev).eval()
        T = args.seq_len or model.cfg.max_seq_len
    else:
        from ..train.train_baseline import build_arch
        mc = ck["model_cfg"]
        model, _ = build_arch(arch, (mc.get("d", mc.get("d_model")), mc.get("L", mc.get("n_layers")),
                                     mc.get("h", mc.get("n_heads", 4)), mc.get("mlp_hidden_override", 0) or 4 * mc.get("d", 64)),
                              mc.get("vocab", mc.get("vocab_size")), args.seq_len or 2048)
        model.load_state_dict(ck["model"])
        model = model.to(dev).eval()
        T = args.seq_len or 2048
    val = load_val(args.val, T, args.rows, args.n_batches)
    ls = score(model, val, dev)
    for i, l in enumerate(ls):
        print(f"batch {i}: {l:.4f}", flush=True)
    mean = float(np.mean(ls))
    print(f"heldout mean CE {mean:.4f}  ppl {np.exp(mean):.2f} ({len(ls)} batches x {val.shape[1]} rows)", flush=True)
    run = os.path.basename(os.path.dirname(os.path.abspath(args.ckpt)))
    split = os.path.splitext(os.path.basename(args.val))[0]
    out = os.path.join(os.path.dirname(os.path.abspath(args.ckpt)), f"heldout_{run}_{ck.get('step', -1)}_{split}.json")
    json.dump({"ckpt": args.ckpt, "step": ck.get("step", -1), "mean_ce": mean, "per_batch": ls}, open(out, "w"), indent=1)
    print("wrote", out, flush=True)
    return mean


if __name__ == "__main__":
    main()
