"""A5 state-tracking benchmark: one-layer Dual-Mod (d=512, 8 heads x 64, ffn 1376, vocab 128) trained on
tagged A5 word-problem batches (T = 64 positions: BOS + 63 ops, batch 256) through the exact cell engine (c=16, K=16).

  python -m dual_mod_public_b200.formal.bench_a5 --steps 200 --warmup 5

Each sequence is BOS plus 63 uniform random ids out of the 60 group elements; the label at position t is the
running product of elements 1..t (at-position targets).  Prints one JSON line: ms per step (CUDA events
around the timed steps, forward + backward + fused AdamW through `EngineTrainer.step`), sequences/s,
tokens/s, and the masked accuracy on a held-out batch before and after the run.

Reference parity: formal_language/a5/run_a5_T64.sh and formal_language/harness/train_statetrack_ws.py
(the exact c=16 / K=16 engine path).
"""

from __future__ import annotations

import argparse
import json
import time

import numpy as np
import torch

from ..config import preset
from ..models import DualModLM
from . import harness as H
from .ws import EngineTrainer


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--bsz", type=int, default=256)
    ap.add_argument("--n_ops", type=int, default=63, help="ops per sequence; the sequence is 1 BOS + n_ops = 64 positions")
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--device", default="")
    a = ap.parse_args(argv)
    dev = torch.device(a.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    args = H.task_args(task="group", group="a5", format="tagged", n_ops=a.n_ops, wd=0.01, lr=a.lr, ws_chunk=16)
    mul, n_elem = H.task_tables(args)
    rng = np.random.default_rng(0)
    tok, tgt, msk, _ = H.make_batch(args, mul, n_elem, rng, a.bsz, a.n_ops)
    T = tok.shape[1]
    assert T % 16 == 0, f"sequence length {T} is not a whole number of chunks"
    torch.manual_seed(0)
    cfg = preset("a5_12m", max_seq_len=max(256, T), gate_bias_init=0.0)
    tr = EngineTrainer(DualModLM(cfg), args, dev)
    put = lambda t: None if t is None else t.to(dev)

    def acc(batch):
        x, y, m, _ = batch
        with torch.no_grad():
            pred = tr.logits(put(x).long()).argmax(-1)
        return (pred[put(m).bool()] == put(y).long()[put(m).bool()]).float().mean().item()

    held = H.make_batch(args, mul, n_elem, np.random.default_rng(123), a.bsz, a.n_ops)
    acc0 = acc(held)
    # a fresh batch per step, drawn before the timed region
    batches = [H.make_batch(args, mul, n_elem, rng, a.bsz, a.n_ops) for _ in range(a.warmup + a.steps)]
    step = lambda i: tr.step(put(batches[i][0]).long(), put(batches[i][1]).long(), put(batches[i][2]), a.lr)
    for i in range(a.warmup):
        step(i)
    cuda = dev.type == "cuda"
    if cuda:
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    loss = float("nan")
    for i in range(a.steps):
        loss = step(a.warmup + i)
    if cuda:
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / a.steps
    else:
        ms = (time.perf_counter() - t0) * 1e3 / a.steps
    out = {"metric": "a5_train_ms_per_step", "value": round(ms, 3), "unit": "ms", "higher_is_better": False,
           "sequences_per_s": round(a.bsz / ms * 1e3, 1), "tokens_per_s": round(a.bsz * T / ms * 1e3, 1),
           "steps": a.steps, "warmup": a.warmup, "dtype": "bf16" if cuda else "fp32",
           "config": {"model": "1-layer DM d512 8x64 ffn1376 vocab128", "task": "A5 tagged word problem", "T": T,
                      "batch": a.bsz, "engine": "wavescan c=16 K=16 (exact)"},
           "loss_last": round(loss, 4), "acc_before": round(acc0, 4), "acc_after": round(acc(held), 4),
           "kernel_launches": getattr(tr._engine(a.bsz, T).ops, "launches", 0)}
    print(json.dumps(out), flush=True)
    return out


if __name__ == "__main__":
    main()
