"""Baseline arms on the same token stream and recipe as the Dual-Mod runs, with torch DDP.

  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      -m dual_mod_public_b200.train.train_baseline --arch ematch --data_bin corpus.bin --out_dir out/ematch

  --arch vanilla   the Dual-Mod model with the modulation off (a plain Transformer++ of the same shape)
  --arch ematch    the same, widened to the parameter count of the Dual-Mod model (d1216 / 19 heads / ffn 3520)
  --arch gdn       gated delta-rule network (`models.baselines.build_gdn`)
  --arch fbt | looped | rdepth | lstm   the small-scale baselines of the formal-language harness

Same AdamW(0.9, 0.95), weight decay on matrices only, warm-up + cosine, clip 1.0, EMA outlier batch skip
with non-finite always skipped (`governors.SkipRule`), as the Dual-Mod arm.  Micro-batch accumulation
runs under `no_sync()` so the gradient all-reduce happens once per optimizer step.  Checkpoints carry
`arch` beside the usual keys.

Reference parity: lm/train_340m/train_baseline.py:1-336 (arms, DDP + no_sync :191-194 / :263-271, skip
protocol, checkpoint keys :245-247).
"""

from __future__ import annotations

import argparse
import contextlib
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..config import DualModConfig, preset
from ..data.packed import SyntheticStream, memmap_stream
from ..engines.schedule import cosine_lr
from ..models import DualModLM
from ..models import baselines as B
from ..parallel.fused_optim import decay_groups
from ..utils.checkpoint import save_atomic
from .governors import MetricsLogger, SkipRule


def build_arch(arch, shape, vocab, T):
    """(model, model_cfg dict).  `shape` = (d, layers, heads, ffn)."""
    d, L, h, ffn = shape
    if arch in ("vanilla", "ematch"):
        if arch == "ematch" and (d, L, h) == (1024, 24, 16):
            d, h, ffn = 1216, 19, 3520
        cfg = DualModConfig(d_model=d, n_layers=L, n_heads=h, mlp_hidden_override=ffn, vocab_size=vocab,
                            max_seq_len=T, attn_mode="vanilla")
        return DualModLM(cfg), cfg.to_dict()
    if arch == "gdn":
        return B.build_gdn(vocab, d, L, h), {"arch": "gdn", "d": d, "L": L, "h": h, "vocab": vocab}
    cfg = DualModConfig(d_model=d, n_layers=L, n_heads=h, mlp_hidden_override=ffn, vocab_size=vocab, max_seq_len=T,
                        attn_mode="vanilla")
    if arch == "fbt":
        return B.FBTLM(cfg), cfg.to_dict()
    if arch in ("looped", "rdepth"):
        return (B.LoopedLM if arch == "looped" else B.RecurrentDepthLM)(cfg), cfg.to_dict()
    if arch == "lstm":
        return B.LSTMLM(vocab, d, L), {"arch": "lstm", "d": d, "L": L, "vocab": vocab}
    raise ValueError(arch)


def logits_of(model, x):
    out = model(x)
    return out[0] if isinstance(out, tuple) else out


def main(argv=None):
    ap = argparse.ArgumentParser()
    a = ap.add_argument
    a("--arch", default="vanilla", choices=["vanilla", "ematch", "gdn", "fbt", "looped", "rdepth", "lstm"])
    a("--shape", default="1024,24,16,2816", help="d,layers,heads,ffn")
    a("--vocab", type=int, default=32000)
    a("--seq_len", type=int, default=2048)
    a("--global_batch", type=int, default=256)
    a("--micro_batch", type=int, default=8)
    a("--total_steps", type=int, default=1000)
    a("--warmup_steps", type=int, default=100)
    a("--lr", type=float, default=3e-4)
    a("--min_lr", type=float, default=3e-5)
    a("--weight_decay", type=float, default=0.01)
    a("--skip_factor", type=float, default=5.0)
    a("--skip_grace_steps", type=int, default=50)
    a("--data_bin", default="")
    a("--synthetic", action="store_true")
    a("--out_dir", default="out/baseline")
    a("--ckpt_every", type=int, default=0)
    a("--seed", type=int, default=1337)
    a("--device", default="")
    a("--log_every", type=int, default=10)
    args = ap.parse_args(argv)
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available() and args.device != "cpu"
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if cuda:
            torch.cuda.set_device(local)
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    T = args.seq_len
    torch.manual_seed(args.seed)
    model, mcfg = build_arch(args.arch, tuple(int(x) for x in args.shape.split(",")), args.vocab, T)
    model = model.to(dev)
    net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local] if cuda else None) if world > 1 else model
    groups = decay_groups(model, args.weight_decay)
    opt = torch.optim.AdamW(groups, lr=args.lr, betas=(0.9, 0.95), eps=1e-8, fused=cuda)
    local_b = args.global_batch // world
    micro = min(args.micro_batch, local_b)
    accum = local_b // micro
    if args.synthetic or not args.data_bin:
        syn = SyntheticStream(args.vocab, T, local_b, rank=rank, seed=args.seed)
        stream = (syn.block(s) for s in range(1 << 62))
    else:
        stream = memmap_stream(args.data_bin, T, local_b, rank, world, seed=42)
    skip = SkipRule(skip_factor=args.skip_factor, grace_steps=args.skip_grace_steps)
    log = MetricsLogger(args.out_dir, enabled=rank == 0)
    params = [p for p in model.parameters() if p.requires_grad]
    final = float("nan")
    for step in range(args.total_steps):
        lr = cosine_lr(step, args.total_steps, args.warmup_steps, args.lr, args.min_lr)
        for g in opt.param_groups:
            g["lr"] = lr
        blk = next(stream).to(dev, non_blocking=True)
        t0 = time.time()
        loss_acc = 0.0
        for i in range(accum):
            x, y = blk[i * micro:(i + 1) * micro, :T], blk[i * micro:(i + 1) * micro, 1:T + 1]
            # all-reduce only with the last micro-batch's backward
            hold = net.no_sync() if world > 1 and i < accum - 1 else contextlib.nullcontext()
            with hold:
                with torch.autocast(dev.type, dtype=torch.bfloat16, enabled=cuda):
                    lg = logits_of(net, x)
                loss = F.cross_entropy(lg.float().view(-1, lg.shape[-1]), y.reshape(-1)) / accum
                loss.backward()
            loss_acc += loss.item()
        gn = torch.nn.utils.clip_grad_norm_(params, 1.0).item()
        skipped = skip.decide(gn, loss_acc, False)
        if not skipped:
            opt.step()
            final = loss_acc
        skip.update(gn, loss_acc, False, skipped)
        opt.zero_grad(set_to_none=True)
        log.log(step, **{"train/loss": loss_acc, "train/lr": lr, "train/grad_norm": gn, "train/skipped": skipped,
                         "train/step_ms": (time.time() - t0) * 1e3, "train/tokens": (step + 1) * args.global_batch * T})
        if rank == 0 and step % args.log_every == 0:
            print(f"step {step} loss {loss_acc:.4f} gn {gn:.3f} lr {lr:.2e}{' SKIPPED' if skipped else ''}", flush=True)
        if args.ckpt_every and step and step % args.ckpt_every == 0 and rank == 0:
            save_atomic({"model": model.state_dict(), "optimizer": opt.state_dict(), "step": step, "model_cfg": mcfg,
                         "arch": args.arch, **skip.state_dict()}, os.path.join(args.out_dir, "ckpt_latest.pt"))
    if rank == 0:
        print(f"FINAL arch {args.arch} step {args.total_steps} loss {final:.4f}", flush=True)
    log.close()
    return {"loss": final, "skipped": skip.skipped_total}


if __name__ == "__main__":
    main()
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
