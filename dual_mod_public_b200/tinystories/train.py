"""TinyStories ablation trainer: the eager exact sequential scan under torch DDP.

  python -m dual_mod_public_b200.tinystories.train --preset B --data_dir data/tinystories
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
      -m dual_mod_public_b200.tinystories.train --preset A --batch_size 64

Presets select the ablation arm; EVERY field of `DualModConfig` and `TrainConfig` is also a command-line
flag (`--d_model 512 --gate_rank 8 ...`), explicit flags win over the preset.

  A     vanilla Transformer++ (modulation off)        B     full Dual-Mod (key + value modulation)
  C     value modulation only                         D     key modulation only
  F1    capacity control: widened queries, grouped KV  F2    capacity control: wider MHA
  F3    static branch: the context branch reads the normed input instead of the read (no recurrence)
  G-A   gate-bias init spread per dimension at mean 0.5   G-B   solution-shaped gate-bias init

Data: `PackedLoader` over `<data_dir>/{train,val}.bin` (written by `data.packed.prepare`), or
`--data_dir synthetic` for uniform random ids.  Checkpoints hold `model, optimizer, step, model_cfg,
train_cfg`; telemetry (gate statistics, gradient-norm ratios) is logged every `telemetry_interval`.

Reference parity: tinystories/train.py:39-69 (presets), :72-102 (flag generation), :105-307 (loop, DDP
static graph :176, checkpoint keys :289-292).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import time
from dataclasses import fields

import torch
import torch.distributed as dist

from ..config import DualModConfig, TrainConfig
from ..data.packed import PackedLoader, SyntheticStream
from ..models import DualModLM
from ..models.telemetry import collect_telemetry, grad_norm_ratios
from ..parallel.fused_optim import decay_groups
from ..utils.checkpoint import save_atomic

PRESETS = {
    "A": dict(attn_mode="vanilla", enable_key_mod=False, enable_value_mod=False, run_name="A-vanilla"),
    "B": dict(attn_mode="sequential", enable_key_mod=True, enable_value_mod=True, run_name="B-dualmod"),
    "C": dict(attn_mode="sequential", enable_key_mod=False, enable_value_mod=True, run_name="C-valuemod"),
    "D": dict(attn_mode="sequential", enable_key_mod=True, enable_value_mod=False, run_name="D-keymod"),
    "F1": dict(attn_mode="vanilla", enable_key_mod=False, enable_value_mod=False, n_heads=32, n_kv_heads=8,
               head_dim_override=64, run_name="F1-qwiden-gqa"),
    "F2": dict(attn_mode="vanilla", enable_key_mod=False, enable_value_mod=False, n_heads=20, n_kv_heads=0,
               head_dim_override=64, run_name="F2-widemha"),
    "F3": dict(attn_mode="static", enable_key_mod=True, enable_value_mod=True, run_name="F3-staticbranch"),
    "G-A": dict(attn_mode="sequential", enable_key_mod=True, enable_value_mod=True, gate_bias_init_k="ugi",
                gate_bias_init_v="ugi", run_name="G-A-ugi"),
    "G-B": dict(attn_mode="sequential", enable_key_mod=True, enable_value_mod=True, gate_bias_init_k="committed",
                gate_bias_init_v="band", run_name="G-B-shaped"),
}


def _flag_type(f):
    d = f.default
    if isinstance(d, bool):
        return lambda s: s.lower() in ("1", "true", "yes")
    if isinstance(d, (int, float, str)):
        return type(d)
    return str                                     # Optional[...] fields default to None: parsed below


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", choices=list(PRESETS), default=None)
    for cls in (DualModConfig, TrainConfig):
        for f in fields(cls):
            ap.add_argument(f"--{f.name}", type=_flag_type(f), default=None)
    ap.add_argument("--resume", default=None)
    ap.add_argument("--max_steps", type=int, default=0, help="stop early (tests)")
    return ap.parse_args(argv)


def _coerce(f, v):
    if isinstance(v, str) and not isinstance(f.default, str):
        if v.lower() in ("none", ""):
            return None
        try:
            return json.loads(v)
        except ValueError:
            return v
    return v


def build_configs(args):
    over = dict(PRESETS[args.preset]) if args.preset else {}
    kws = []
    for cls in (DualModConfig, TrainConfig):
        kw = {}
        for f in fields(cls):
            v = getattr(args, f.name, None)
            if v is not None:
                kw[f.name] = _coerce(f, v)
            elif f.name in over:
                kw[f.name] = over[f.name]
        kws.append(kw)
    return DualModConfig(**kws[0]), TrainConfig(**kws[1])


def main(argv=None):
    args = parse_args(argv)
    mcfg, tcfg = build_configs(args)
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available() and tcfg.device != "cpu"
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if cuda:
            torch.cuda.set_device(local)
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world)
    master = rank == 0
    torch.manual_seed(tcfg.seed)
    model = DualModLM(mcfg).to(dev)
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local] if cuda else None, static_graph=True)
    opt = torch.optim.AdamW(decay_groups(model, tcfg.weight_decay), lr=tcfg.lr, betas=(tcfg.beta1, tcfg.beta2),
                            fused=cuda)
    T, Bl = mcfg.max_seq_len, tcfg.batch_size // world
    if tcfg.data_dir == "synthetic":
        syn = SyntheticStream(mcfg.vocab_size, T, Bl, rank=rank, seed=tcfg.data_seed)
        train_xy = lambda s: (lambda b: (b[:, :T].to(dev), b[:, 1:T + 1].to(dev)))(syn.block(s))
        val_xy = lambda i: train_xy(10 ** 8 + i)
    else:
        tl = PackedLoader(tcfg.data_dir, "train", T, Bl * world, data_seed=tcfg.data_seed)
        vl = PackedLoader(tcfg.data_dir, "val", T, Bl, data_seed=tcfg.data_seed)
        shard = lambda xy: tuple(t[rank * Bl:(rank + 1) * Bl].to(dev) for t in xy)
        train_xy = lambda s: shard(tl.train_batch(s))
        val_xy = lambda i: tuple(t.to(dev) for t in vl.val_batch(i))
    tok_per_step = tcfg.batch_size * tcfg.grad_accum * T
    total = max(1, int(tcfg.tokens_target // tok_per_step))
    if args.max_steps:
        total = min(total, args.max_steps)
    warm = max(1, int(tcfg.warmup_frac * total))
    out_dir = os.path.join(tcfg.out_dir, tcfg.run_name)
    step = 0
    if args.resume:
        ck = torch.load(args.resume, map_location="cpu", weights_only=False)
        model.load_state_dict(ck["model"])
        opt.load_state_dict(ck["optimizer"])
        step = ck["step"] + 1
    if master:
        os.makedirs(out_dir, exist_ok=True)
        mlog = open(os.path.join(out_dir, "metrics.jsonl"), "a")
        print(f"{tcfg.run_name}: {model.num_params() / 1e6:.2f}M non-embedding params, {total} steps", flush=True)
    amp = lambda: torch.autocast(dev.type, dtype=torch.bfloat16, enabled=cuda and mcfg.dtype != "fp32")
    last = float("nan")
    while step < total:
        lr = tcfg.lr * (step + 1) / warm if step < warm else \
            tcfg.min_lr + 0.5 * (tcfg.lr - tcfg.min_lr) * (1 + math.cos(math.pi * (step - warm) / max(1, total - warm)))
        for g in opt.param_groups:
            g["lr"] = lr
        t0 = time.time()
        model.train()
        tot = 0.0
        for a in range(tcfg.grad_accum):
            x, y = train_xy(step * tcfg.grad_accum + a)
            with amp():
                _, loss = net(x, targets=y)
            (loss / tcfg.grad_accum).backward()
            tot += loss.item() / tcfg.grad_accum
        rec = {"step": step, "train/loss": tot, "train/lr": lr}
        if tcfg.telemetry_interval and step % tcfg.telemetry_interval == 0 and mcfg.dual_mod_active:
            rec.update(grad_norm_ratios(model))
        gn = torch.nn.utils.clip_grad_norm_(model.parameters(), tcfg.grad_clip).item()
        opt.step()
        opt.zero_grad(set_to_none=True)
        last = tot
        rec.update({"train/grad_norm": gn, "train/step_ms": (time.time() - t0) * 1e3,
                    "train/tokens": (step + 1) * tok_per_step})
        if tcfg.eval_interval and step % tcfg.eval_interval == 0 and step > 0:
            model.eval()
            vs = []
            with torch.no_grad(), amp():
                for i in range(tcfg.eval_iters):
                    xv, yv = val_xy(i)
                    vs.append(model(xv, targets=yv)[1].item())
            rec["val/loss"] = sum(vs) / len(vs)
            if tcfg.telemetry_interval and mcfg.dual_mod_active:
                xv = val_xy(0)[0]
                fmask = torch.zeros(mcfg.vocab_size, dtype=torch.bool)       # no function-word list: all content
                with torch.no_grad(), amp():
                    rec.update(collect_telemetry(model, xv, fmask)[0])
        if master:
            mlog.write(json.dumps({k: (v if isinstance(v, (int, float, str, bool)) else float(v)) for k, v in rec.items()
                                   if isinstance(v, (int, float, str, bool)) or hasattr(v, "__float__")}) + "\n")
            mlog.flush()
            if step % tcfg.log_interval == 0:
                print(f"step {step}/{total} loss {tot:.4f} gn {gn:.3f} lr {lr:.2e}", flush=True)
            if tcfg.ckpt_interval and step > 0 and step % tcfg.ckpt_interval == 0:
                save_atomic({"model": model.state_dict(), "optimizer": opt.state_dict(), "step": step,
                             "model_cfg": mcfg.to_dict(), "train_cfg": tcfg.to_dict()},
                            os.path.join(out_dir, "ckpt_latest.pt"))
        step += 1
    if master:
        save_atomic({"model": model.state_dict(), "optimizer": opt.state_dict(), "step": step - 1,
                     "model_cfg": mcfg.to_dict(), "train_cfg": tcfg.to_dict()}, os.path.join(out_dir, "ckpt_latest.pt"))
        mlog.close()
        print(f"FINAL {tcfg.run_name} step {step} loss {last:.4f}", flush=True)
    return {"loss": last, "steps": step}


if __name__ == "__main__":
    main()
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()
