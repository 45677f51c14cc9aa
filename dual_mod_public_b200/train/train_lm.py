"""Language-model trainer: recipes for the 340M (cell engine) and 1.3B (wavefront engine) Dual-Mod runs.

  python -m dual_mod_public_b200.train.train_lm --recipe 340m --out_dir out/dm340 --data_bin corpus.bin
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      -m dual_mod_public_b200.train.train_lm --recipe 1p3b --synthetic --total_steps 100

One optimizer step = `Trainer.step` (H2D of the rank's token block, micro-batches through the engine at
the step's ladder rung, bucket-overlapped fused reduce + clip + skip + AdamW + all-gather, loss read-back)
wrapped by the governors of `governors.py`:

  K-ladder / probes      `KLadder.sid_of(step)`: a pure function of the step (every rank, every resume)
  LR                     warm-up + cosine, times the chain-rho governor's multiplier
  skip                   per batch type EMA threshold handed to the optimizer kernel as `skip_norm`
  clip                   fixed or calibrated (EMA x clip_mult, probe-aware) handed over as `max_norm`
  rank outliers          optional per-rank rejection before the reduction
  rewind                 ring of in-memory healthy checkpoints, wedge detection, rotated data seed
  checkpoints            `ckpt_latest.pt` / `ckpt_prev.pt` (atomic), `snap_%06d.pt`, `persist_%07d.pt`,
                         optional background writer; keys as the reference trainers write them
  metrics                `metrics.jsonl`, one record per step

Data is a flat uint16 token file (`--data_bin`, a pure function of (seed, step) so resume fast-forwards
exactly) or uniform random ids (`--synthetic`).

Reference parity: lm/train_340m/train_flagship.py (ladders :60-100, LR :103-107, loop :848-1165, rewind
:1167-1261) and lm/train_1p3b/train_hero_wave3d.py (ladder :108-153, loop :848-1196, async writer :705-749).
"""

from __future__ import annotations

import argparse
import json
import math
import os
import time

import torch
import torch.distributed as dist

from ..config import DualModConfig, preset
from ..data.packed import SyntheticStream, memmap_stream
from ..engines.schedule import KLadder, cosine_lr, uniform_chunks
from ..utils.checkpoint import AsyncCheckpointWriter, build_checkpoint, load_checkpoint, save_atomic, save_persist
from .governors import (CalibratedClip, ChainRhoGovernor, CreepDetector, FaultInjector, MetricsLogger,
                        RewindGovernor, SkipRule)
from .trainer import Trainer

RECIPES = {
    # name: (model preset, engine, seq_len, global sequences, rungs (c, K), phase bounds, micro-batch)
    "tiny": ("tiny_cpu", "wavescan", 64, 8, ((16, 2), (16, 4), (16, 16)), (0.3, 0.7), 4),
    "340m": ("dm_340m", "wavescan", 2048, 256, ((64, 8), (64, 16), (64, 32), (64, 64)), (0.075, 0.70), 32),
    # the reference's own 340M run (its launch script passes --protocol pdn --dm_lr 3e-4 --clip_mult 2 --skip_factor 20)
    "d960": ("dm_d960", "wavescan", 2048, 256, ((64, 8), (64, 16), (64, 32), (64, 64)), (0.075, 0.70), 32),
    "1p3b": ("dm_1p3b", "wave3d", 4096, 256, ((64, 2), (64, 4), (64, 8)), (0.10, 0.60), 16),
    "hero": ("hero_1p3b", "wave3d", 4096, 128, ((64, 8), (64, 16), (64, 24)), (0.10, 0.60), 16),
}


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    a = ap.add_argument
    a("--recipe", default="340m", choices=sorted(RECIPES))
    a("--engine", default=None, choices=[None, "wavescan", "wave3d"])
    a("--model_overrides", default="{}", help="JSON dict of DualModConfig fields")
    a("--engine_kwargs", default="{}", help="JSON dict passed to the engine constructor")
    a("--ladder", default="", help="rungs as c:K,c:K,... (default: the recipe's)")
    a("--bounds", default="", help="phase boundaries as fractions of total_steps, e.g. 0.075,0.70")
    a("--probe_frac", type=float, default=0.1)
    a("--probe_mult", type=int, default=0)
    a("--seq_len", type=int, default=0)
    a("--global_batch", type=int, default=0, help="sequences per optimizer step over all ranks")
    a("--micro_batch", type=int, default=0)
    a("--total_steps", type=int, default=1000)
    a("--warmup_steps", type=int, default=100)
    a("--lr", type=float, default=3e-4)
    a("--min_lr", type=float, default=3e-5)
    a("--weight_decay", type=float, default=0.1)
    a("--decay_all", action="store_true")
    a("--eps", type=float, default=1e-8)
    a("--wd_doctrine", default="", choices=["", "split", "all", "branch"],
      help="weight-decay layout: matrices only / every parameter / grown-branch parameters at 10x in a group of their own")
    a("--protocol", default="", choices=["", "fs1", "pdn"],
      help="pdn: batch 256, 30000 steps, lr 4e-4 -> 0.1 lr, warm-up 1024, decay on every parameter, skip only non-finite steps")
    a("--dm_accum", type=int, default=1, help="> 1: the Dual-Mod parameters step every this many iterations on the mean gradient")
    a("--dm_lr", type=float, default=None, help="learning rate of the Dual-Mod parameters (two-speed optimizer)")
    a("--cooldown_steps", type=int, default=0, help="> 0: only the write-law parameters move, for this many applied steps")
    a("--cooldown_lr_start", type=float, default=5e-5)
    a("--cooldown_lr_end", type=float, default=1e-6)
    a("--sam", action="store_true", help="sharpness-aware step on the ctx operators (two backward passes)")
    a("--sam_rho", type=float, default=0.05)
    a("--sam_every", type=int, default=1)
    a("--telemetry_every", type=int, default=0, help="> 0: per-layer gate / value-tail / logit telemetry on a fixed batch")
    a("--sat_tau", type=float, default=0.0, help="> 0: saturating backward of the engine")
    a("--max_norm", type=float, default=1.0)
    a("--clip_mult", type=float, default=0.0, help="> 0: calibrated clip at clip_mult x EMA of the norm")
    a("--skip_factor", type=float, default=5.0)
    a("--skip_grace_steps", type=int, default=50)
    a("--gn_hard", type=float, default=0.0)
    a("--rank_outlier_factor", type=float, default=0.0)
    a("--rank_outlier_max", type=int, default=1)
    a("--curv_every", type=int, default=0, help="> 0: log curv/ctx_top_eig (Hessian power iteration, eager scan on a short slice) and gradnorm/L%%02d every this many steps")
    a("--curv_len", type=int, default=256, help="tokens of the first micro-batch rows used for the curvature probe")
    a("--peer_watch_s", type=float, default=0.0, help="> 0: host-side peer check before every step, with this timeout")
    a("--lr_gov", action="store_true")
    a("--auto_rewind", action="store_true")
    a("--rewind_window", type=int, default=50)
    a("--rewind_skip_thresh", type=int, default=10)
    a("--rewind_ring", type=int, default=4)
    a("--snap_interval", type=int, default=100)
    a("--rewind_lookback", type=int, default=100)
    a("--rewind_max", type=int, default=8)
    a("--optimizer", default="fused", choices=["fused", "nccl"])
    a("--no_graphs", action="store_true")
    a("--fp32", action="store_true")
    a("--data_bin", default="")
    a("--val_bin", default="")
    a("--synthetic", action="store_true")
    a("--val_every", type=int, default=0)
    a("--val_batches", type=int, default=4)
    a("--ckpt_every", type=int, default=0)
    a("--persist_every", type=int, default=0)
    a("--async_ckpt", action="store_true")
    a("--out_dir", default="out/run")
    a("--resume", default="", help="checkpoint path, or 'auto' for <out_dir>/ckpt_latest.pt")
    a("--seed", type=int, default=1337)
    a("--log_every", type=int, default=10)
    a("--wandb_project", default="", help="mirror metrics.jsonl to this project")
    a("--eager_val_every", type=int, default=0,
      help="> 0 (needs --val_exact_K): every this many steps score one validation batch both through the engine at the exact setting and through the eager scan, and log the pair")
    a("--eager_val_rows", type=int, default=2)
    a("--eager_val_len", type=int, default=256, help="tokens of the cross-check slice (the eager scan is slow)")
    a("--val_exact_K", type=int, default=0, help="> 0: also validate through the engine at this K (the chunk length is exact for the cell engine) and log val/loss_exact")
    a("--device", default="")
    args = ap.parse_args(argv)
    if args.protocol == "pdn":                           # only where the user left the default
        d = lambda k: getattr(args, k) == ap.get_default(k)
        args.global_batch = 256 if d("global_batch") else args.global_batch
        args.total_steps = 30000 if d("total_steps") else args.total_steps
        args.skip_factor = 1e30 if d("skip_factor") else args.skip_factor
        args.lr = 4e-4 if d("lr") else args.lr
        args.min_lr = 0.1 * args.lr if d("min_lr") else args.min_lr
        args.warmup_steps = 1024 if d("warmup_steps") else args.warmup_steps
        args.wd_doctrine = args.wd_doctrine or "all"
    return args


def _dist_setup(device_arg):
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available() and device_arg != "cpu"
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world,
                                **({"device_id": dev} if cuda else {}))
    return rank, world, dev


def _peer_watch(args, rank, world):
    if args.peer_watch_s <= 0 or world == 1:
        return None
    from ..parallel.heartbeat import PeerWatch
    store = dist.distributed_c10d._get_default_store()
    return PeerWatch(store, rank, world, timeout=args.peer_watch_s)


def run(args):
    rank, world, dev = _dist_setup(args.device)
    master = rank == 0
    model_name, engine, T, gseqs, rungs, bounds, micro = RECIPES[args.recipe]
    engine = args.engine or engine
    T, gseqs, micro = args.seq_len or T, args.global_batch or gseqs, args.micro_batch or micro
    if args.ladder:
        rungs = tuple(tuple(int(x) for x in r.split(":")) for r in args.ladder.split(","))
    if args.bounds:
        bounds = tuple(float(x) for x in args.bounds.split(","))
    bounds = bounds[:max(0, len(rungs) - 1)]
    assert gseqs % world == 0, "global batch must divide over the ranks"
    local = gseqs // world
    micro = min(micro, local)
    cfg = preset(model_name, **json.loads(args.model_overrides))
    cfg.max_seq_len = max(cfg.max_seq_len, T)
    ladder = KLadder(rungs=rungs, bounds=bounds, probe_frac=args.probe_frac, probe_mult=args.probe_mult or None,
                     total_steps=args.total_steps)
    n_sid = len(rungs)
    rung_of = lambda sid: rungs[sid]
    if engine == "wave3d":
        C = rungs[0][0]
        assert all(c == C for c, _ in rungs), "the wavefront engine runs one chunk length"
        schedules, ekw = [k for _, k in rungs], dict(C=C)
    else:
        schedules, ekw = [uniform_chunks(T, c, min(c, k)) for c, k in rungs], {}
    exact_sid = None
    if args.val_exact_K > 0:                             # one more schedule, used by validation only
        exact_sid = len(schedules)
        schedules = schedules + ([args.val_exact_K] if engine == "wave3d"
                                 else [uniform_chunks(T, rungs[-1][0], min(rungs[-1][0], args.val_exact_K))])
    if args.sat_tau > 0:
        ekw["sat_tau"] = args.sat_tau
    ekw.update(json.loads(args.engine_kwargs))
    cooldown = args.cooldown_steps > 0
    tr = Trainer(cfg, schedules, seq_len=T, micro_batch=micro, local_batch=local, lr=args.lr, eps=args.eps,
                 weight_decay=args.weight_decay, decay_all=args.decay_all, max_norm=args.max_norm,
                 wd_doctrine=args.wd_doctrine or None, cooldown=cooldown, dm_accum=args.dm_accum, dm_lr=args.dm_lr,
                 optimizer=args.optimizer, device=dev, autocast_bf16=not args.fp32 and dev.type == "cuda",
                 use_graphs=not args.no_graphs, seed=args.seed, engine=engine, engine_kwargs=ekw,
                 rank_outlier_factor=args.rank_outlier_factor, rank_outlier_max=args.rank_outlier_max,
                 peer_watch=_peer_watch(args, rank, world))
    if args.lr_gov and hasattr(tr.engine, "track_rho"):
        tr.engine.track_rho = True                       # before the first step: the graphs record it
    skip = SkipRule(skip_factor=args.skip_factor, grace_steps=args.skip_grace_steps, gn_hard=args.gn_hard)
    clip = CalibratedClip(max_norm=args.max_norm, clip_mult=args.clip_mult, grace_steps=args.skip_grace_steps)
    gov, creep, inject = ChainRhoGovernor(), CreepDetector(), FaultInjector()
    rewind = RewindGovernor(window=args.rewind_window, skip_thresh=args.rewind_skip_thresh, ring=args.rewind_ring,
                            snap_interval=args.snap_interval, lookback=args.rewind_lookback,
                            max_rewinds=args.rewind_max, seed=args.seed,
                            log_path=os.path.join(args.out_dir, "rewind_events.jsonl") if master else None)
    log = MetricsLogger(args.out_dir, enabled=master, wandb_project=args.wandb_project,
                        wandb_name=os.path.basename(os.path.normpath(args.out_dir)), wandb_config=vars(args))
    capt_seen = set()
    writer = AsyncCheckpointWriter() if args.async_ckpt and master else None
    step, applied, seed_offset, tokens_seen = 0, 0, 0, 0
    hybrid = hasattr(tr.opt, "dm")
    # the ctx operators: what the sharpness-aware step perturbs
    sam_params = [p for n, p in tr.model.named_parameters() if "w_kctx" in n or "w_vctx" in n] if args.sam else []
    tel_x = None

    def checkpoint_now():
        return build_checkpoint(tr.model, tr.opt.trunk if hybrid else tr.opt, step=step, applied=applied,
                                extra=extra_state(), optimizer_dm=tr.opt.dm if hybrid else None)

    def load_optimizer(ck):
        """Optimizer state of a checkpoint into the current group layout; a cooldown starts its moments fresh."""
        from ..parallel.hybrid_optim import regroup_state
        if cooldown or "optimizer" not in ck:
            return
        halves = [(tr.opt.trunk, "optimizer"), (tr.opt.dm, "optimizer_dm")] if hybrid else [(tr.opt, "optimizer")]
        for o, key in halves:
            sd = ck.get(key) or ck["optimizer"]          # a one-optimizer checkpoint feeds both halves
            groups = o.param_groups if hasattr(o, "layout") else o.opt.param_groups
            o.load_state_dict(regroup_state(sd, tr.model, groups, args.weight_decay))

    def extra_state():
        return {**skip.state_dict(), **clip.state_dict(), **rewind.state_dict(), "seed_offset": seed_offset,
                "tokens": tokens_seen, "arch": "dualmod", "engine": engine, "engine_kwargs": ekw,
                "wb_tick": log.tick, "recipe": args.recipe}

    def restore(ck):
        nonlocal step, applied, seed_offset, tokens_seen
        with torch.no_grad():
            tr.model.load_state_dict(ck["model"])
        load_optimizer(ck)
        tr.engine.pack()
        skip.load_state_dict(ck)
        clip.load_state_dict(ck)
        step, applied = int(ck["step"]) + 1, int(ck.get("applied", ck["step"]))
        seed_offset, tokens_seen = int(ck.get("seed_offset", 0)), int(ck.get("tokens", 0))

    resume = os.path.join(args.out_dir, "ckpt_latest.pt") if args.resume == "auto" else args.resume
    if resume and os.path.exists(resume):
        ck = load_checkpoint(resume)
        restore(ck)
        rewind.load_state_dict(ck)
        log.tick = int(ck.get("wb_tick", 0))
        if master:
            print(f"resumed from {resume} at step {step}", flush=True)
    cd_start = applied                                   # a cooldown counts applied steps from here

    def make_stream(start, seed):
        if args.synthetic or not args.data_bin:
            syn = SyntheticStream(cfg.vocab_size, T, local, rank=rank, seed=seed)
            return (syn.block(s) for s in range(start, 1 << 62))
        return memmap_stream(args.data_bin, T, local, rank, world, start_step=start, seed=seed)

    stream = make_stream(step, args.seed + seed_offset)
    val_stream = None
    if args.val_every:
        val_stream = [next(make_stream(10 ** 9 + i, args.seed + 7)) if not args.val_bin else None
                      for i in range(args.val_batches)]
        if args.val_bin:
            g = memmap_stream(args.val_bin, T, micro, rank, world, seed=args.seed)
            val_stream = [next(g) for _ in range(args.val_batches)]

    def validate(sid):
        tot = torch.zeros((), dtype=torch.float32, device=dev)
        for blk in val_stream:
            b = blk[:micro].to(dev)
            tot += tr.engine.forward(b[:, :T], b[:, 1:T + 1], sid=sid, train=False)
        tot /= len(val_stream)
        if world > 1:
            dist.all_reduce(tot)
            tot /= world
        return tot.item()

    t_last, final_loss = time.time(), float("nan")
    while step < args.total_steps:
        if cooldown and applied - cd_start >= args.cooldown_steps:
            if master:
                save_persist(args.out_dir, tr.model, step, name=f"snap_cooldown_{step:06d}.pt")
                print(f"cooldown done after {applied - cd_start} applied steps", flush=True)
            break
        sid, is_probe = ladder.sid_of(step)
        sid = min(sid, n_sid - 1)
        lr = cosine_lr(step, args.total_steps, args.warmup_steps, args.lr, args.min_lr) * (gov.mult if args.lr_gov else 1.0)
        if cooldown:                                     # linear in applied steps
            prog = min(1.0, (applied - cd_start) / max(1, args.cooldown_steps))
            lr = args.cooldown_lr_start + (args.cooldown_lr_end - args.cooldown_lr_start) * prog
        thr = skip.threshold(is_probe)
        if inject.spiked(step, rewind.count) or step in inject.nans:
            thr = 1e-30                                      # the injected spike: every finite norm exceeds this
        tr.opt.skip_norm, tr.opt.max_norm = thr, clip.threshold(is_probe)
        tr.local_norm_factor = inject.rank_factor(step, rank)
        t0 = time.time()
        do_sam = bool(sam_params) and not is_probe and step % args.sam_every == 0
        if do_sam:
            loss = tr.sam_step(next(stream), sam_params, args.sam_rho, sid=sid, lr=lr)
        else:
            loss = tr.step(next(stream), sid=sid, lr=lr)
        ctrl = tr.opt.ctrl.tolist()
        gn, skipped = ctrl[0], ctrl[2] > 0.5
        # a bounded cross-GPU wait of the optimizer kernels that ran out voids this and every later step
        # (the status word is sticky): name the peer and the phase, keep the newest resident snapshot, stop
        wait_code = ctrl[7] if len(ctrl) > 7 else 0.0
        if wait_code or (skipped and hasattr(tr.opt, "check_status")):
            try:
                tr.opt.check_status(int(wait_code)) if len(ctrl) > 7 else tr.opt.check_status()
            except RuntimeError as e:
                if rewind.ring:
                    snap_step, ck = rewind.ring[-1]
                    path = os.path.join(args.out_dir, f"ckpt_emergency_rank{rank}.pt")
                    save_atomic(ck, path)
                    print(f"[rank {rank}] step {step}: {e}; resident snapshot of step {snap_step} -> {path}", flush=True)
                else:
                    print(f"[rank {rank}] step {step}: {e}; no resident snapshot (resume from ckpt_latest.pt)", flush=True)
                if writer is not None:
                    writer.close()
                log.close()
                raise
        gn_seen, loss_seen = inject.apply(step, gn, loss, rewind.count)
        step_ms = (time.time() - t0) * 1e3
        if world > 1:
            lt = torch.tensor(loss, device=dev)
            dist.all_reduce(lt)
            loss = lt.item() / world
        rewarmed = skip.update(gn_seen, loss_seen, is_probe, skipped)
        if (not math.isfinite(gn) or gn > 1e3) and hasattr(tr.engine, "debug_scan"):
            # every rank scans its own persistent buffers (a residue on one rank only would otherwise go unseen)
            bad = tr.engine.debug_scan()[:6]
            found = [None] * world
            if world > 1:
                dist.all_gather_object(found, (rank, bad))
            else:
                found = [(0, bad)]
            if master:
                print(f"DEBUG-SCAN step {step}: gn {gn:.3g}; non-finite buffers by rank: "
                      f"{[(r, b) for r, b in found if b] or 'none'}", flush=True)
        if not skipped:
            applied += 1
            clip.update(gn, is_probe)
            final_loss = loss
        if args.lr_gov and step >= args.warmup_steps:
            # the engine's largest carried-gradient amplification of this backward when it tracks it
            # (1-step lag), else the norm against its running level
            rho = float(tr.engine.chain_rho_max) if getattr(tr.engine, "track_rho", False) else 0.0
            e = skip.ema[is_probe]
            gov.update(rho if rho > 0 else (gn_seen / e if e else 1.0))
        creeping = creep.update(gn) if not skipped else False
        tokens_seen += gseqs * T
        c_r, k_r = rung_of(sid)
        rec = {"train/loss": loss, "train/lr": lr, "train/grad_norm": gn, "train/sid": sid, "train/K": k_r,
               "train/c": c_r, "train/phase": ladder.phase_of(step), "train/is_probe": is_probe,
               "train/clip_event": ctrl[1] < 1.0, "train/clip_thr": tr.opt.max_norm, "train/skipped": skipped,
               "train/skipped_total": skip.skipped_total, "train/rank_excl": tr.rank_excluded,
               "train/applied": applied, "train/tokens": tokens_seen, "train/step_ms": step_ms,
               "train/breaker": rewarmed, "train/creep": creeping, "train/gov_mult": gov.mult}
        kind = "probe" if is_probe else "base"
        rec[f"{kind}/loss"], rec[f"{kind}/grad_norm"] = loss, gn
        if is_probe and skip.ema[False]:
            rec["probe/gn_ratio_vs_base"] = gn / max(skip.ema[False], 1e-9)
        for s_, sec in getattr(tr.engine, "capture_seconds", {}).items():
            if s_ not in capt_seen and sec > 0:          # once per rung, when its graphs have been recorded
                capt_seen.add(s_)
                rec[f"engine/capture_K{rung_of(s_)[1]}_s"] = sec
        if args.sam:
            rec["train/sam_active"] = int(do_sam)
            if do_sam:
                rec["train/sam_sharp"] = tr.sam_sharpness
        if hybrid:
            rec["train/dm_stepped"], rec["train/dm_grad_norm"] = ctrl[3] > 0.5, tr.opt.last_dm_norm
        if dev.type == "cuda":
            rec["train/step_peak_gb"] = torch.cuda.max_memory_allocated(dev) / 2 ** 30
            rec["train/gpu_reserved_gb"] = torch.cuda.memory_reserved(dev) / 2 ** 30
        if val_stream is not None and step % args.val_every == 0 and step > 0:
            base_sid = min(ladder.phase_of(step), n_sid - 1)
            rec["val/loss"], rec["val/base_K"] = validate(base_sid), rung_of(base_sid)[1]
            rec["val/loss_deep"] = validate(n_sid - 1)
            rec["val/base_minus_deep"] = rec["val/loss"] - rec["val/loss_deep"]
            if exact_sid is not None:
                rec["val/loss_exact"] = validate(exact_sid)
                rec[f"val/base_minus_k{args.val_exact_K}"] = rec["val/loss"] - rec["val/loss_exact"]
        if (args.eager_val_every and exact_sid is not None and val_stream is not None and step > 0
                and step % args.eager_val_every == 0):
            # same rows through the engine at the exact setting and through the eager scan: the two agree to
            # rounding when the engine is healthy.  The eager scan sees only a prefix slice, so the engine's
            # loss is taken on the same positions (targets beyond the slice are masked).
            n_tok, rows_x = min(T, args.eager_val_len), min(micro, args.eager_val_rows)
            b = val_stream[0][:micro].to(dev)
            tg = b[:, 1:T + 1].clone()
            tg[rows_x:] = -1
            tg[:, n_tok:] = -1
            rec["val/loss_engine_xcheck"] = float(tr.engine.forward(b[:, :T], tg, sid=exact_sid, train=False))
            mode, tr.model.cfg.attn_mode = tr.model.cfg.attn_mode, "sequential"
            was = tr.model.training
            tr.model.eval()
            with torch.no_grad(), torch.autocast(dev.type, dtype=torch.bfloat16, enabled=dev.type == "cuda" and not args.fp32):
                lg = tr.model(b[:rows_x, :n_tok])[0]
            rec["val/loss_eager_xcheck"] = float(torch.nn.functional.cross_entropy(
                lg.float().flatten(0, 1), b[:rows_x, 1:n_tok + 1].reshape(-1)))
            tr.model.train(was)
            tr.model.cfg.attn_mode = mode
        if args.telemetry_every and step % args.telemetry_every == 0 and master:
            from .curvature import gate_stats_layerwise
            if tel_x is None:                            # one fixed batch, so the dials compare step to step
                tel_x = next(make_stream(10 ** 9 + 99, args.seed))[:2, :min(T, 256)].to(dev)
            mode, tr.model.cfg.attn_mode = tr.model.cfg.attn_mode, "sequential"
            rec.update(gate_stats_layerwise(tr.model, tel_x))
            tr.model.cfg.attn_mode = mode
        if args.curv_every and step % args.curv_every == 0 and step > 0:
            from .curvature import ctx_top_eig, layer_grad_norms
            rec.update(layer_grad_norms(tr.model, tr.opt.grad_buffers(), tr.opt if getattr(tr.opt, "use_kernel", False) else None))
            if master:
                blk = next(make_stream(10 ** 9 + 77, args.seed))[:2, :args.curv_len + 1].to(dev)
                mode, tr.model.cfg.attn_mode = tr.model.cfg.attn_mode, "sequential"
                rec["curv/ctx_top_eig"] = ctx_top_eig(tr.model, blk[:, :-1], blk[:, 1:], n_iter=3)
                tr.model.cfg.attn_mode = mode
        log.log(step, **rec)
        if master and (step % args.log_every == 0 or skipped):
            dt = time.time() - t_last
            t_last = time.time()
            print(f"step {step} loss {loss:.4f} gn {gn:.3f} lr {lr:.2e} K {k_r}{' probe' if is_probe else ''}"
                  f"{' SKIPPED' if skipped else ''} {step_ms:.0f} ms", flush=True)
        # ---- rewind -------------------------------------------------------------------------------------
        if args.auto_rewind:
            rewind.note(step, skipped)
            if rewind.want_snapshot(step):
                ck = checkpoint_now()
                rewind.add_snapshot(step, AsyncCheckpointWriter.to_cpu(ck))       # resident, in host memory
            if rewind.wedged():
                pick = rewind.choose(step, extra={"skips_in_window": sum(rewind.recent), "rho_ema": gov.rho_ema or 0.0})
                if pick is None:
                    if master:
                        print(f"[auto-rewind] giving up at step {step}: rewind limit reached", flush=True)
                    break
                snap_step, ck, new_seed = pick
                restore(ck)
                seed_offset = new_seed - args.seed
                stream = make_stream(step, new_seed)
                gov.reset()
                if master:
                    print(f"[auto-rewind #{rewind.count}] wedged -> snapshot of step {snap_step}, seed {new_seed}",
                          flush=True)
                continue
        # ---- checkpoints --------------------------------------------------------------------------------
        if args.ckpt_every and step > 0 and step % args.ckpt_every == 0:
            ck = checkpoint_now()                            # collective
            if master:
                path = os.path.join(args.out_dir, "ckpt_latest.pt")
                writer.submit(ck, path) if writer is not None else save_atomic(ck, path)
        if args.persist_every and step > 0 and step % args.persist_every == 0 and master:
            save_persist(args.out_dir, tr.model, step)
        step += 1
    if writer is not None:
        writer.close()
    if master:
        print(f"FINAL step {step} applied {applied} skipped {skip.skipped_total} rewinds {rewind.count} "
              f"loss {final_loss:.4f}", flush=True)
    log.close()
    if hasattr(tr.opt, "close"):
        tr.opt.close()
    return {"step": step, "applied": applied, "skipped": skip.skipped_total, "rewinds": rewind.count,
            "loss": final_loss}


def main(argv=None):
    out = run(parse_args(argv))
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
