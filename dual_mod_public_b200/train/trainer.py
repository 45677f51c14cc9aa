"""Training step driver: model + engine + data-parallel optimizer behind one call.

`Trainer.step(tokens)` is the call a user makes per optimizer step: it takes the
rank's token block from (pinned) host memory, copies each micro-batch to the
device, runs the engine's forward + reverse-scan backward at the schedule id of
the step, lets finished layer buckets start their reduce-scatter, then runs the
fused reduce + clip + AdamW + all-gather kernel, refreshes the bf16 weight packs
and returns the loss read back to the host.

Reference parity: the step bodies of lm/train_340m/train_flagship.py:864-1045
(engine.train_step -> finish_grads -> clip -> skip -> opt.step) and
lm/train_1p3b/train_hero_wave3d.py:848-997, without their logging and governors,
which live in `governors.py` and wrap this class.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ..engines.wavescan import WaveScanEngine
from ..models import DualModLM
from ..parallel.fused_optim import FusedDPAdamW, NcclAdamW, default_buckets
from ..parallel.hybrid_optim import (DM_NAMES, HybridAdamW, matches, optimizer_groups, recall_only,
                                     restrict_buckets)


class Trainer:
    def __init__(self, cfg, schedules, *, seq_len, micro_batch, local_batch, lr=3e-4,
                 betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, decay_all=False, max_norm=1.0,
                 skip_norm=0.0, optimizer="fused", device=None, autocast_bf16=True, use_graphs=True,
                 overlap_buckets=True, process_group=None, seed=1337, engine="wavescan",
                 engine_kwargs=None, model=None, rank_outlier_factor=0.0, rank_outlier_max=1, peer_watch=None,
                 wd_doctrine=None, cooldown=False, dm_accum=1, dm_lr=None):
        assert local_batch % micro_batch == 0, "local batch must be a whole number of micro-batches"
        self.device = torch.device(device) if device is not None else torch.device(
            "cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.cfg, self.T = cfg, seq_len
        self.micro_batch, self.accum = micro_batch, local_batch // micro_batch
        self.world = dist.get_world_size(process_group) if dist.is_available() and dist.is_initialized() else 1
        if model is None:
            torch.manual_seed(seed)
            model = DualModLM(cfg)
        self.model = model.to(self.device)
        # wd_doctrine: "split" (matrices decay), "all", "branch" (grown-branch parameters at 10x the decay);
        # cooldown: only the write-law parameters move; dm_accum / dm_lr: two-speed optimizer
        # (parallel/hybrid_optim.py)
        doctrine = wd_doctrine or ("all" if decay_all else "split")
        common = dict(lr=lr, betas=betas, eps=eps, max_norm=max_norm, skip_norm=skip_norm,
                      grad_accum=self.accum, process_group=process_group)

        def make(only):
            groups = optimizer_groups(self.model, doctrine, weight_decay, only=only)
            if cooldown:
                groups = recall_only(groups, self.model)
            if optimizer == "fused":
                owned = [p for g in groups for p in g["params"]]
                return FusedDPAdamW(groups, restrict_buckets(default_buckets(self.model), owned),
                                    device=self.device, **common)
            return NcclAdamW(groups, **common)

        if dm_accum > 1 or dm_lr is not None:
            is_dm = lambda n: matches(n, DM_NAMES)
            self.opt = HybridAdamW(make(lambda n: not is_dm(n)), make(is_dm), dm_accum=dm_accum, dm_lr=dm_lr)
        else:
            self.opt = make(None)
        # per-rank rejection needs every rank's LOCAL norm before anything is reduced: no early buckets then
        self.rank_outlier = (rank_outlier_factor, rank_outlier_max) if rank_outlier_factor > 0 and self.world > 1 else None
        if self.rank_outlier is not None and isinstance(self.opt, HybridAdamW):
            raise NotImplementedError("per-rank outlier rejection reads one flat gradient array; the two-speed optimizer has two")
        self.group, self.rank_excluded = process_group, 0
        self.local_norm_factor = 1.0
        self.overlap = (overlap_buckets and optimizer == "fused" and self.opt.use_kernel and self.world > 1
                        and self.rank_outlier is None)
        self._side = torch.cuda.Stream(device=self.device) if self.overlap else None
        self._last_micro = False
        self.trace = None                      # set by `trace_overlap`: CUDA events of one step's gradient exchange
        kw = dict(engine_kwargs or {})
        common_e = dict(device=self.device, autocast_bf16=autocast_bf16, use_graphs=use_graphs,
                        grads=self.opt.grad_buffers(),
                        on_layer_grads_final=self._layer_done if self.overlap else None)
        if engine == "wavescan":
            # schedules: list of cell lists [(pos0, c, sweeps), ...], one per schedule id
            self.engine = WaveScanEngine(self.model, schedules, micro_batch, seq_len, **common_e, **kw)
        else:
            # schedules: the K-ladder (sweep counts) of the wavefront engine, one per schedule id
            from ..engines.wave3d import Wave3DEngine
            self.engine = Wave3DEngine(self.model, schedules, micro_batch, seq_len, **common_e, **kw)
        # optional host-side check that every peer is about to run the same step (parallel/heartbeat.py)
        self.peer_watch = peer_watch
        self.engine.pack()
        self.steps_done = 0
        self._loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        self._loss_host = torch.zeros((), dtype=torch.float32).pin_memory() if self.device.type == "cuda" \
            else torch.zeros((), dtype=torch.float32)

    # bucket b of `default_buckets` : 0 = head/final norm, 1 + (L-1-li) = layer li, last = embedding
    def _layer_done(self, li):
        if not self._last_micro:
            return
        b = 0 if li < 0 else 1 + (self.cfg.n_layers - 1 - li)
        cur = torch.cuda.current_stream(self.device)
        self._side.wait_stream(cur)
        if self.trace is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            ev[0].record(self._side)
            self.opt.bucket_ready(b, stream=self._side)
            ev[1].record(self._side)
            self.trace["buckets"].append((b, ev[0], ev[1]))
            return
        self.opt.bucket_ready(b, stream=self._side)

    def trace_overlap(self, tokens, sid=0, lr=None):
        """One optimizer step with CUDA events around the last micro-batch's backward, every bucket's early
        reduce-scatter (second stream) and the fused optimizer step.  Returns a dict of milliseconds relative to
        the start of the last micro-batch: `backward_end`, `buckets` = [(bucket, start, end)], `wait_start` (the main
        stream starts waiting for the second stream), `opt_start`, `opt_end`, and the derived `reduce_total`
        (sum of the buckets' kernel times), `reduce_exposed` (time the main stream waited for the last buckets
        after its own backward was done) and `step_kernel` (the fused optimizer kernel)."""
        if not self.overlap:
            raise RuntimeError("no early buckets in this configuration (one rank, NCCL optimizer or per-rank rejection)")
        E = lambda: torch.cuda.Event(enable_timing=True)
        cur = torch.cuda.current_stream(self.device)
        mb, T = self.micro_batch, self.T
        self.opt.zero_grad()
        self._loss_acc.zero_()
        for a in range(self.accum):
            blk = tokens[a * mb:(a + 1) * mb].to(self.device, non_blocking=True)
            self._last_micro = a == self.accum - 1
            if self._last_micro:
                self.trace = {"buckets": []}
                t0 = E()
                t0.record(cur)
            self._loss_acc += self.engine.train_step(blk[:, :T], blk[:, 1:T + 1], sid=sid)
        t_bwd, t_wait, t_opt0, t_opt1 = E(), E(), E(), E()
        t_bwd.record(cur)
        t_wait.record(cur)
        cur.wait_stream(self._side)
        t_opt0.record(cur)
        self.opt.step(lr=lr)
        t_opt1.record(cur)
        self.engine.pack()
        self.steps_done += 1
        torch.cuda.synchronize(self.device)
        tr, self.trace = self.trace, None
        ms = lambda e: t0.elapsed_time(e)
        buckets = [(b, ms(e0), ms(e1)) for b, e0, e1 in tr["buckets"]]
        out = {"backward_end": ms(t_bwd), "buckets": buckets, "wait_start": ms(t_wait), "opt_start": ms(t_opt0),
               "opt_end": ms(t_opt1)}
        out["reduce_total"] = sum(e - s for _, s, e in buckets)
        out["reduce_exposed"] = out["opt_start"] - out["wait_start"]
        out["step_kernel"] = out["opt_end"] - out["opt_start"]
        return out

    def accumulate(self, tokens, sid=0, final=True):
        """Zero the gradients, then forward + backward over the rank's micro-batches.  final=False: a pass
        whose gradients will be recomputed (no bucket may start its reduction yet)."""
        mb, T = self.micro_batch, self.T
        self.opt.zero_grad()
        self._loss_acc.zero_()
        nb = self.device.type == "cuda"
        for a in range(self.accum):
            blk = tokens[a * mb:(a + 1) * mb].to(self.device, non_blocking=nb)   # one contiguous H2D copy
            idx, tgt = blk[:, :T], blk[:, 1:T + 1]
            self._last_micro = final and a == self.accum - 1
            self._loss_acc += self.engine.train_step(idx, tgt, sid=sid)

    def apply(self, lr=None):
        """The optimizer step on what `accumulate` left, then the refreshed weight packs."""
        if self._side is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._side)
        keep_skip = self.opt.skip_norm
        if self.rank_outlier is not None:
            self._reject_outlier_ranks()
        self.opt.step(lr=lr)
        self.opt.grad_scale_override, self.opt.skip_norm = None, keep_skip
        self.engine.pack()
        self.steps_done += 1

    def _read_loss(self, read_loss):
        if not read_loss:
            return self._loss_acc / self.accum
        nb = self.device.type == "cuda"
        self._loss_host.copy_(self._loss_acc / self.accum, non_blocking=nb)
        if nb:
            torch.cuda.current_stream(self.device).synchronize()
        return float(self._loss_host)

    def step(self, tokens, sid=0, lr=None, read_loss=True):
        """tokens: [local_batch, T+1] int64 (host, ideally pinned) — inputs are
        tokens[:, :-1], targets tokens[:, 1:].  Returns the mean loss over the rank's
        micro-batches as a Python float (or the device tensor when read_loss=False)."""
        if self.peer_watch is not None:
            self.peer_watch.sync(self.steps_done)            # raises PeerLost before anything is launched
        self.accumulate(tokens, sid)
        self.apply(lr)
        return self._read_loss(read_loss)

    def sam_step(self, tokens, params, rho, sid=0, lr=None, read_loss=True):
        """Sharpness-aware step (lm/train_340m/train_flagship.py:902-934): a first backward gives the mean
        gradient g of `params`; they move to theta + rho g / |g|, a second backward gives the gradient the
        optimizer uses, and theta comes back by copy (bit-exact, so ranks stay identical).  Also sets
        `sam_sharpness` = <g / |g|, g' - g> / rho, the curvature along the gradient."""
        if self.peer_watch is not None:
            self.peer_watch.sync(self.steps_done)
        G = self.opt.grad_buffers()
        self.accumulate(tokens, sid, final=False)
        with torch.no_grad():
            g = torch.cat([G.get(p).reshape(-1).float() for p in params])
            if self.world > 1:
                dist.all_reduce(g, group=self.group)
            g /= self.world * self.accum
            gnorm = g.norm() + 1e-12
            saved = [p.detach().clone() for p in params]
            o = 0
            for p in params:
                p.add_(g[o:o + p.numel()].view_as(p).to(p.dtype), alpha=float(rho / gnorm))
                o += p.numel()
        self.engine.pack()
        # no bucket starts its reduction during this pass: g2 below is read from the flat array on the main
        # stream and must still be this rank's plain local gradient (the fused step reduces every bucket)
        self.accumulate(tokens, sid, final=False)
        with torch.no_grad():
            g2 = torch.cat([G.get(p).reshape(-1).float() for p in params]) / (self.world * self.accum)
            dot = (g2 * g).sum()
            if self.world > 1:
                dist.all_reduce(dot, group=self.group)
            self.sam_sharpness = float((dot - (g * g).sum()) / (gnorm * rho))
            for p, sv in zip(params, saved):
                p.copy_(sv)
        self.apply(lr)
        return self._read_loss(read_loss)

    def _reject_outlier_ranks(self):
        """All-gather the local gradient norms; ranks far above the median zero their gradients and the
        average is taken over the ranks kept (the same mask on every rank); too many outliers void the
        step through the optimizer's skip predicate (train_hero_wave3d.py:894-920)."""
        from .governors import rank_outlier_mask
        flat = self.opt.grad_buffers().flat if not hasattr(self.opt, "flat_grads") else self.opt.flat_grads
        mine = flat.norm().float().reshape(1) * self.local_norm_factor     # factor != 1: host-side fault injection
        allv = [torch.zeros_like(mine) for _ in range(self.world)]
        dist.all_gather(allv, mine, group=self.group)
        norms = [float(v) for v in torch.cat(allv).tolist()]
        keep, void = rank_outlier_mask(norms, *self.rank_outlier)
        self.rank_excluded = len(keep) - sum(keep)
        if not keep[dist.get_rank(self.group)]:
            flat.zero_()
        if void:
            self.opt.skip_norm = 1e-30                       # every finite norm exceeds it: the step is void
        elif self.rank_excluded:
            self.opt.grad_scale_override = 1.0 / (sum(keep) * self.accum)

    def h2d_bytes_per_step(self):
        return self.micro_batch * self.accum * (self.T + 1) * 8

    def d2h_bytes_per_step(self):
        return 4
