"""Optimizer group doctrines and the two-speed (trunk / Dual-Mod) optimizer.

`optimizer_groups` names the weight-decay layouts the 340M trainer of the reference
switches between (lm/train_340m/train_flagship.py:616-660): matrices decay and 1-D
parameters do not ("split"), everything decays ("all"), and the grown-branch
parameters additionally sit in a group of their own with 10x the decay ("branch").
`recall_only` is the cooldown of the same file (lines 662-690): only the write-law
parameters move, everything else keeps its gradient but gets a learning-rate
multiplier of zero.

`HybridAdamW` is the hybrid recipe of lines 628-655 and 1005-1060: the trunk steps
every iteration on its own clipped norm; the Dual-Mod parameters accumulate their
gradient, unclipped, over `dm_accum` iterations and then take one step on the mean,
with their own learning rate and clip; an iteration the trunk skips voids the
accumulation.  Both halves are ordinary optimizers of this package (fused kernel or
the library chain) over disjoint parameter sets, so each half keeps its flat
buffers, its reduce-scatter and its state dict.
"""

from __future__ import annotations

import math

import torch

from ..engines.gradbuf import GradBuffers, unique_params

BRANCH = ("v_pre", "v_map", "v_gate", "v_comb", "k_pre")
DM_NAMES = ("w_kctx", "w_vctx", "w_gk", "w_gv", "norm_ctx", "v_gain", "ctx_gain", "k_gain") + BRANCH
RECALL = ("w_kctx", "w_vctx", "v_gate", "v_map", "w_gk", "w_gv", "norm_ctx", "k_gain", "v_gain", "ctx_gain")


def named_unique(model):
    seen, out = set(), []
    for n, p in model.named_parameters():
        if id(p) not in seen:
            seen.add(id(p))
            out.append((n, p))
    return out


def matches(name, tags):
    return any(t in name for t in tags)


def optimizer_groups(model, doctrine="split", weight_decay=0.1, branch_mult=10.0, only=None, lr_mult=1.0):
    """Parameter groups ({"params", "weight_decay", "lr_mult"}) for one optimizer.

    doctrine: "split" | "all" | "branch".  only: predicate on the parameter name selecting the
    subset this optimizer owns (None = every parameter)."""
    named = [(n, p) for n, p in named_unique(model) if only is None or only(n)]
    if doctrine == "all":
        groups = [([p for _, p in named], weight_decay)]
    else:
        br = [(n, p) for n, p in named if doctrine == "branch" and matches(n, BRANCH)]
        bids = {id(p) for _, p in br}
        rest = [(n, p) for n, p in named if id(p) not in bids]
        groups = [([p for _, p in rest if p.dim() >= 2], weight_decay),
                  ([p for _, p in rest if p.dim() < 2], 0.0)]
        if br:
            groups.append(([p for _, p in br], weight_decay * branch_mult))
    return [{"params": ps, "weight_decay": wd, "lr_mult": lr_mult} for ps, wd in groups if ps]


def recall_only(groups, model):
    """Cooldown: split every group into the write-law parameters (unchanged) and the rest (lr_mult 0, so
    neither the step nor the decay moves them)."""
    name_of = {id(p): n for n, p in named_unique(model)}
    out = []
    for g in groups:
        live = [p for p in g["params"] if matches(name_of[id(p)], RECALL)]
        frozen = [p for p in g["params"] if not matches(name_of[id(p)], RECALL)]
        if live:
            out.append({**g, "params": live})
        if frozen:
            out.append({**g, "params": frozen, "lr_mult": 0.0})
    return out


def restrict_buckets(buckets, params):
    """The bucket list with only `params` kept (empty buckets dropped, order preserved)."""
    ids = {id(p) for p in params}
    out = [[p for p in b if id(p) in ids] for b in buckets]
    return [b for b in out if b]


class HybridAdamW:
    """trunk: steps every iteration.  dm: steps every `dm_accum` iterations on the mean gradient.

    Same surface as the single optimizers as far as the trainers use it: `grad_buffers`, `zero_grad`,
    `step`, `ctrl`, `skip_norm`, `max_norm`, `grad_scale_override`, `state_dict`, `load_state_dict`.
    `ctrl` after a step = [trunk gradient norm, trunk clip coefficient, skipped, 1 if the Dual-Mod half
    stepped]; the skip decision (and the EMA a caller keeps for it) runs on the trunk's norm, the norm of
    the Dual-Mod half's last step is `last_dm_norm`."""

    use_kernel = False                                   # no early bucket reduction through this wrapper

    def __init__(self, trunk, dm, dm_accum=1, dm_lr=None, dm_max_norm=None):
        assert dm_accum >= 1
        self.trunk, self.dm, self.dm_accum = trunk, dm, dm_accum
        self.dm_lr = dm_lr
        self.dm_max_norm = dm.max_norm if dm_max_norm is None else dm_max_norm
        self.dm_iter = 0
        self.dm_steps = 0
        self.last_dm_norm = 0.0
        self._base_accum = dm.grad_accum
        dm.grad_accum = self._base_accum * dm_accum
        dm.skip_norm = 0.0                               # the trunk's decision governs both halves
        self.lr = trunk.lr
        self.ctrl = torch.zeros(4, dtype=torch.float32, device=trunk.ctrl.device)
        tg, dg = trunk.grad_buffers(), dm.grad_buffers()
        merged = GradBuffers.__new__(GradBuffers)
        merged.order = unique_params(list(tg.order) + list(dg.order))
        merged.flats, merged.layouts = list(tg.flats) + list(dg.flats), list(tg.layouts) + list(dg.layouts)
        merged.buf = {**tg.buf, **dg.buf}
        merged.flat = tg.flat
        self._grads = merged
        self._dm_flats = list(dg.flats)

    # the trainers set these on "the optimizer": they are the trunk's
    skip_norm = property(lambda s: s.trunk.skip_norm, lambda s, v: setattr(s.trunk, "skip_norm", v))
    max_norm = property(lambda s: s.trunk.max_norm, lambda s, v: setattr(s.trunk, "max_norm", v))
    grad_scale_override = property(lambda s: s.trunk.grad_scale_override,
                                   lambda s, v: setattr(s.trunk, "grad_scale_override", v))

    def grad_buffers(self):
        return self._grads

    def zero_grad(self):
        self.trunk.zero_grad()
        if self.dm_iter == 0:
            self.dm.zero_grad()

    def step(self, lr=None):
        lr = self.lr if lr is None else lr
        t = self.trunk.step(lr=lr).tolist()              # host read: this recipe decides on the host
        gn_t, skipped = t[0], t[2] > 0
        self.dm_iter += 1
        stepped = 0.0
        if skipped or not math.isfinite(gn_t):
            for f in self._dm_flats:                     # a wild iteration voids the accumulation
                f.zero_()
            self.dm_iter = 0
        elif self.dm_iter >= self.dm_accum:
            self.dm.max_norm = self.dm_max_norm
            scale = lr / self.lr if self.lr > 0 else 1.0
            d = self.dm.step(lr=(self.dm_lr if self.dm_lr is not None else self.lr) * scale).tolist()
            self.last_dm_norm, self.dm_iter, stepped = d[0], 0, 1.0
            self.dm_steps += 1
        self.ctrl.copy_(torch.tensor([gn_t, t[1], float(skipped), stepped]))
        return self.ctrl

    def check_status(self):
        for o in (self.trunk, self.dm):
            if hasattr(o, "check_status"):
                o.check_status()

    def state_dict(self):
        return {"optimizer": self.trunk.state_dict(), "optimizer_dm": self.dm.state_dict(),
                "dm_steps": self.dm_steps}

    def load_state_dict(self, sd):
        self.trunk.load_state_dict(sd["optimizer"])
        if sd.get("optimizer_dm") is not None:
            self.dm.load_state_dict(sd["optimizer_dm"])
        # a partly accumulated Dual-Mod gradient is not saved: the accumulation restarts after a resume
        self.dm_iter, self.dm_steps = 0, sd.get("dm_steps", 0)
        for f in self._dm_flats:
            f.zero_()

    def close(self):
        for o in (self.trunk, self.dm):
            if hasattr(o, "close"):
                o.close()


def regroup_state(sd, model, new_groups, weight_decay=0.1):
    """Re-key an AdamW state dict (torch layout: state by parameter index in group order) that was saved
    under another group layout of the same model, so that a run may change its weight-decay doctrine or
    split off the Dual-Mod half on resume (lm/train_340m/train_flagship.py:712-766).  The old layout is
    recognised by its group sizes among the layouts `optimizer_groups` builds; parameters the old state
    does not hold start fresh.  Returns `sd` itself when the sizes already agree."""
    old_sizes = [len(g["params"]) for g in sd["param_groups"]]
    if old_sizes == [len(g["params"]) for g in new_groups]:
        return sd
    is_dm = lambda n: matches(n, DM_NAMES)
    for doctrine in ("split", "all", "branch"):
        for only in (None, lambda n: not is_dm(n), is_dm):
            cand = optimizer_groups(model, doctrine, weight_decay, only=only)
            if [len(g["params"]) for g in cand] == old_sizes:
                old_idx, i = {}, 0
                for g in cand:
                    for p in g["params"]:
                        old_idx[id(p)] = i
                        i += 1
                state, groups, j = {}, [], 0
                proto = {k: v for k, v in sd["param_groups"][0].items() if k != "params"}
                for g in new_groups:
                    ids = []
                    for p in g["params"]:
                        st = sd["state"].get(old_idx.get(id(p), -1))
                        if st is not None:
                            state[j] = st
                        ids.append(j)
                        j += 1
                    groups.append({**proto, "weight_decay": g.get("weight_decay", 0.0), "params": ids})
                return {"state": state, "param_groups": groups}
    raise ValueError(f"optimizer state with group sizes {old_sizes} matches no known layout of this model")
