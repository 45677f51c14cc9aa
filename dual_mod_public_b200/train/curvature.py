"""Curvature and per-layer gradient telemetry for the trainers.

`ctx_top_eig`: the top eigenvalue of the loss Hessian restricted to a parameter subset (by default the
context operators w_kctx / w_vctx), by power iteration on Hessian-vector products of the plain model
forward (double backward).  A rising value means the loss is sharpening along the context branch; the
340M trainer logs it at a coarse cadence as `curv/ctx_top_eig`.  Independent of the engines, best effort:
any failure returns nan.

`layer_grad_norms`: `gradnorm/L%02d` = the gradient norm of every block, read from the flat gradient
buffers after a step.

Reference parity: lm/train_340m/train_flagship.py:176-208 (`ctx_top_eig`), :211-294 (telemetry keys).
"""

from __future__ import annotations

import torch


def ctx_params(model):
    """The context operators' weights of every block."""
    out = []
    for blk in model.blocks:
        for name in ("w_kctx", "w_vctx"):
            mod = getattr(blk.attn, name, None)
            if mod is not None:
                out += [p for p in mod.parameters() if p.dim() >= 2]
    return out


def ctx_top_eig(model, xb, yb, params=None, n_iter=5, seed=0):
    """Power iteration: v <- H v / |H v| on the Hessian of the loss w.r.t. `params`; returns v . H v of the
    last iterate (a Python float; nan on failure).  `requires_grad` flags and train / eval mode are restored."""
    params = list(params) if params is not None else ctx_params(model)
    if not params:
        return float("nan")
    was_training = model.training
    flags = [(p, p.requires_grad) for p in model.parameters()]
    try:
        model.train()
        for p, _ in flags:
            p.requires_grad_(False)
        for p in params:
            p.requires_grad_(True)
        g = torch.Generator(device="cpu").manual_seed(seed)
        vs = [torch.randn(p.shape, generator=g).to(p) for p in params]
        norm = torch.sqrt(sum((v.float() ** 2).sum() for v in vs))
        vs = [v / (norm + 1e-12) for v in vs]
        eig = float("nan")
        for _ in range(n_iter):
            _, loss = model(xb, targets=yb)
            grads = torch.autograd.grad(loss.float(), params, create_graph=True)
            gv = sum((gr * v).sum() for gr, v in zip(grads, vs))
            hv = torch.autograd.grad(gv, params)
            eig = float(sum((h_ * v).sum() for h_, v in zip(hv, vs)))
            norm = torch.sqrt(sum((h_.float() ** 2).sum() for h_ in hv))
            vs = [(h_ / (norm + 1e-12)).detach() for h_ in hv]
        return eig
    except Exception:
        return float("nan")
    finally:
        for p, r in flags:
            p.requires_grad_(r)
        model.train(was_training)


@torch.no_grad()
def layer_grad_norms(model, grads, opt=None):
    """{"gradnorm/L00": ..., ...}: norm of each layer's gradient as the optimizer step saw it (the mean over
    ranks and micro-batches).  `grads`: a `GradBuffers`-like object with `.get(param)`.  `opt`: the sharded
    optimizer, when there is one and more than one rank: after its step only the slice a rank OWNS of each
    bucket holds the reduced mean (the rest still holds that rank's raw local sums), so every rank sums the
    squares of its owned part of each parameter and the ranks add them up."""
    sharded = opt is not None and getattr(opt, "world", 1) > 1 and hasattr(opt, "layout")
    sq = torch.zeros(len(model.blocks), dtype=torch.float32, device=next(model.parameters()).device)
    if sharded:
        lay, flat = opt.layout, opt.flat_grads
        bucket_of = {id(p): b for b, ps in enumerate(lay.buckets) for p in ps}
    for li, blk in enumerate(model.blocks):
        for p in blk.parameters():
            if not sharded:
                sq[li] += grads.get(p).float().pow(2).sum()
                continue
            lo, hi = lay.slice_of(bucket_of[id(p)], opt.rank)
            a, b = max(lo, lay.offsets[id(p)]), min(hi, lay.offsets[id(p)] + p.numel())
            if b > a:
                sq[li] += flat[a:b].float().pow(2).sum()
    if sharded:
        import torch.distributed as dist
        dist.all_reduce(sq, group=opt.group)
    return {f"gradnorm/L{li:02d}": float(v) for li, v in enumerate(torch.sqrt(sq).tolist())}


@torch.no_grad()
def gate_stats_layerwise(model, x):
    """Per-layer write-law telemetry on a fixed batch `x` (eager forward with collection hooks):
    gates/g_{k,v}_Lxx (mean gate), gates/rf_* (share of tokens whose mean gate is below 0.5: mostly
    context), gates/fraclt03_* (share of gate entries below 0.3), vtail/p999_Lxx and vtail/max (norm of
    the written value per position and head: what `v_clamp_tau` governs), attnlogit/p999_Lxx (largest
    read logit per position and head), kgain/* (learned key gain), and their all-layer summaries.
    Key names follow lm/train_340m/train_flagship.py:211-294."""
    was_training = model.training
    model.eval()
    collect = [dict() for _ in model.blocks]
    model(x, collect=collect)
    model.train(was_training)
    out = {}
    hd = model.blocks[0].attn.head_dim
    mean = lambda v: float(sum(v) / len(v))

    def quantile(t, q):                                   # torch.quantile caps its input size
        t = t.flatten().float()
        k = min(t.numel(), max(1, int(round(q * t.numel()))))
        return float(t.kthvalue(k).values)

    p999, vmax = [], []
    for li, c in enumerate(collect):
        if "vpp" not in c:
            break
        v = torch.cat([t if t.dim() == 3 else t.unsqueeze(1) for t in c["vpp"]], dim=1)
        rn = v.reshape(v.shape[0], v.shape[1], -1, hd).norm(dim=-1)
        p999.append(quantile(rn, 0.999))
        vmax.append(float(rn.max()))
        out[f"vtail/p999_L{li:02d}"] = p999[-1]
    if p999:
        out["vtail/p999_all_layers"], out["vtail/p999_max_layer"] = mean(p999), max(p999)
        out["vtail/max_all_layers"] = max(vmax)
    lp, lmax = [], []
    for li, c in enumerate(collect):
        if "attn_logit_max" not in c:
            break
        sm = torch.cat([t.flatten() for t in c["attn_logit_max"]])
        lp.append(quantile(sm, 0.999))
        lmax.append(float(sm.max()))
        out[f"attnlogit/p999_L{li:02d}"] = lp[-1]
    if lp:
        out["attnlogit/p999_all_layers"], out["attnlogit/p999_max_layer"] = mean(lp), max(lp)
        out["attnlogit/max_all_layers"] = max(lmax)
    gains = [blk.attn.k_gain.detach().float().flatten() for blk in model.blocks
             if getattr(blk.attn, "k_gain", None) is not None]
    if gains:
        allg = torch.cat(gains)
        out.update({"kgain/mean_all_layers": float(allg.mean()), "kgain/max_all_layers": float(allg.max()),
                    "kgain/min_all_layers": float(allg.min()),
                    "kgain/std_all_layers": float(allg.std()) if allg.numel() > 1 else 0.0,
                    "kgain/spread_all_layers": float(allg.max() / (allg.min() + 1e-6))})
        for li, g in enumerate(gains):
            out[f"kgain/mean_L{li:02d}"] = float(g.mean())
    for tag in ("k", "v"):
        gm, rf, lo, ratios, effs = [], [], [], [], []
        for li, c in enumerate(collect):
            if f"g_{tag}" not in c:
                continue
            g = torch.cat([t if t.dim() == 3 else t.unsqueeze(1) for t in c[f"g_{tag}"]], dim=1).float()
            gbar = float(g.mean())
            if f"ratio_{tag}" in c:
                r = mean([float(t.float().mean()) if torch.is_tensor(t) else float(t) for t in c[f"ratio_{tag}"]])
                ratios.append(r)
                effs.append((1 - gbar) * r / (gbar + (1 - gbar) * r + 1e-8))
            gm.append(gbar)
            rf.append(float(((1 - g.mean(dim=-1)) > 0.5).float().mean()))
            lo.append(float((g < 0.3).float().mean()))
            out[f"gates/g_{tag}_L{li:02d}"], out[f"gates/rf_{tag}_L{li:02d}"] = gm[-1], rf[-1]
            out[f"gates/fraclt03_{tag}_L{li:02d}"] = lo[-1]
        if gm:
            out[f"telemetry/g_{tag}_mean_all_layers"] = mean(gm)
            out[f"telemetry/register_frac_{tag}_all_layers"] = mean(rf)
            out[f"telemetry/fraclt03_{tag}_all_layers"] = mean(lo)
        if ratios:
            out[f"telemetry/ratio_{tag}_mean"], out[f"telemetry/eff_ctx_share_{tag}"] = mean(ratios), mean(effs)
    return out
