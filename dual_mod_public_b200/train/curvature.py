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
def layer_grad_norms(model, grads):
    """{"gradnorm/L00": ..., ...} from a `GradBuffers`-like object with `.get(param)`."""
    out = {}
    for li, blk in enumerate(model.blocks):
        sq = sum(grads.get(p).float().pow(2).sum() for p in blk.parameters())
        out[f"gradnorm/L{li:02d}"] = float(torch.sqrt(sq))
    return out
