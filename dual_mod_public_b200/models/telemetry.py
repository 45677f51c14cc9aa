"""Gate / attention telemetry on a fixed validation batch.

`collect_telemetry` runs the model with per-layer `collect` dicts and reduces what
the attention layers recorded: mean gates, the fraction of "register" tokens (mean
1-g above 0.5), gates by token class (function vs content), ctx/raw norm ratios and
the attention mass received by the most / least register-like keys.
`grad_norm_ratios` compares the gradient norms of the ctx projections with those of
the raw projections.  Reference parity: models/dualmod/telemetry.py:10-92.
"""

from __future__ import annotations

import numpy as np
import torch


def _layer_stats(c, tag, is_function, out, hists, p):
    g = torch.cat(c[f"g_{tag}"], dim=1)                       # [B, T, d]
    mean_tok, min_tok = g.mean(-1), g.min(-1).values
    out[f"{p}/g_{tag}_mean"] = mean_tok.mean().item()
    out[f"{p}/g_{tag}_tokmin_mean"] = min_tok.mean().item()
    out[f"{p}/register_frac_{tag}"] = ((1 - mean_tok) > 0.5).float().mean().item()
    out[f"{p}/g_{tag}_function"] = mean_tok[is_function].mean().item()
    out[f"{p}/g_{tag}_content"] = mean_tok[~is_function].mean().item()
    out[f"{p}/norm_ratio_{tag}"] = torch.cat(c[f"ratio_{tag}"], dim=1).mean().item()
    hists[f"{p}/g_{tag}_hist"] = mean_tok.flatten().cpu().numpy()
    hists[f"{p}/g_{tag}_tokmin_hist"] = min_tok.flatten().cpu().numpy()
    return mean_tok


@torch.no_grad()
def collect_telemetry(model, x_val, function_mask, prefix="telemetry"):
    """Returns (scalars: dict[str, float], hists: dict[str, np.ndarray])."""
    was_training = model.training
    model.eval()
    collect = [dict() for _ in model.blocks]
    model(x_val, collect=collect)
    model.train(was_training)
    T = x_val.shape[1]
    is_function = function_mask.to(x_val.device)[x_val]
    scalars, hists = {}, {}
    for li, c in enumerate(collect):
        p = f"{prefix}/L{li}"
        gk_tok = None
        for tag in ("k", "v"):
            if f"g_{tag}" in c:
                m = _layer_stats(c, tag, is_function, scalars, hists, p)
                gk_tok = m if tag == "k" else gk_tok
        if "inc_mass" in c and gk_tok is not None:
            readers = torch.arange(T, 0, -1, device=x_val.device).float()     # queries that can see key j
            received = (c["inc_mass"] / readers).flatten()
            reg = (1 - gk_tok).flatten()
            hi, lo = torch.quantile(reg, 0.9), torch.quantile(reg, 0.1)
            scalars[f"{p}/attn_mass_top_decile_1mgk"] = received[reg >= hi].mean().item()
            scalars[f"{p}/attn_mass_bot_decile_1mgk"] = received[reg <= lo].mean().item()
    for tag in ("k", "v"):
        for stem in (f"g_{tag}_mean", f"register_frac_{tag}"):
            vals = [v for k, v in scalars.items() if k.endswith("/" + stem)]
            if vals:
                scalars[f"{prefix}/{stem}_all_layers"] = float(np.mean(vals))
    return scalars, hists


@torch.no_grad()
def grad_norm_ratios(model, prefix="telemetry", grads=None):
    """Per layer: ||grad W_ctx|| and its ratio to ||grad W_raw||.  `grads` may be a
    `GradBuffers` (engine runs); otherwise `p.grad` is read."""
    def g_of(mod):
        w = mod.weight if not hasattr(mod, "up") else mod.up.weight
        return grads.get(w) if grads is not None else w.grad
    out = {}
    for li, blk in enumerate(model.blocks):
        a, p = blk.attn, f"{prefix}/L{li}"
        for ctx, raw, tag in (("w_kctx", "wk", "k"), ("w_vctx", "wv", "v")):
            if not hasattr(a, ctx):
                continue
            gc, gr = g_of(getattr(a, ctx)), g_of(getattr(a, raw))
            if gc is None or gr is None:
                continue
            out[f"{p}/gradnorm_w{tag}ctx"] = gc.norm().item()
            out[f"{p}/gradnorm_ratio_{tag}ctx_over_raw"] = gc.norm().item() / (gr.norm().item() + 1e-12)
    return out
