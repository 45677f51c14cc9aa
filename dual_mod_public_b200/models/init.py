"""Weight initialisation for `DualModLM`.

Same distributions as the reference (models/dualmod/model.py:152-263): every
Linear / Embedding N(0, 0.02); residual outputs (`wo`, `w2`) N(0, 0.02/sqrt(2L));
ctx projections N(0, ctx_proj_init_std); gate biases by the selected scheme;
factored operators initialised so the composed matrix has the dense target
variance; ctx_mod-specific identity inits.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from .layers import LoRALinear

STD = 0.02


def _logit(u: torch.Tensor) -> torch.Tensor:
    return torch.log(u) - torch.log1p(-u)


def _spread(n: int, lo: float, hi: float, gen) -> torch.Tensor:
    """n gate values evenly covering [lo, hi] (exact mean 0.5 when lo+hi=1) in a
    seeded random order."""
    return torch.linspace(lo, hi, n)[torch.randperm(n, generator=gen)]


def key_bias_ugi(n_heads, head_dim, gen, eps=0.04):
    """Uniform-gate init for keys: one bias per RoPE pair, shared by both members
    (dims i and i + dh/2 are mixed by the rotation)."""
    half = head_dim // 2
    out = torch.empty(n_heads, head_dim)
    for h in range(n_heads):
        pair = _logit(_spread(half, eps, 1 - eps, gen))
        out[h] = torch.cat((pair, pair))
    return out.reshape(-1)


def value_bias_spread(n_heads, head_dim, gen, lo, hi):
    """Per-dim spread of value gates over [lo, hi]."""
    out = torch.empty(n_heads, head_dim)
    for h in range(n_heads):
        out[h] = _logit(_spread(head_dim, lo, hi, gen))
    return out.reshape(-1)


def key_bias_committed(n_heads, head_dim, gen, b_commit=3.0, n_frontier=6, frontier_hi=1.5):
    """Per head, RoPE pairs are split into raw-committed (+b), ctx-committed (-b)
    and a mobile frontier.  Returns (bias [d], cls [d]) with cls 0/1/2."""
    half = head_dim // 2
    n_commit = (half - n_frontier) // 2
    assert 2 * n_commit + n_frontier == half, "frontier count must keep pairs even"
    base_b = torch.cat((torch.full((n_commit,), b_commit), torch.full((n_commit,), -b_commit),
                        torch.linspace(-frontier_hi, frontier_hi, n_frontier)))
    base_c = torch.cat((torch.zeros(n_commit), torch.ones(n_commit),
                        torch.full((n_frontier,), 2.0))).long()
    bias = torch.empty(n_heads, head_dim)
    cls = torch.empty(n_heads, head_dim, dtype=torch.long)
    for h in range(n_heads):
        perm = torch.randperm(half, generator=gen)
        bias[h] = torch.cat((base_b[perm], base_b[perm]))
        cls[h] = torch.cat((base_c[perm], base_c[perm]))
    return bias.reshape(-1), cls.reshape(-1)


def _init_factored(mod: LoRALinear, target_std: float):
    """Both factors N(0, s) with r*s^4 = target_std^2 so Var((up@down)_ij) = target_std^2."""
    r = mod.down.weight.shape[0]
    s = math.sqrt(target_std) / r ** 0.25
    nn.init.normal_(mod.down.weight, 0.0, s)
    nn.init.normal_(mod.up.weight, 0.0, s)
    if mod.up.bias is not None:
        nn.init.zeros_(mod.up.bias)


def _init_ctx_proj(mod, std):
    if isinstance(mod, LoRALinear):
        _init_factored(mod, std)
    else:
        nn.init.normal_(mod.weight, 0.0, std)


def _gate_generator(cfg, path: int, layer: int):
    return torch.Generator().manual_seed(cfg.gate_init_seed * 1000 + 10 * layer + path)


def _set_gate_bias(cfg, bias, scheme, path, layer):
    if scheme == "scalar":
        nn.init.constant_(bias, cfg.gate_bias_init)
        return
    assert bias.numel() == cfg.d_model, "structured init assumes a d-wide convex gate"
    gen = _gate_generator(cfg, path, layer)
    if scheme == "ugi" and path == 0:
        b = key_bias_ugi(cfg.n_heads, cfg.head_dim, gen, cfg.ugi_eps)
    elif scheme == "ugi":
        b = value_bias_spread(cfg.n_heads, cfg.head_dim, gen, cfg.ugi_eps, 1 - cfg.ugi_eps)
    elif scheme == "band":
        b = value_bias_spread(cfg.n_heads, cfg.head_dim, gen, cfg.value_band_lo, cfg.value_band_hi)
    else:
        raise NotImplementedError(scheme)
    with torch.no_grad():
        bias.copy_(b.to(bias.dtype))


def _init_gate_weights(cfg, gate):
    if cfg.gate_rank > 0:
        nn.init.normal_(gate.a.weight, 0.0, STD)
        nn.init.normal_(gate.b.weight, 0.0, STD)
    else:
        nn.init.normal_(gate.weight, 0.0, STD)


def init_dualmod_lm(model) -> None:
    cfg = model.cfg
    for m in model.modules():
        if isinstance(m, nn.Linear):
            nn.init.normal_(m.weight, 0.0, STD)
            if m.bias is not None:
                nn.init.zeros_(m.bias)
        elif isinstance(m, nn.Embedding):
            nn.init.normal_(m.weight, 0.0, STD)
    resid_std = STD / math.sqrt(2 * cfg.n_layers)
    for li, blk in enumerate(model.blocks):
        a = blk.attn
        nn.init.normal_(a.wo.weight, 0.0, resid_std)
        nn.init.normal_(blk.mlp.w2.weight, 0.0, resid_std)
        if hasattr(a, "w_kctx"):
            _init_ctx_proj(a.w_kctx, cfg.ctx_proj_init_std)
            _init_gate_weights(cfg, a.w_gk)
            if cfg.gate_bias_init_k == "committed":
                gen = _gate_generator(cfg, 0, li)
                b, cls = key_bias_committed(cfg.n_heads, cfg.head_dim, gen, cfg.key_commit_bias,
                                            cfg.key_frontier_pairs, cfg.key_frontier_hi)
                with torch.no_grad():
                    a.w_gk.bias.copy_(b.to(a.w_gk.bias.dtype))
                    rows = (cls == 1).nonzero(as_tuple=True)[0]
                    # ctx-committed dims start with real content in their W_Kctx rows
                    a.w_kctx.weight[rows, :] = torch.randn(
                        len(rows), cfg.d_model, generator=gen) * cfg.ctx_reserved_init_std
            else:
                _set_gate_bias(cfg, a.w_gk.bias, cfg.gate_bias_init_k, 0, li)
        if hasattr(a, "w_vctx"):
            _init_ctx_proj(a.w_vctx, cfg.ctx_proj_init_std)
            _init_gate_weights(cfg, a.w_gv)
            if cfg.gate_type_v == "independent":
                nn.init.zeros_(a.w_gv.bias)          # g_raw = g_ctx = 0.5
            else:
                _set_gate_bias(cfg, a.w_gv.bias, cfg.gate_bias_init_v, 1, li)
        mod = cfg.ctx_mod
        if mod in ("vmlp", "fusion", "kmlp"):
            for pre in ("v_pre", "k_pre"):
                if hasattr(a, pre):
                    nn.init.zeros_(getattr(a, pre).weight)
        elif mod in ("mult", "mult_res") and hasattr(a, "v_gate"):
            if cfg.ctx_rank > 0:
                _init_factored(a.v_gate, STD)
                if mod == "mult_res":
                    nn.init.zeros_(a.v_map.up.weight)    # composed W = 0: identity carry
                else:
                    _init_factored(a.v_map, STD)
            elif mod == "mult_res":
                nn.init.zeros_(a.v_map.weight)
        elif mod == "linpoint" and hasattr(a, "v_pre"):
            eye = torch.eye(cfg.d_model)
            with torch.no_grad():               # silu(x) - silu(-x) = x: starts as the identity
                a.v_pre.weight.copy_(torch.cat((eye, -eye), dim=0))
                a.v_comb.weight.copy_(torch.cat((eye, -eye), dim=1))
        elif mod.endswith("_hw") and hasattr(a, "w_vctx"):
            nn.init.normal_(a.w_vctx.weight, 0.0, STD)
