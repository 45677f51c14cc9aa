"""Exact sequential scan: the semantic oracle every engine is tested against.

All raw projections of a layer are one batched matmul; only the position axis
is serial, and each position runs `attend_one` + `refine_kv` + rotate-at-write,
the same step incremental decode uses.  Because the tape is append-only, the
state at the start of a span of positions is exactly the first rows of the
final tape, so a span can be re-materialised in backward from its inputs and
that prefix alone: `checkpoint_chunk` bounds activation memory that way.
Reference parity: models/dualmod/scan.py:19-95.
"""

from __future__ import annotations

import torch
from torch.utils.checkpoint import checkpoint

from .rope import apply_rope


def _record_mass(collect, probs):
    """Attention-mass telemetry for one position (head-averaged)."""
    pm = probs.mean(dim=1)[:, 0, :]                      # [B, n_keys]
    n = pm.shape[-1]
    collect["inc_mass"][:, :n] += pm
    collect.setdefault("hop_mass", []).append(pm[:, -2] if n >= 2 else torch.zeros_like(pm[:, -1]))
    collect.setdefault("self_mass", []).append(pm[:, -1])
    collect.setdefault("max_mass", []).append(pm.amax(dim=-1))


def _scan_chunk(attn, xhat_c, q_r_c, k_c, k_self_r_c, v_c, cos_c, sin_c, K_past, V_past,
                collect=None):
    """Positions of one span, in order.

    xhat_c [B,n,d]; q_r_c / k_c (unrotated) / k_self_r_c / v_c [B,h,n,dh];
    cos_c / sin_c [n, dh/2]; K_past / V_past [B,h,P,dh] the tape so far.
    Returns (o [B,h,n,dh], K_rows [B,h,n,dh], V_rows [B,h,n,dh]).
    """
    n = xhat_c.shape[1]
    k_rows, v_rows, reads = [], [], []
    K_cur, V_cur = K_past, V_past
    for j in range(n):
        sl = slice(j, j + 1)
        o_j, probs = attn.attend_one(q_r_c[:, :, sl], k_self_r_c[:, :, sl], v_c[:, :, sl],
                                     K_cur, V_cur, need_probs=collect is not None, collect=collect)
        kpp, vpp = attn.refine_kv(xhat_c[:, sl], attn._merge(o_j),
                                  attn._merge(k_c[:, :, sl]), attn._merge(v_c[:, :, sl]),
                                  collect=collect)
        k_rows.append(apply_rope(attn._split(kpp), cos_c[sl], sin_c[sl]))
        v_rows.append(attn._split(vpp))
        reads.append(o_j)
        if j + 1 < n:
            K_cur = torch.cat((K_cur, k_rows[-1]), dim=2)
            V_cur = torch.cat((V_cur, v_rows[-1]), dim=2)
        if probs is not None:
            _record_mass(collect, probs)
    return torch.cat(reads, dim=2), torch.cat(k_rows, dim=2), torch.cat(v_rows, dim=2)


def sequential_scan(attn, xhat, cos, sin, collect=None, return_tape=False):
    """Whole-layer exact scan.  Returns o_cat [B,T,d] (before W_O); with
    `return_tape` also the final tape (K [B,h,T,dh] rotated, V [B,h,T,dh])."""
    cfg = attn.cfg
    B, T, _ = xhat.shape
    q_r = apply_rope(attn._split(attn.wq(xhat)), cos, sin)
    k = attn._split(attn.wk(xhat))
    k_self_r = apply_rope(k, cos, sin)
    v = attn._split(attn.project_v(xhat))
    if collect is not None:
        collect["inc_mass"] = torch.zeros(B, T, device=xhat.device)

    span = cfg.checkpoint_chunk if cfg.checkpoint_chunk and cfg.checkpoint_chunk > 0 else T
    rematerialise = (0 < span < T and torch.is_grad_enabled() and attn.training and collect is None)

    K_tape = q_r.new_zeros(B, attn.n_heads, 0, attn.head_dim)
    V_tape = v.new_zeros(B, attn.n_heads, 0, attn.head_dim)
    reads = []
    for a in range(0, T, span):
        s = slice(a, min(a + span, T))
        args = (attn, xhat[:, s], q_r[:, :, s], k[:, :, s], k_self_r[:, :, s], v[:, :, s],
                cos[s], sin[s], K_tape, V_tape)
        if rematerialise:
            o_c, K_new, V_new = checkpoint(_scan_chunk, *args, use_reentrant=False)
        else:
            o_c, K_new, V_new = _scan_chunk(*args, collect=collect)
        K_tape = torch.cat((K_tape, K_new), dim=2)
        V_tape = torch.cat((V_tape, V_new), dim=2)
        reads.append(o_c)
    o = attn._merge(torch.cat(reads, dim=2))
    return (o, K_tape, V_tape) if return_tape else o
