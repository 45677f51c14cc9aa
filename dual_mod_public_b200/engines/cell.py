"""Chunked Jacobi cell in plain torch: the semantic reference of the engines.

A cell covers c consecutive positions of one layer.  It reads the committed
tape rows written by earlier cells, and solves the intra-chunk recurrence by K
Jacobi sweeps: sweep 0 reads the chunk's RAW rows, sweep s reads the rows
refined by sweep s-1.  A position's own entry is always its raw key/value,
kept as a separate softmax column so it never mixes with refined rows.  After
s sweeps the first s chunk positions are exact; K = c is exact.

The write law is `DualModAttention.refine_kv` itself, so every config knob is
covered and the cell is differentiable by autograd (the engines' generic
backward re-runs it).  Reference parity: engines/wavescan/cells/scan_cell_fwd.py:56-116
(cell), :119-149 (committed-prefix merge algebra), cells/reference.py:14-37.
"""

from __future__ import annotations

import torch

from ..models.rope import apply_rope
from ..models.scan import _scan_chunk

NEG = -1e30          # finite mask value: fully masked rows stay NaN-free in backward


def intra_mask(c: int, device, window: int = 0) -> torch.Tensor:
    """[c, c] bool, True where chunk row t may read intra column s (s < t, and
    inside the sliding window when one is set)."""
    i = torch.arange(c, device=device)
    m = i[None, :] < i[:, None]
    if window:
        m = m & (i[None, :] > i[:, None] - window)
    return m


def committed_mask(c: int, a: int, device, window: int) -> torch.Tensor | None:
    """[c, a] bool for a sliding window: chunk row t (absolute a + t) reads
    committed column j iff j > a + t - window.  None when no window."""
    if not window:
        return None
    t = torch.arange(c, device=device)[:, None] + a
    j = torch.arange(a, device=device)[None, :]
    return j > t - window


class PrefixRead:
    """Sweep-invariant part of a cell's read: the softmax partial of the chunk
    queries over the committed prefix, as a normalised output and its
    log-sum-exp.  Computed once per cell, merged with every sweep's tail."""

    def __init__(self, q_r, K_comm, V_comm, scale, window=0):
        a = 0 if K_comm is None else K_comm.shape[2]
        self.empty = a == 0
        if self.empty:
            return
        s = (q_r @ K_comm.transpose(-1, -2)).float() * scale          # [B,h,c,a]
        cm = committed_mask(q_r.shape[2], a, q_r.device, window)
        if cm is not None:
            s = s.masked_fill(~cm, NEG)
        self.lse = torch.logsumexp(s, dim=-1, keepdim=True)            # ~NEG if a row sees no key
        p = torch.exp(s - self.lse)
        self.o = (p.to(V_comm.dtype) @ V_comm).float()                  # [B,h,c,dh]


def merged_read(q_r, k_self_r, v_raw, K_intra, V_intra, prefix: PrefixRead, mask, scale):
    """One sweep's read for all chunk rows: softmax over [committed | intra rows
    (masked) | raw self] assembled from the prefix partial and the tail block."""
    s_in = (q_r @ K_intra.transpose(-1, -2)).float() * scale
    s_in = s_in.masked_fill(~mask, NEG)
    s_self = (q_r.float() * k_self_r.float()).sum(-1, keepdim=True) * scale
    tail = torch.cat((s_in, s_self), dim=-1)                            # [B,h,c,c+1]
    lse_t = torch.logsumexp(tail, dim=-1, keepdim=True)
    lse = lse_t if prefix.empty else torch.logaddexp(lse_t, prefix.lse)
    p = torch.exp(tail - lse)
    o = (p[..., :-1].to(V_intra.dtype) @ V_intra).float() + p[..., -1:] * v_raw.float()
    if not prefix.empty:
        o = o + torch.exp(prefix.lse - lse) * prefix.o
    return o.to(v_raw.dtype)


def chunk_cell_forward(attn, xhat_c, cos_c, sin_c, K_comm, V_comm, n_sweeps, mask=None):
    """One (layer, chunk) cell.

    xhat_c [B,c,d] normed chunk input; cos_c / sin_c RoPE rows of the chunk's
    absolute positions; K_comm / V_comm [B,h,a,dh] committed tape (None or a=0
    for the first chunk).  Returns (o_cat [B,c,d], K_rows [B,h,c,dh] rotated,
    V_rows [B,h,c,dh]): the last sweep's read and the rows to commit.
    """
    c = xhat_c.shape[1]
    W = attn.cfg.local_window or 0
    if mask is None:
        mask = intra_mask(c, xhat_c.device, W)
    q_r = apply_rope(attn._split(attn.wq(xhat_c)), cos_c, sin_c)
    k_flat, v_flat = attn.wk(xhat_c), attn.project_v(xhat_c)
    k_self_r = apply_rope(attn._split(k_flat), cos_c, sin_c)
    v_raw = attn._split(v_flat)
    prefix = PrefixRead(q_r, K_comm, V_comm, attn.scale, W)
    K_in, V_in, o_cat = k_self_r, v_raw, None
    for _ in range(n_sweeps):
        o = merged_read(q_r, k_self_r, v_raw, K_in, V_in, prefix, mask, attn.scale)
        o_cat = attn._merge(o)
        kpp, vpp = attn.refine_kv(xhat_c, o_cat, k_flat, v_flat)
        K_in, V_in = apply_rope(attn._split(kpp), cos_c, sin_c), attn._split(vpp)
    return o_cat, K_in, V_in


# ---- oracle wrappers in cell-test shapes -------------------------------------------

def eager_cell(attn, xhat_c, cos_c, sin_c, K_past, V_past):
    """The exact per-position scan over one chunk: (o [B,h,c,dh], K_rows, V_rows)."""
    q_r = apply_rope(attn._split(attn.wq(xhat_c)), cos_c, sin_c)
    k = attn._split(attn.wk(xhat_c))
    v = attn._split(attn.project_v(xhat_c))
    return _scan_chunk(attn, xhat_c, q_r, k, apply_rope(k, cos_c, sin_c), v, cos_c, sin_c,
                       K_past, V_past)


def eager_layer(attn, xhat, cos, sin):
    """Exact scan over a whole layer from an empty tape."""
    B = xhat.shape[0]
    empty = xhat.new_zeros(B, attn.n_heads, 0, attn.head_dim)
    return eager_cell(attn, xhat, cos, sin, empty, empty.clone())


# ---- layer / model forward over a schedule (generic path) ----------------------------

def layer_forward(attn, xhat, cos, sin, schedule, K_cache, V_cache, o_out=None):
    """All cells of one layer in order; rows [pos0, pos0+c) of K_cache / V_cache
    ([B,h,T_max,dh]) are written append-only.  Returns o_cat [B,T,d]."""
    B, T, _ = xhat.shape
    if o_out is None:
        o_out = xhat.new_empty(B, T, attn.d_attn)
    for pos0, c, k in schedule:
        rows = slice(pos0, pos0 + c)
        o_cat, K_rows, V_rows = chunk_cell_forward(
            attn, xhat[:, rows], cos[rows], sin[rows],
            K_cache[:, :, :pos0], V_cache[:, :, :pos0], k)
        K_cache[:, :, rows] = K_rows.to(K_cache.dtype)
        V_cache[:, :, rows] = V_rows.to(V_cache.dtype)
        o_out[:, rows] = o_cat
    return o_out


def model_forward(model, idx, schedule, K_caches, V_caches, xl_saved=None):
    """Chunked forward of the whole model -> logits [B,T,V]; optionally records
    every layer's input (and the final activations) in `xl_saved`."""
    x = model.tok_emb(idx)
    T = x.shape[1]
    cos, sin = model.rope_cos[:T], model.rope_sin[:T]
    for li, blk in enumerate(model.blocks):
        if xl_saved is not None:
            xl_saved[li].copy_(x)
        o = layer_forward(blk.attn, blk.attn_norm(x), cos, sin, schedule,
                          K_caches[li], V_caches[li])
        x = x + blk.attn.wo(o)
        x = x + blk.mlp(blk.mlp_norm(x))
    if xl_saved is not None:
        xl_saved[len(model.blocks)].copy_(x)
    return model.lm_head(model.norm_f(x))
