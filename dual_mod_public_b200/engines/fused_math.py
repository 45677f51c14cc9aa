"""Explicit forward and hand-derived backward of the chunk cell, op by op.

Each function here is the plain-torch statement of one device kernel of the
fused engine (same arguments, same outputs, same accumulation semantics) and is
what the kernels' numerics tests compare against.  It is also the engine's
fallback on a device without the extension (CPU tests).

Layout is token-major throughout: per-head tensors are [B, c, h, dh] views of
[B, c, d] rows, the tape is [B, T, h, dh].

Read algebra.  For one sweep, a chunk row's read is a softmax over
[committed prefix | intra rows (strictly earlier) | raw self].  The prefix part
is sweep-invariant, so it is reduced once per cell to (o_c, lse_c) — normalised
output and log-sum-exp — and every sweep merges its tail against it:

    lse = logaddexp(lse_c, logsumexp(tail));   P_c = exp(lse_c - lse)
    o   = P_c o_c + sum_j P_j v_j,             P_j = exp(s_j - lse)

Backward of the merge, with delta = dO . o:
    d o_c = P_c dO;   d lse_c = P_c (dO . o_c - delta)
    d s_j = P_j (dO . v_j - delta);   d v_j = P_j dO
and of the prefix partial (p_j = exp(s_j - lse_c)):
    d s_j = p_j (d o_c . v_j - d o_c . o_c + d lse_c)
so no running-max bookkeeping is needed (the reference's (A, Z, m) form needs an
argmax sub-gradient fix-up, engines/wavescan/cells/fused_sweep.py:1837-1850).

Reference parity: the fused sweep path of engines/wavescan/cells/fused_sweep.py
(`_comm_fwd_kernel` 154-208, `_attend_head_kernel` 367-420, `_rms_u_kernel` 423-445,
`_refine2_kernel` 514-611 and their backward twins 211-357, 634-1052).
"""

from __future__ import annotations

import torch

NEG = -1e30


# ---- rotary helpers on token-major [B, c, h, dh] ----------------------------------------

def rope_tm(x, cos, sin):
    """x [B,c,h,dh]; cos/sin [c, dh/2]. fp32 math, result in x.dtype."""
    half = x.shape[-1] // 2
    xf = x.float()
    lo, hi = xf[..., :half], xf[..., half:]
    c_, s_ = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat((lo * c_ - hi * s_, hi * c_ + lo * s_), dim=-1).to(x.dtype)


def unrope_tm(x, cos, sin):
    return rope_tm(x, cos, -sin)


# ---- masks ------------------------------------------------------------------------------

def _prefix_mask(c, lo, hi, pos0, window, device):
    """[c, hi-lo] bool or None: chunk row t (absolute pos0+t) reads committed j in
    [lo, hi) iff j > pos0 + t - window."""
    if not window:
        return None
    t = torch.arange(c, device=device)[:, None] + pos0
    j = torch.arange(lo, hi, device=device)[None, :]
    return j > t - window


def _intra_mask(c, window, device):
    i = torch.arange(c, device=device)
    m = i[None, :] < i[:, None]
    if window:
        m = m & (i[None, :] > i[:, None] - window)
    return m


def prefix_lo(pos0: int, window: int, qoff: int = 0) -> int:
    """First committed row any chunk row can read.  `qoff`: the chunk's first query sits qoff rows after
    the end of the key range (0 for a cell reading its own committed prefix)."""
    return min(pos0, max(0, pos0 + qoff - window + 1)) if window else 0


# ---- committed-prefix pass --------------------------------------------------------------

def prefix_fwd(q_r, Kc, Vc, pos0, scale, window=0, qoff=0):
    """q_r [B,c,h,dh]; Kc/Vc tape [B,T,h,dh]; keys are the rows [lo, pos0), query row t sits at absolute
    position pos0 + qoff + t.  Returns (o_c fp32 [B,c,h,dh], lse_c fp32 [B,c,h]); an empty prefix gives (0, NEG)."""
    B, c, h, dh = q_r.shape
    lo = prefix_lo(pos0, window, qoff)
    if pos0 - lo <= 0:
        return (torch.zeros(B, c, h, dh, dtype=torch.float32, device=q_r.device),
                torch.full((B, c, h), NEG, dtype=torch.float32, device=q_r.device))
    K, V = Kc[:, lo:pos0], Vc[:, lo:pos0]
    s = torch.einsum("bchd,bjhd->bhcj", q_r, K).float() * scale
    m = _prefix_mask(c, lo, pos0, pos0 + qoff, window, q_r.device)
    if m is not None:
        s = s.masked_fill(~m, NEG)
    lse = torch.logsumexp(s, dim=-1)                                   # [B,h,c]
    p = torch.exp(s - lse.unsqueeze(-1))
    if m is not None:
        p = p * m                                                       # dead rows contribute 0
    o = torch.einsum("bhcj,bjhd->bchd", p.to(V.dtype), V).float()
    return o, lse.permute(0, 2, 1).contiguous()


def prefix_dq(q_r, Kc, Vc, pos0, scale, window, lse_c, do_c, corr, dq_acc, qoff=0):
    """Query side of the prefix backward for one cell: dq_acc [B,c,h,dh] fp32 += dS K over the
    committed rows.  do_c [B,c,h,dh] (any float dtype), corr [B,c,h] fp32 = do_c.o_c - dlse_c."""
    B, c, h, dh = q_r.shape
    lo = prefix_lo(pos0, window, qoff)
    if pos0 - lo <= 0:
        return
    K, V = Kc[:, lo:pos0], Vc[:, lo:pos0]
    s = torch.einsum("bchd,bjhd->bhcj", q_r, K).float() * scale
    m = _prefix_mask(c, lo, pos0, pos0 + qoff, window, q_r.device)
    if m is not None:
        s = s.masked_fill(~m, NEG)
    p = torch.exp(s - lse_c.permute(0, 2, 1).unsqueeze(-1))
    if m is not None:
        p = p * m
    dov = torch.einsum("bchd,bjhd->bhcj", do_c.float(), V.float())
    ds = p * (dov - corr.permute(0, 2, 1).unsqueeze(-1)) * scale
    dq_acc += torch.einsum("bhcj,bjhd->bchd", ds, K.float())


def prefix_dkv(q_all, doc_all, corr_all, lsec_all, Kc, Vc, pos0, c, q_start, scale, window=0, q_end=None):
    """Key side of the prefix backward, owner-computes: the gradient of tape rows
    [pos0, pos0+c) from every later query (absolute rows >= q_start of the full-sequence
    arrays q_all / doc_all [B,T,h,dh], corr_all / lsec_all [B,T,h]).  Returns fp32
    (dK, dV) [B,c,h,dh]; nothing is accumulated in global memory."""
    B, T, h, dh = q_all.shape
    T = T if q_end is None else min(T, q_end)          # queries [q_start, q_end) only
    dK = torch.zeros(B, c, h, dh, dtype=torch.float32, device=q_all.device)
    dV = torch.zeros_like(dK)
    if q_start >= T:
        return dK, dV
    q, do = q_all[:, q_start:T], doc_all[:, q_start:T].float()
    K, V = Kc[:, pos0:pos0 + c], Vc[:, pos0:pos0 + c]
    s = torch.einsum("bthd,bjhd->bhtj", q, K).float() * scale
    vis = None
    if window:
        t = torch.arange(q_start, T, device=q_all.device)[:, None]
        j = torch.arange(pos0, pos0 + c, device=q_all.device)[None, :]
        vis = j > t - window
        s = s.masked_fill(~vis, NEG)
    p = torch.exp(s - lsec_all[:, q_start:T].permute(0, 2, 1).unsqueeze(-1))
    if vis is not None:
        p = p * vis
    dov = torch.einsum("bthd,bjhd->bhtj", do, V.float())
    ds = p * (dov - corr_all[:, q_start:T].permute(0, 2, 1).unsqueeze(-1)) * scale
    dK += torch.einsum("bhtj,bthd->bjhd", ds, q.float())
    dV += torch.einsum("bhtj,bthd->bjhd", p, do)
    return dK, dV


# ---- per-sweep tail read ------------------------------------------------------------------

def tail_fwd(q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, scale, window=0):
    """One sweep's merged read.  All per-head tensors [B,c,h,dh]; returns
    (o [B,c,h,dh] in v_raw.dtype, lse fp32 [B,c,h], ssq fp32 [B,c,h] = sum_d o^2 per head,
    from which the row's RMS over all heads follows without another pass over o)."""
    c = q_r.shape[1]
    s_in = torch.einsum("bchd,bjhd->bhcj", q_r, K_in).float() * scale
    s_in = s_in.masked_fill(~_intra_mask(c, window, q_r.device), NEG)
    s_self = (q_r.float() * kself_r.float()).sum(-1).permute(0, 2, 1) * scale     # [B,h,c]
    lse_ch = lse_c.permute(0, 2, 1)
    lse = torch.logsumexp(torch.cat((s_in, s_self.unsqueeze(-1), lse_ch.unsqueeze(-1)), dim=-1), dim=-1)
    p_in = torch.exp(s_in - lse.unsqueeze(-1))
    p_self = torch.exp(s_self - lse)
    p_c = torch.exp(lse_ch - lse)
    o = torch.einsum("bhcj,bjhd->bchd", p_in.to(V_in.dtype), V_in).float()
    o = o + p_self.permute(0, 2, 1).unsqueeze(-1) * v_raw.float()
    o = o + p_c.permute(0, 2, 1).unsqueeze(-1) * o_c
    ssq = o.square().sum(-1)                              # [B,c,h]: per-head sum of squares of the read
    return o.to(v_raw.dtype), lse.permute(0, 2, 1).contiguous(), ssq


def tail_bwd(dO, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, o, lse, scale, window=0):
    """Backward of `tail_fwd` for upstream grad dO [B,c,h,dh].  Returns fp32
    (dq, dkself, dvraw, dK_in, dV_in, do_c, dlse_c)."""
    c = q_r.shape[1]
    dOf = dO.float()
    s_in = torch.einsum("bchd,bjhd->bhcj", q_r, K_in).float() * scale
    s_in = s_in.masked_fill(~_intra_mask(c, window, q_r.device), NEG)
    s_self = (q_r.float() * kself_r.float()).sum(-1).permute(0, 2, 1) * scale
    lse_h = lse.permute(0, 2, 1)
    p_in = torch.exp(s_in - lse_h.unsqueeze(-1))                       # [B,h,c,c]
    p_self = torch.exp(s_self - lse_h).permute(0, 2, 1)               # [B,c,h]
    p_c = torch.exp(lse_c - lse)                                       # [B,c,h]
    delta = (dOf * o.float()).sum(-1)                                  # [B,c,h]
    # prefix partial
    do_c = p_c.unsqueeze(-1) * dOf
    dlse_c = p_c * ((dOf * o_c).sum(-1) - delta)
    # self column
    ds_self = p_self * ((dOf * v_raw.float()).sum(-1) - delta) * scale
    dvraw = p_self.unsqueeze(-1) * dOf
    dq = ds_self.unsqueeze(-1) * kself_r.float()
    dkself = ds_self.unsqueeze(-1) * q_r.float()
    # intra block
    dov = torch.einsum("bchd,bjhd->bhcj", dOf, V_in.float())
    ds = p_in * (dov - delta.permute(0, 2, 1).unsqueeze(-1)) * scale
    dq = dq + torch.einsum("bhcj,bjhd->bchd", ds, K_in.float())
    dK_in = torch.einsum("bhcj,bchd->bjhd", ds, q_r.float())
    dV_in = torch.einsum("bhcj,bchd->bjhd", p_in, dOf)
    return dq, dkself, dvraw, dK_in, dV_in, do_c, dlse_c


def tail_self_scalars(dO, q_r, kself_r, v_raw, o, lse, scale):
    """The self column's per-(row, head) scalars of `tail_bwd`: (p_self, dss) with d v_raw = p_self dO,
    d k_self = dss q, and dss k_self the self column's part of d q."""
    dOf = dO.float()
    p_self = torch.exp((q_r.float() * kself_r.float()).sum(-1) * scale - lse)
    delta = (dOf * o.float()).sum(-1)
    return p_self, p_self * ((dOf * v_raw.float()).sum(-1) - delta) * scale


def tail_bwd_sweep(dO, q_r, kself_r, K_in, V_in, lse_c, o, lse, scale, window=0):
    """The per-sweep part of `tail_bwd` when the row-scalar x row products are deferred to the end of the cell:
    returns fp32 (dq_intra, dK_in, dV_in, p_self, p_c, delta); dq_intra lacks the self-column term."""
    c = q_r.shape[1]
    dOf = dO.float()
    s_in = torch.einsum("bchd,bjhd->bhcj", q_r, K_in).float() * scale
    s_in = s_in.masked_fill(~_intra_mask(c, window, q_r.device), NEG)
    s_self = (q_r.float() * kself_r.float()).sum(-1) * scale            # [B,c,h]
    p_in = torch.exp(s_in - lse.permute(0, 2, 1).unsqueeze(-1))         # [B,h,c,c]
    p_self = torch.exp(s_self - lse)
    p_c = torch.exp(lse_c - lse)
    delta = (dOf * o.float()).sum(-1)
    dov = torch.einsum("bchd,bjhd->bhcj", dOf, V_in.float())
    ds = p_in * (dov - delta.permute(0, 2, 1).unsqueeze(-1)) * scale
    dq = torch.einsum("bhcj,bjhd->bchd", ds, K_in.float())
    dK_in = torch.einsum("bhcj,bchd->bjhd", ds, q_r.float())
    dV_in = torch.einsum("bhcj,bchd->bjhd", p_in, dOf)
    return dq, dK_in, dV_in, p_self, p_c, delta


def cell_finish_sweeps(dOs, scal, q_r, kself_r, v_raw, o_c, scale):
    """The deferred sums of a cell's sweeps.  dOs: the sweeps' d o [B,c,h,dh]; scal [K,3,B,c,h] = their
    (p_self, p_c, delta).  Returns fp32 (dq_self, dkself, dvraw, do_c, dlse_c) summed over the sweeps."""
    vf, of = v_raw.float(), o_c.float()
    dss = torch.zeros_like(scal[0, 0])
    dl = torch.zeros_like(dss)
    dvraw = torch.zeros_like(of)
    do_c = torch.zeros_like(of)
    for k in range(len(dOs) - 1, -1, -1):
        g = dOs[k].float()
        ps, pc, delta = scal[k, 0], scal[k, 1], scal[k, 2]
        dss = dss + ps * ((g * vf).sum(-1) - delta) * scale
        dl = dl + pc * ((g * of).sum(-1) - delta)
        dvraw = dvraw + ps.unsqueeze(-1) * g
        do_c = do_c + pc.unsqueeze(-1) * g
    return dss.unsqueeze(-1) * kself_r.float(), dss.unsqueeze(-1) * q_r.float(), dvraw, do_c, dl


# ---- RMSNorm ------------------------------------------------------------------------------------

def rms_fwd(x, w, eps=1e-5):
    """y = x * rstd * w (fp32 math, y in x.dtype); returns (y, rstd fp32 [..., 1])."""
    xf = x.float()
    rstd = torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    return (xf * rstd * w.float()).to(x.dtype), rstd


def rms_bwd(dy, x, w, rstd):
    """Returns (dx fp32, dw fp32 [d])."""
    xf, dyf = x.float(), dy.float()
    xn = xf * rstd
    g = dyf * w.float()
    dx = rstd * (g - xn * (g * xn).mean(-1, keepdim=True))
    dw = (dyf * xn).reshape(-1, x.shape[-1]).sum(0)
    return dx, dw


# ---- refine (gate, blend, rotate) ----------------------------------------------------------------

def row_rstd(ssq, d, eps=1e-5):
    """1/rms of each row over all heads, from the per-head sums of squares: [B,c,h] -> [B,c,1]."""
    return torch.rsqrt(ssq.sum(-1, keepdim=True) / d + eps)


def refine_fwd(raw, ssq, glx, k, v, cos, sin, h, pin_cols=0, eps=1e-5):
    """Write law for the packed layout, with the context norm folded in.

    raw [B,c,4d] = o @ W'^T where W' = W_pack * w_ctx (norm gain folded into the weight
    columns) and o is the UN-normalised read; the row's 1/rms (from ssq [B,c,h]) is applied
    here, so cg = rstd * raw = [k_ctx | v_ctx | gate-u logits k | gate-u logits v].
    glx [B,c,2d]: x̂-half of the gate logits plus bias (sweep-invariant).
    k, v [B,c,d] raw (unrotated) key / value.  `pin_cols`: the first pin_cols value
    columns keep the raw value (kmod_vraw_heads * dh).
    Returns (K_out [B,c,h,dh] rotated, V_out [B,c,h,dh]) in k.dtype.
    """
    B, c, d = k.shape
    cg = raw.float() * row_rstd(ssq, d, eps)
    kc, vc, gku, gvu = cg.split(d, dim=-1)
    gk = torch.sigmoid(glx[..., :d].float() + gku)
    gv = torch.sigmoid(glx[..., d:].float() + gvu)
    kpp = gk * k.float() + (1.0 - gk) * kc
    vpp = gv * v.float() + (1.0 - gv) * vc
    if pin_cols:
        vpp = torch.cat((v[..., :pin_cols].float(), vpp[..., pin_cols:]), dim=-1)
    K_out = rope_tm(kpp.view(B, c, h, d // h), cos, sin)
    return K_out.to(k.dtype), vpp.view(B, c, h, d // h).to(k.dtype)


def refine_bwd(dK_out, dV_out, raw, ssq, o, glx, k, v, cos, sin, pin_cols=0, eps=1e-5):
    """Backward of `refine_fwd`.  dK_out/dV_out [B,c,h,dh]; o [B,c,d] the read.  Returns fp32
    (dcg [B,c,4d] = gradient w.r.t. cg = rstd*raw, dk [B,c,d], dv [B,c,d], uhat [B,c,d] = o*rstd);
    the gate-logit grads dcg[..., 2d:] are also the grads of glx."""
    B, c, d = k.shape
    rstd = row_rstd(ssq, d, eps)
    cg = raw.float() * rstd
    kc, vc, gku, gvu = cg.split(d, dim=-1)
    gk = torch.sigmoid(glx[..., :d].float() + gku)
    gv = torch.sigmoid(glx[..., d:].float() + gvu)
    dkpp = unrope_tm(dK_out.float(), cos, sin).reshape(B, c, d)
    dvpp = dV_out.float().reshape(B, c, d)
    dv_pin = None
    if pin_cols:
        dv_pin = dvpp[..., :pin_cols]
        dvpp = torch.cat((torch.zeros_like(dv_pin), dvpp[..., pin_cols:]), dim=-1)
    kf, vf = k.float(), v.float()
    dgk = dkpp * (kf - kc) * gk * (1.0 - gk)
    dgv = dvpp * (vf - vc) * gv * (1.0 - gv)
    dcg = torch.cat((dkpp * (1.0 - gk), dvpp * (1.0 - gv), dgk, dgv), dim=-1)
    dk = dkpp * gk
    dv = dvpp * gv
    if pin_cols:
        dv = torch.cat((dv_pin, dv[..., pin_cols:]), dim=-1)
    return dcg, dk, dv, o.float() * rstd


# ---- write law of the mult_res family (the reference's 1.3B recipe) ------------------------------
#
#   u    = rstd(o) * o * w_ctx                                    (context norm)
#   cg   = rstd * (o @ W'^T) = [k_c | v_m | gate-u logits k | gate-u logits v],   W' = [W_kctx ; V_map ; W_gk_u ; W_gv_u] * w_ctx
#   v_in = lam * u + sigmoid(vgx) * tanh(v_m)                     (vgx = v_gate(x) + bias, sweep-invariant)
#   v_c  = v_in @ W_vctx^T                                        (second GEMM, outside these functions)
#   k_n  = per-head rms(k_c) * k_gain                             (k_ctx_norm = rms, eps 1e-6)
#   k''  = g_k k + (1 - g_k) k_n ,  v'' = g_v v + (1 - g_v) v_c  (convex sigmoid gates, fp32)
#   v''  : first pin_cols columns keep the raw value; each head is projected onto the L2 ball of radius tau
#   K    = rope(k'')

def mrk_vin_fwd(raw, ssq, o, w_ctx, vgx, lam, eps=1e-5):
    """v_in [B,c,d] in o.dtype.  raw [B,c,4d] un-normalised packed logits; vgx [B,c,d] the x-logits of the
    multiplicative branch's gate (bias included)."""
    d = o.shape[-1]
    rstd = row_rstd(ssq, d, eps)
    u = o.float() * rstd * w_ctx.float()
    vm = raw[..., d:2 * d].float() * rstd
    return (lam * u + torch.sigmoid(vgx.float()) * torch.tanh(vm)).to(o.dtype)


def mrk_vin_bwd(dvin, raw, ssq, o, w_ctx, vgx, lam, eps=1e-5):
    """Returns fp32 (dvm [B,c,d] = gradient w.r.t. cg[..., d:2d], dvgx [B,c,d], du_hat [B,c,d] = the direct path's
    gradient w.r.t. uhat = rstd * o).  The direct path's gradient of the context-norm gain is
    lam * sum_rows(dvin * uhat), formed once per layer from the stashed rows."""
    d = o.shape[-1]
    rstd = row_rstd(ssq, d, eps)
    t = torch.tanh(raw[..., d:2 * d].float() * rstd)
    sg = torch.sigmoid(vgx.float())
    g = dvin.float()
    dvm = g * sg * (1.0 - t * t)
    dvgx = g * t * sg * (1.0 - sg)
    du_hat = lam * g * w_ctx.float()
    return dvm, dvgx, du_hat


def _mrk_parts(raw, vc, ssq, glx, k, v, h, pin_cols, k_gain, tau, eps, eps_h):
    B, c, d = k.shape
    dh = d // h
    rstd = row_rstd(ssq, d, eps)
    cg = raw.float() * rstd
    kc, gku, gvu = cg[..., :d], cg[..., 2 * d:3 * d], cg[..., 3 * d:]
    kch = kc.view(B, c, h, dh)
    rh = torch.rsqrt(kch.pow(2).mean(-1, keepdim=True) + eps_h)                # [B,c,h,1]
    kn = (kch * rh * k_gain.float().view(1, 1, h, 1)).view(B, c, d)
    gk = torch.sigmoid(glx[..., :d].float() + gku)
    gv = torch.sigmoid(glx[..., d:].float() + gvu)
    vcf = vc.float()
    vpre = gv * v.float() + (1.0 - gv) * vcf
    if pin_cols:
        vpre = torch.cat((v[..., :pin_cols].float(), vpre[..., pin_cols:]), dim=-1)
    vh = vpre.view(B, c, h, dh)
    if tau and tau > 0:
        nrm = vh.norm(dim=-1, keepdim=True).clamp_min(1e-20)
        shrink = (tau / nrm).clamp(max=1.0)
    else:
        nrm, shrink = None, None
    return rstd, kc, kch, rh, kn, gk, gv, vcf, vpre, vh, nrm, shrink


def mrk_refine_fwd(raw, vc, ssq, glx, k, v, cos, sin, h, pin_cols, k_gain, tau, eps=1e-5, eps_h=1e-6):
    """(K_out [B,c,h,dh] rotated, V_out [B,c,h,dh]) in k.dtype."""
    B, c, d = k.shape
    _, _, _, _, kn, gk, _, _, _, vh, _, shrink = _mrk_parts(raw, vc, ssq, glx, k, v, h, pin_cols, k_gain, tau, eps, eps_h)
    kpp = gk * k.float() + (1.0 - gk) * kn
    if shrink is not None:
        vh = vh * shrink
    K_out = rope_tm(kpp.view(B, c, h, d // h), cos, sin)
    return K_out.to(k.dtype), vh.to(k.dtype)


def mrk_refine_bwd(dK_out, dV_out, raw, vc, ssq, o, glx, k, v, cos, sin, h, pin_cols, k_gain, tau, eps=1e-5, eps_h=1e-6):
    """Returns fp32 (dcg [B,c,4d] with the v_m block left zero, dvc [B,c,d], dk [B,c,d], dv [B,c,d],
    uhat [B,c,d], dkg [B,c,h] = per-row gradient of k_gain); dcg[..., 2d:] are also the gradients of glx."""
    B, c, d = k.shape
    dh = d // h
    rstd, kc, kch, rh, kn, gk, gv, vcf, vpre, vh, nrm, shrink = _mrk_parts(
        raw, vc, ssq, glx, k, v, h, pin_cols, k_gain, tau, eps, eps_h)
    dkpp = unrope_tm(dK_out.float(), cos, sin).reshape(B, c, d)
    dvo = dV_out.float()                                                        # [B,c,h,dh]
    if shrink is not None:                                                      # projection onto the ball
        inside = (nrm <= tau)
        proj = (dvo * vh).sum(-1, keepdim=True) / (nrm * nrm)
        dvpre = torch.where(inside, dvo, shrink * (dvo - vh * proj))
    else:
        dvpre = dvo
    dvpre = dvpre.reshape(B, c, d)
    dv_pin = None
    if pin_cols:
        dv_pin = dvpre[..., :pin_cols]
        dvpre = torch.cat((torch.zeros_like(dv_pin), dvpre[..., pin_cols:]), dim=-1)
    kf, vf = k.float(), v.float()
    dgk = dkpp * (kf - kn) * gk * (1.0 - gk)
    dgv = dvpre * (vf - vcf) * gv * (1.0 - gv)
    dvc = dvpre * (1.0 - gv)
    dk = dkpp * gk
    dv = dvpre * gv
    if pin_cols:
        dv = torch.cat((dv_pin, dv[..., pin_cols:]), dim=-1)
    # per-head rms + gain backward
    dkn = (dkpp * (1.0 - gk)).view(B, c, h, dh)
    gn = k_gain.float().view(1, 1, h, 1)
    xhat_h = kch * rh
    dk_gain = (dkn * xhat_h).sum(-1)
    dx = dkn * gn
    dkc = (rh * (dx - xhat_h * (dx * xhat_h).mean(-1, keepdim=True))).view(B, c, d)
    dcg = torch.cat((dkc, torch.zeros_like(dkc), dgk, dgv), dim=-1)
    return dcg, dvc, dk, dv, o.float() * rstd, dk_gain


def rmsn_bwd(du, o, ssq, eps=1e-5):
    """Backward of uhat = o * rstd(o) (no gain): d o = rstd * (du - uhat * mean(du * uhat)). fp32."""
    d = o.shape[-1]
    rstd = row_rstd(ssq, d, eps)
    uhat = o.float() * rstd
    duf = du.float()
    return rstd * (duf - uhat * (duf * uhat).mean(-1, keepdim=True))


# ---- SwiGLU pointwise ---------------------------------------------------------------------------

def swiglu_fwd(h1, h3):
    return (torch.nn.functional.silu(h1.float()) * h3.float()).to(h1.dtype)


def swiglu_bwd(dg, h1, h3):
    """g = silu(h1) * h3 -> (dh1, dh3) in h1.dtype."""
    h1f, h3f, dgf = h1.float(), h3.float(), dg.float()
    sg = torch.sigmoid(h1f)
    silu = h1f * sg
    dh1 = dgf * h3f * (sg * (1.0 + h1f * (1.0 - sg)))
    return dh1.to(h1.dtype), (dgf * silu).to(h1.dtype)


# ---- chunked cross-entropy head ---------------------------------------------------------------------

def ce_chunk(logits, targets, inv_n):
    """Sum-reduced CE * inv_n over one slab, and d(logits) for it.  logits [n,V]
    (any float dtype), targets [n] with -1 = ignore.  Returns (loss fp32 scalar,
    dlogits in logits.dtype)."""
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    valid = targets >= 0
    tgt = targets.clamp_min(0)
    picked = lf.gather(-1, tgt[:, None]).squeeze(-1)
    loss = ((lse - picked) * valid).sum() * inv_n
    p = torch.exp(lf - lse[:, None])
    p.scatter_add_(-1, tgt[:, None], -torch.ones_like(picked)[:, None])
    return loss, (p * (valid[:, None] * inv_n)).to(logits.dtype)
