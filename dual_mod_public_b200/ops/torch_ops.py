"""Op table in plain torch: the CPU/fallback implementation of every device op
the fused engines call.  `CudaOps` (cuda_ops.py) overrides entries with the
sm_100a kernels; the numerics tests compare the two entry by entry."""

from __future__ import annotations

import torch

from ..engines import fused_math as fm


def _into(out, vals, accumulate):
    """`vals` as they are, or written into (added to, when `accumulate`) the tensors `out` and those returned."""
    if out is None:
        return vals
    for o, v in zip(out, vals):
        if accumulate:
            o += v
        else:
            o.copy_(v)
    return tuple(out)


class TorchOps:
    name = "torch"
    launches = 0                      # custom-kernel launch counter (0 here by construction)

    # ---- GEMMs ------------------------------------------------------------------
    def linear(self, x, w, bias=None, out_dtype=None, out=None, narrow=False):
        """x [..., k] @ w[n, k]^T (+ bias).  `out`: a [rows, n] view (dense last dim, any row stride, e.g. a
        column block of a wider matrix) to write into instead of a fresh tensor.  `narrow`: the product is a factor of
        a low-rank operator (a hint for the kernel table; no effect here)."""
        y = x @ w.t()
        if bias is not None:
            y = y + bias.to(y.dtype)
        if out is not None:
            out.copy_(y.reshape(out.shape))
            return out
        return y if out_dtype is None else y.to(out_dtype)

    def linear_dx(self, dy, w, out=None, narrow=False):
        """dy [..., n] @ w[n, k] -> [..., k] (`out` as for `linear`)"""
        if out is not None:
            out.copy_((dy @ w).reshape(out.shape))
            return out
        return dy @ w

    def linear_dw_acc(self, dW, dy, x):
        """dW[n, k] (fp32) += dy[rows, n]^T @ x[rows, k]"""
        dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
        if dy2.dtype == torch.float32:
            dW.addmm_(dy2.t(), x2)
        else:
            dW.add_(torch.mm(dy2.t(), x2, out_dtype=torch.float32)
                    if dy2.is_cuda else (dy2.t().float() @ x2.float()))

    # ---- pointwise / norms --------------------------------------------------------
    def rms_fwd(self, x, w, eps=1e-5):
        return fm.rms_fwd(x, w, eps)

    def rms_bwd(self, dy, x, w, rstd, dw_acc, residual=None, out_dtype=torch.float32):
        """dw_acc (fp32 [d]) += weight grad; returns residual + dx in out_dtype."""
        dx, dw = fm.rms_bwd(dy, x, w, rstd)
        dw_acc.add_(dw)
        if residual is not None:
            dx = dx + residual.float()
        return dx.to(out_dtype)

    def col_sum_acc(self, out, dy):
        """out (fp32 [n]) += column sums of dy [rows, n]."""
        out.add_(dy.reshape(-1, dy.shape[-1]).float().sum(0))

    def rope(self, x, cos, sin):
        return fm.rope_tm(x, cos, sin)

    def unrope(self, x, cos, sin):
        return fm.unrope_tm(x, cos, sin)

    def swiglu_fwd(self, h1, h3):
        return fm.swiglu_fwd(h1, h3)

    def swiglu_bwd(self, dg, h1, h3):
        return fm.swiglu_bwd(dg, h1, h3)

    # ---- cell ops -------------------------------------------------------------------
    def prefix_fwd(self, q_r, Kc, Vc, pos0, scale, window=0, out=None, qoff=0):
        """`out`: optional (o_c, lse_c) fp32 tensors to write into (and return).  `qoff`: rows between the end
        of the key range and the first query (0 for a cell reading its own committed prefix)."""
        o_c, lse_c = fm.prefix_fwd(q_r, Kc, Vc, pos0, scale, window, qoff)
        if out is None:
            return o_c, lse_c
        out[0].copy_(o_c)
        out[1].copy_(lse_c)
        return out

    def prefix_dq(self, q_r, Kc, Vc, pos0, scale, window, lse_c, do_c, corr, dq_acc, qoff=0):
        fm.prefix_dq(q_r, Kc, Vc, pos0, scale, window, lse_c, do_c, corr, dq_acc, qoff)

    def prefix_dkv(self, q_all, doc_all, corr_all, lsec_all, Kc, Vc, pos0, c, q_start, scale, window=0, q_end=None,
                   out=None, accumulate=False):
        """`out`: optional (dK, dV) fp32 views [B, c, h, dh] to write into, or to add to when `accumulate`."""
        dK, dV = fm.prefix_dkv(q_all, doc_all, corr_all, lsec_all, Kc, Vc, pos0, c, q_start, scale, window, q_end)
        return _into(out, (dK, dV), accumulate)

    # ---- window ops: G consecutive chunks of C rows of the same sequences (statement: a loop over the
    # chunks; the kernel table does each in one launch).  Window tensors are [B, G*C, ...]; group z reads
    # the tape rows [max(0, lo + z*C), pos0 + z*C).
    def win_near_fwd(self, q_win, Kc, Vc, pos0, lo, C, scale, window=0):
        outs = []
        for z in range(q_win.shape[1] // C):
            l, p = max(0, lo + z * C), pos0 + z * C
            outs.append(fm.prefix_fwd(q_win[:, z * C:(z + 1) * C], Kc[:, l:], Vc[:, l:], p - l, scale, window))
        return torch.cat([o for o, _ in outs], 1), torch.cat([l for _, l in outs], 1)

    def win_near_dq(self, q_win, Kc, Vc, pos0, lo, C, scale, lse_n, do_n, corr_n, dq_acc, window=0):
        for z in range(q_win.shape[1] // C):
            l, p, r = max(0, lo + z * C), pos0 + z * C, slice(z * C, (z + 1) * C)
            fm.prefix_dq(q_win[:, r], Kc[:, l:], Vc[:, l:], p - l, scale, window, lse_n[:, r], do_n[:, r], corr_n[:, r],
                         dq_acc[:, r])

    def win_tail_fwd(self, q_win, ks_win, vr_win, K_in, V_in, o_c, lse_c, C, scale, window=0):
        outs = []
        for z in range(q_win.shape[1] // C):
            r = slice(z * C, (z + 1) * C)
            outs.append(fm.tail_fwd(q_win[:, r], ks_win[:, r], vr_win[:, r], K_in[:, r], V_in[:, r], o_c[:, r],
                                    lse_c[:, r], scale, window))
        return tuple(torch.cat([t[i] for t in outs], 1) for i in range(3))

    def win_tail_bwd(self, dO, q_win, ks_win, vr_win, K_in, V_in, o_c, lse_c, o, lse, C, scale,
                     dq_acc, dks_acc, dv_acc, doc_acc, dlsec_acc, window=0, init=0, dkv_out=None, raw_stash=None):
        """`tail_bwd` for every chunk of a window.  With `raw_stash` [2, B, rows, h] the raw-row gradients are left to
        `chunk_finish`: dks_acc / dv_acc are not touched and the stash receives (p_self, dss) per (row, head)."""
        if raw_stash is not None:
            ps, dss = fm.tail_self_scalars(dO, q_win, ks_win, vr_win, o, lse, scale)
            raw_stash[0].copy_(ps)
            raw_stash[1].copy_(dss)
            dks_acc, dv_acc = torch.zeros_like(dO), torch.zeros_like(dO)        # discarded
        dKs, dVs = [], []
        for z in range(q_win.shape[1] // C):
            r = slice(z * C, (z + 1) * C)
            dk, dv = self.tail_bwd(dO[:, r], q_win[:, r], ks_win[:, r], vr_win[:, r], K_in[:, r], V_in[:, r],
                                   o_c[:, r], lse_c[:, r], o[:, r], lse[:, r], scale, window, dq_acc[:, r],
                                   dks_acc[:, r], dv_acc[:, r], doc_acc[:, r], dlsec_acc[:, r], init=init)
            dKs.append(dk)
            dVs.append(dv)
        return _into(dkv_out, (torch.cat(dKs, 1), torch.cat(dVs, 1)), False)

    def win_near_dkv(self, q_all, docn_all, corrn_all, lsen_all, Kc, Vc, j0, G, C, q_lo, q_hi, span, scale, window=0,
                     out=None, accumulate=False):
        """Key side of the near reads of one step for the G key chunks j0 .. j0+G-1: chunk j is read by the
        query rows [max(q_lo, (j+1)C), min(q_hi, jC + span)).  Returns (dK, dV) [B, G*C, h, dh]: dense, or the
        views `out` written (added to when `accumulate`)."""
        outs = []
        for z in range(G):
            p0 = (j0 + z) * C
            outs.append(TorchOps.prefix_dkv(self, q_all, docn_all, corrn_all, lsen_all, Kc, Vc, p0, C, max(q_lo, p0 + C),
                                            scale, window, q_end=min(q_hi, p0 + span)))
        return _into(out, (torch.cat([a for a, _ in outs], 1), torch.cat([b for _, b in outs], 1)), accumulate)

    def cell_finish(self, do_c, dlse_c, o_c, lse_c, dK0, dV0, doc, corr, lsec, dks, dv):
        """End of a cell's backward: doc = d o_c, corr = d o_c . o_c - d lse_c, lsec = lse_c at the cell's rows
        of the per-layer arrays (views by absolute position), and dks += dK0, dv += dV0 (sweep 0 read the
        raw rows).  Returns corr as a dense [B, c, h] tensor."""
        doc.copy_(do_c)
        cv = (do_c * o_c).sum(-1) - dlse_c
        corr.copy_(cv)
        lsec.copy_(lse_c)
        dks += dK0
        dv += dV0
        return cv

    def merge_partials(self, o_f, lse_f, o_n, lse_n):
        """Log-sum-exp merge of the far partial (views by absolute position) and the near partial (dense):
        (o_c, lse_c, w_f, w_n), all dense fp32."""
        lse = torch.logaddexp(lse_f, lse_n)
        wf, wn = torch.exp(lse_f - lse), torch.exp(lse_n - lse)
        return wf.unsqueeze(-1) * o_f + wn.unsqueeze(-1) * o_n, lse, wf, wn

    def win_near_merged(self, q_win, Kc, Vc, pos0, lo, C, scale, window, o_f, lse_f, keep_near=True):
        """`win_near_fwd` followed by `merge_partials` with the chunks' far partials (o_f, lse_f: views by absolute
        position): (o_c, lse_c, w_f, w_n, o_n, lse_n); the near partial is None when `keep_near` is false."""
        o_n, lse_n = self.win_near_fwd(q_win, Kc, Vc, pos0, lo, C, scale, window)
        o_c, lse_c, w_f, w_n = self.merge_partials(o_f, lse_f, o_n, lse_n)
        return (o_c, lse_c, w_f, w_n) + ((o_n, lse_n) if keep_near else (None, None))

    def split_partials(self, do_c, dlse_c, o_f, o_c, o_n, lse_n, w_f, w_n, DOf, DLf, docn, corrn, lsen, corrn_dense=None):
        """Backward of `merge_partials`: accumulates the far gradients into DOf / DLf (+=) and writes the
        near read's (d o, corr, lse) into docn / corrn / lsen (views by absolute position); `corrn_dense`
        (contiguous, optional) receives a second copy of corr."""
        g_f = (do_c * (o_f - o_c)).sum(-1) + dlse_c
        g_n = (do_c * (o_n - o_c)).sum(-1) + dlse_c
        DOf += w_f.unsqueeze(-1) * do_c
        DLf += w_f * g_f
        do_n = w_n.unsqueeze(-1) * do_c
        docn.copy_(do_n)
        corrn.copy_((do_n * o_n).sum(-1) - w_n * g_n)
        if corrn_dense is not None:
            corrn_dense.copy_(corrn)
        lsen.copy_(lse_n)

    def chunk_finish(self, DOf, DLf, o_f, lse_f, dKp, dVp, dks, dv, doc, corr, lsec, sweeps=None, q=None, dglx=None):
        """End of a wavefront chunk's backward, all arguments views of the chunk's rows in per-layer arrays:
        the far read's accumulated gradient becomes the prefix kernels' inputs (doc = DOf, corr = DOf . o_f -
        DLf, lsec = lse_f) and the pending gradient of the chunk's raw rows moves out (dks += dKp, dv += dVp,
        dKp = dVp = 0).  `sweeps`: (d o rows, p_self, dss) of every sweep of the chunk whose raw-row gradients
        `win_tail_bwd` deferred: dv += sum p_self dO, dks += (sum dss) q.  With `dglx` ([B, R, 2d] view, written) every
        sweep tuple carries a 4th entry, the sweep's stashed d(ctx / gate logits) rows [B, R, 4d], whose gate columns
        [2d, 4d) summed over the sweeps are the gates' x-logit gradient.  Returns contiguous copies of (corr, lse_f)."""
        if dglx is not None:
            dglx.zero_()
        for t in reversed(sweeps or []):
            g, ps, dss = t[:3]
            dv += ps.unsqueeze(-1) * g.float()
            dks += dss.unsqueeze(-1) * q.float()
            if dglx is not None:
                half = t[3].shape[-1] // 2
                dglx += t[3][..., half:].float()
        cv = ((DOf * o_f).sum(-1) - DLf).contiguous()
        doc.copy_(DOf)
        corr.copy_(cv)
        lsec.copy_(lse_f)
        dks += dKp
        dv += dVp
        dKp.zero_()
        dVp.zero_()
        return cv, lse_f.contiguous()

    def copy_pair(self, d0, s0, d1, s1):
        d0.copy_(s0)
        d1.copy_(s1)

    def tail_fwd(self, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, scale, window=0):
        return fm.tail_fwd(q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, scale, window)

    def tail_bwd(self, dO, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, o, lse, scale, window,
                 dq_acc, dks_acc, dv_acc, doc_acc, dlsec_acc, init=0, dkv_out=None):
        """Accumulates (+=) into the fp32 buffers dq_acc / dks_acc / dv_acc [B,c,h,dh] (views allowed),
        doc_acc [B,c,h,dh], dlsec_acc [B,c,h]; returns fp32 (dK_in, dV_in), written into the views `dkv_out`
        when given.  `init`: bit 0 = dq_acc is overwritten instead of added to, bit 1 = the same for doc_acc and
        dlsec_acc (the first sweep processed of a cell initialises the cell's accumulators)."""
        dq, dks, dvr, dK_in, dV_in, doc, dlse = fm.tail_bwd(
            dO, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, o, lse, scale, window)
        if init & 1:
            dq_acc.copy_(dq)
        else:
            dq_acc += dq
        dks_acc += dks
        dv_acc += dvr
        if init & 2:
            doc_acc.copy_(doc)
            dlsec_acc.copy_(dlse)
        else:
            doc_acc += doc
            dlsec_acc += dlse
        return _into(dkv_out, (dK_in, dV_in), False)

    def tail_bwd_sweep(self, dO, q_r, kself_r, K_in, V_in, lse_c, o, lse, scale, window, dq_acc, init, scal):
        """`tail_bwd` with the row-scalar x row products deferred to `cell_finish_sweeps`: accumulates only the
        intra-block d q into dq_acc (written when `init`), stores this sweep's (p_self, p_c, delta) in `scal`
        [3, B, c, h] and returns fp32 (dK_in, dV_in)."""
        dq, dK_in, dV_in, ps, pc, delta = fm.tail_bwd_sweep(dO, q_r, kself_r, K_in, V_in, lse_c, o, lse, scale, window)
        if init:
            dq_acc.copy_(dq)
        else:
            dq_acc += dq
        scal[0].copy_(ps)
        scal[1].copy_(pc)
        scal[2].copy_(delta)
        return dK_in, dV_in

    def cell_finish_sweeps(self, dOs, scal, q_r, kself_r, v_raw, o_c, lse_c, dK0, dV0, doc, corr, lsec, dks, dv, dq,
                           scale):
        """End of a cell's backward after deferred sweeps (`tail_bwd_sweep`): the sums over the sweeps of d v_raw,
        d o_c, d lse_c and the self-column terms are formed here from the kept d o of every sweep, then `cell_finish`:
        doc, corr, lsec at the cell's rows (views by absolute position), dks / dv / dq += (views).  Returns corr dense."""
        dq_s, dks_s, dv_s, do_c, dlse_c = fm.cell_finish_sweeps(dOs, scal, q_r, kself_r, v_raw, o_c, scale)
        dq += dq_s
        dks += dks_s
        dv += dv_s
        return self.cell_finish(do_c, dlse_c, o_c, lse_c, dK0, dV0, doc, corr, lsec, dks, dv)

    def refine_fwd(self, raw, ssq, glx, k, v, cos, sin, h, pin_cols=0, out=None):
        """`out`: optional (K, V) [B,c,h,dh] views to write into (e.g. the cell's rows of the tape)."""
        K, V = fm.refine_fwd(raw, ssq, glx, k, v, cos, sin, h, pin_cols)
        if out is None:
            return K, V
        out[0].copy_(K)
        out[1].copy_(V)
        return out

    # ---- write law of the mult_res family (engines/fused_math.py: mrk_*) ------------------------------------
    def mrk_vin_fwd(self, raw, ssq, o, w_ctx, vgx, lam, out=None):
        """`out`: optional contiguous [B, c, d] tensor to write into (e.g. the rows of a stash)."""
        vin = fm.mrk_vin_fwd(raw, ssq, o, w_ctx, vgx, lam)
        return vin if out is None else out.copy_(vin)

    def mrk_vin_bwd(self, dvin, raw, ssq, o, w_ctx, vgx, lam, dcg, dvgx_acc):
        """Writes d v_m into dcg[..., d:2d], accumulates dvgx_acc [B,c,d] (fp32, +=); returns the direct
        path's gradient w.r.t. uhat [B,c,d] fp32."""
        d = o.shape[-1]
        dvm, dvgx, du_hat = fm.mrk_vin_bwd(dvin, raw, ssq, o, w_ctx, vgx, lam)
        dcg[..., d:2 * d].copy_(dvm)
        dvgx_acc += dvgx
        return du_hat

    def mrk_refine_fwd(self, raw, vc, ssq, glx, k, v, cos, sin, h, pin_cols, k_gain, tau, out=None):
        K, V = fm.mrk_refine_fwd(raw, vc, ssq, glx, k, v, cos, sin, h, pin_cols, k_gain, tau)
        if out is None:
            return K, V
        out[0].copy_(K)
        out[1].copy_(V)
        return out

    def mrk_refine_bwd(self, dK_out, dV_out, raw, vc, ssq, o, glx, k, v, cos, sin, pin_cols, k_gain, tau,
                       dk_acc, dv_acc, dglx_acc, dcg_out, uhat_out, dvc_out, dkg_out):
        """Accumulates dk_acc / dv_acc [B,c,d], dglx_acc [B,c,2d] (fp32, +=); writes dcg_out [B,c,4d] (its v_m
        block is filled by `mrk_vin_bwd`), uhat_out [B,c,d], dvc_out [B,c,d] and dkg_out [B,c,h] (per-row
        gradient of k_gain, summed over rows once per layer)."""
        h = dK_out.shape[2]
        d = k.shape[-1]
        dcg, dvc, dk, dv, uhat, dkg = fm.mrk_refine_bwd(dK_out, dV_out, raw, vc, ssq, o, glx, k, v, cos, sin, h,
                                                         pin_cols, k_gain, tau)
        dk_acc += dk
        dv_acc += dv
        if dglx_acc is not None:                         # None: the caller uses `stash_gate_sum` once per layer
            dglx_acc += dcg[..., 2 * d:]
        dkg_out.copy_(dkg)
        blk = dcg_out[..., d:2 * d].clone()
        dcg_out.copy_(dcg)
        dcg_out[..., d:2 * d].copy_(blk)                 # leave the v_m block to mrk_vin_bwd
        uhat_out.copy_(uhat)
        dvc_out.copy_(dvc)

    def refine_bwd(self, dK_out, dV_out, raw, ssq, o, glx, k, v, cos, sin, pin_cols, dk_acc, dv_acc, dglx_acc,
                   dcg_out, uhat_out):
        """Accumulates dk_acc / dv_acc [B,c,d] and dglx_acc [B,c,2d] (fp32, +=); writes the
        gradient of the ctx/gate logits into dcg_out [B,c,4d] and the normalised read o*rstd
        into uhat_out [B,c,d] (both activation dtype; rows of the layer's deferred-dW stash)."""
        dcg, dk, dv, uhat = fm.refine_bwd(dK_out, dV_out, raw, ssq, o, glx, k, v, cos, sin, pin_cols)
        d = k.shape[-1]
        dk_acc += dk
        dv_acc += dv
        if dglx_acc is not None:                         # None: the caller uses `stash_gate_sum` once per layer
            dglx_acc += dcg[..., 2 * d:]
        dcg_out.copy_(dcg)
        uhat_out.copy_(uhat)

    def stash_gate_sum(self, dcg_stash, B, T, c, K):
        """Gradient of the gates' x-logits [B, T, 2d] (activation dtype) from the layer's stash of d(ctx / gate
        logits) [n_cells * K * B * c, 4d], whose rows are ordered (cell, sweep, batch, row): the sum over the
        sweeps of the gate columns (a gate's x-logit and u-logit share one gradient)."""
        d = dcg_stash.shape[1] // 4
        g = dcg_stash.view(T // c, K, B, c, 4 * d)[..., 2 * d:].float().sum(1)        # [cells, B, c, 2d]
        return g.permute(1, 0, 2, 3).reshape(B, T, 2 * d).to(dcg_stash.dtype)

    def embed_bwd(self, gw, idx, dx):
        """gw (fp32 [V, d]) += scatter of dx rows [N, d] by token id idx [N]."""
        gw.index_add_(0, idx.reshape(-1), dx.reshape(-1, dx.shape[-1]).float())

    def col_dot_acc(self, out, a, b):
        """out (fp32 [n]) += column sums of a * b, both [rows, n]."""
        out.add_((a.reshape(-1, a.shape[-1]).float() * b.reshape(-1, b.shape[-1]).float()).sum(0))

    def rmsn_bwd(self, du, o, ssq, residual=None, out_dtype=torch.float32, extra=None):
        """d o of the gain-free row normalisation (+ residual), in out_dtype.  `extra`: fp32 term added to du."""
        if extra is not None:
            du = du.float() + extra
        dx = fm.rmsn_bwd(du, o, ssq)
        if residual is not None:
            dx = dx + residual.float()
        return dx.to(out_dtype)

    # ---- head ---------------------------------------------------------------------------
    def ce_chunk(self, logits, targets, inv_n):
        return fm.ce_chunk(logits, targets, inv_n)
