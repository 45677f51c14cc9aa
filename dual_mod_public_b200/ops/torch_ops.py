"""Op table in plain torch: the CPU/fallback implementation of every device op
the fused engines call.  `CudaOps` (cuda_ops.py) overrides entries with the
sm_100a kernels; the numerics tests compare the two entry by entry."""

from __future__ import annotations

import torch

from ..engines import fused_math as fm


class TorchOps:
    name = "torch"
    launches = 0                      # custom-kernel launch counter (0 here by construction)

    # ---- GEMMs ------------------------------------------------------------------
    def linear(self, x, w, bias=None, out_dtype=None):
        """x [..., k] @ w[n, k]^T (+ bias)."""
        y = x @ w.t()
        if bias is not None:
            y = y + bias.to(y.dtype)
        return y if out_dtype is None else y.to(out_dtype)

    def linear_dx(self, dy, w):
        """dy [..., n] @ w[n, k] -> [..., k]"""
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
    def prefix_fwd(self, q_r, Kc, Vc, pos0, scale, window=0):
        return fm.prefix_fwd(q_r, Kc, Vc, pos0, scale, window)

    def prefix_bwd(self, q_r, Kc, Vc, pos0, scale, window, o_c, lse_c, do_c, dlse_c, dq_acc, dKc, dVc):
        return fm.prefix_bwd(q_r, Kc, Vc, pos0, scale, window, o_c, lse_c, do_c, dlse_c,
                             dq_acc, dKc, dVc)

    def prefix_dq(self, q_r, Kc, Vc, pos0, scale, window, lse_c, do_c, corr, dq_acc):
        return fm.prefix_dq(q_r, Kc, Vc, pos0, scale, window, lse_c, do_c, corr, dq_acc)

    def prefix_dkv(self, q_all, doc_all, corr_all, lsec_all, Kc, Vc, pos0, c, q_start, scale, window=0, q_end=None):
        return fm.prefix_dkv(q_all, doc_all, corr_all, lsec_all, Kc, Vc, pos0, c, q_start, scale, window, q_end)

    def tail_fwd(self, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, scale, window=0):
        return fm.tail_fwd(q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, scale, window)

    def tail_bwd(self, dO, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, o, lse, scale, window,
                 dq_acc, dks_acc, dv_acc, doc_acc, dlsec_acc):
        """Accumulates (+=) into the fp32 buffers dq_acc / dks_acc / dv_acc [B,c,h,dh],
        doc_acc [B,c,h,dh], dlsec_acc [B,c,h]; returns fp32 (dK_in, dV_in)."""
        dq, dks, dvr, dK_in, dV_in, doc, dlse = fm.tail_bwd(
            dO, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, o, lse, scale, window)
        dq_acc += dq
        dks_acc += dks
        dv_acc += dvr
        doc_acc += doc
        dlsec_acc += dlse
        return dK_in, dV_in

    def refine_fwd(self, raw, ssq, glx, k, v, cos, sin, h, pin_cols=0):
        return fm.refine_fwd(raw, ssq, glx, k, v, cos, sin, h, pin_cols)

    def refine_bwd(self, dK_out, dV_out, raw, ssq, o, glx, k, v, cos, sin, pin_cols, dk_acc, dv_acc, dglx_acc,
                   dcg_out, uhat_out):
        """Accumulates dk_acc / dv_acc [B,c,d] and dglx_acc [B,c,2d] (fp32, +=); writes the
        gradient of the ctx/gate logits into dcg_out [B,c,4d] and the normalised read o*rstd
        into uhat_out [B,c,d] (both activation dtype; rows of the layer's deferred-dW stash)."""
        dcg, dk, dv, uhat = fm.refine_bwd(dK_out, dV_out, raw, ssq, o, glx, k, v, cos, sin, pin_cols)
        d = k.shape[-1]
        dk_acc += dk
        dv_acc += dv
        dglx_acc += dcg[..., 2 * d:]
        dcg_out.copy_(dcg)
        uhat_out.copy_(uhat)

    def rmsn_bwd(self, du, o, ssq, residual=None, out_dtype=torch.float32):
        """d o of the gain-free row normalisation (+ residual), in out_dtype."""
        dx = fm.rmsn_bwd(du, o, ssq)
        if residual is not None:
            dx = dx + residual.float()
        return dx.to(out_dtype)

    # ---- head ---------------------------------------------------------------------------
    def ce_chunk(self, logits, targets, inv_n):
        return fm.ce_chunk(logits, targets, inv_n)
