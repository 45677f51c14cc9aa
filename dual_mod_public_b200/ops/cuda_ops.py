"""sm_100a op table: ctypes bindings of `libdmb200.so` behind the `TorchOps` interface.

Every method runs the hand-written kernel when the operands are in the layout
it was built for (bf16 activations, head_dim 64/128, chunk 16/32/64, ...), and
otherwise defers to the plain-torch statement of the same op, so exotic shapes
stay correct.  `launches` counts kernel launches issued by this table.
"""

from __future__ import annotations

import ctypes
import os

import torch

from .torch_ops import TorchOps

_LIB = None
_HERE = os.path.dirname(os.path.abspath(__file__))


class TView(ctypes.Structure):
    _fields_ = [("bs", ctypes.c_longlong), ("rs", ctypes.c_longlong)]


def load_library():
    """Load (building if needed and possible) the kernel library; raises when it
    cannot be had — a GPU run must never silently fall back."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.path.join(_HERE, "libdmb200.so")
    if not os.path.exists(path):
        from .build import build
        build()
    _LIB = ctypes.CDLL(path)
    for name in dir(_Sigs):
        if name.startswith("dmb_"):
            fn = getattr(_LIB, name)
            fn.restype = ctypes.c_int
            fn.argtypes = getattr(_Sigs, name)
    return _LIB


_p, _i, _f, _ll, _v = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong, TView


class _Sigs:
    dmb_rms_fwd = [_p, _ll, _p, _p, _p, _i, _i, _f, _p]
    dmb_rms_bwd_dx = [_p, _i, _p, _ll, _p, _p, _p, _p, _i, _i, _i, _p]
    dmb_col_reduce_acc = [_p, _i, _p, _ll, _p, _p, _i, _p, _i, _i, _p]
    dmb_embed_bwd_sorted = [_p, _p, _p, _i, _p, _i, _i, _p]
    dmb_rope = [_p, _i, _ll, _ll, _p, _p, _p, _i, _i, _i, _i, _i, _f, _p]
    dmb_refine_fwd = [_p, _p, _p, _v, _p, _v, _p, _v, _p, _p, _p, _p, _v, _i, _i, _i, _i, _i, _f, _p]
    dmb_refine_bwd = [_p, _p, _v, _p, _p, _p, _p, _v, _p, _v, _p, _v, _p, _p, _p, _p, _p, _v, _p, _v, _p, _v,
                      _i, _i, _i, _i, _i, _f, _p]
    dmb_stash_gate_sum = [_p, _p, _i, _i, _i, _i, _i, _p]
    dmb_rmsn_bwd = [_p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _p]
    dmb_mrk_vin_fwd = [_p, _p, _p, _p, _p, _v, _p, _i, _i, _i, _i, _f, _f, _p]
    dmb_mrk_vin_bwd = [_p, _p, _p, _p, _p, _v, _p, _p, _v, _p, _i, _i, _i, _i, _f, _f, _p]
    dmb_mrk_refine_fwd = [_p, _p, _p, _p, _v, _p, _v, _p, _v, _p, _p, _p, _p, _p, _v, _i, _i, _i, _i, _i, _f, _f, _p]
    dmb_mrk_refine_bwd = [_p, _p, _v, _p, _p, _p, _p, _p, _v, _p, _v, _p, _v, _p, _p, _p, _p, _p, _p, _p, _p, _v, _p, _v,
                          _p, _v, _i, _i, _i, _i, _i, _f, _f, _p]
    dmb_swiglu_fwd = [_p, _p, _p, _ll, _p]
    dmb_swiglu_bwd = [_p, _p, _p, _p, _p, _ll, _p]
    dmb_ce = [_p, _p, _p, _p, _p, _i, _i, _p]
    dmb_tail_fwd = [_p, _v, _p, _v, _p, _v, _p, _v, _p, _v, _p, _p, _p, _p, _p, _i, _i, _i, _i, _f, _i, _i, _i, _p]
    dmb_tail_bwd = [_p, _p, _v, _p, _v, _p, _v, _p, _v, _p, _v, _p, _p, _p, _p, _p, _v, _p, _v, _p, _v,
                    _p, _p, _p, _p, _v, _i, _i, _i, _i, _f, _i, _i, _i, _i, _p]
    dmb_prefix_fwd = [_p, _v, _p, _p, _v, _p, _p, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _p]
    dmb_prefix_dkv = [_p, _p, _p, _p, _p, _p, _v, _p, _p, _v, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _p]
    dmb_cell_finish = [_p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _ll, _ll, _i, _i, _i, _i, _p]
    dmb_wave_merge_fwd = [_p, _p, _ll, _ll, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _p]
    dmb_wave_split_bwd = [_p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _ll, _ll, _i, _i, _i, _i, _p]
    dmb_attn_fwd_tc_merged = [_p, _v, _i, _p, _p, _v, _i, _p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i,
                              _i, _i, _p, _p, _ll, _ll, _p, _p, _p, _p, _p, _p]
    dmb_attn_dkv_rows128 = [_i]
    dmb_cell_finish_sweeps = [_p, _i, _p, _p, _v, _p, _v, _p, _v, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _p, _p, _f, _ll,
                              _ll, _i, _i, _i, _i, _p]
    dmb_wave_chunk_finish = [_p, _p, _p, _p, _p, _p, _p, _p, _p, _i, _p, _p, _p, _p, _ll, _ll, _i, _i, _i, _i, _i, _p, _p,
                             _p, _p, _p, _p, _v, _p, _p, _ll, _p]
    dmb_copy_pair = [_p, _p, _p, _p, _ll, _ll, _ll, _i, _p]
    dmb_prefix_dq = [_p, _v, _p, _v, _p, _p, _v, _p, _p, _p, _v, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i, _i, _p]
    dmb_attn_dq_tc = [_p, _v, _p, _v, _i, _p, _p, _v, _i, _p, _p, _p, _v, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _p, _p]
    dmb_attn_dkv_tc = [_p, _p, _p, _p, _i, _p, _p, _v, _i, _p, _p, _v, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _p, _p]
    dmb_attn_fwd_tc = [_p, _v, _i, _p, _p, _v, _i, _p, _i, _p, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _i, _i, _i,
                       _i, _i, _p, _p]


BF16 = torch.bfloat16
F32 = torch.float32


def _tv(t: torch.Tensor) -> TView:
    """(batch stride, row stride) of a [B, rows, ...] tensor whose trailing dims are dense."""
    return TView(t.stride(0), t.stride(1))


def _dense_tail(t: torch.Tensor, n_tail: int) -> bool:
    """True when the last n_tail dims are laid out densely (row-contiguous)."""
    exp = 1
    for i in range(1, n_tail + 1):
        if t.shape[-i] != 1 and t.stride(-i) != exp:
            return False
        exp *= t.shape[-i]
    return True


class CudaOps(TorchOps):
    name = "sm100a"

    def __init__(self, device):
        self.device = torch.device(device)
        self.lib = load_library()
        self.launches = 0
        self.lib_gemms = 0                     # plain products handed to the library GEMM (see LIB_NARROW)
        self.fallbacks = {}                    # op name -> calls that took the torch statement instead of a kernel
        self._scratch = {}
        self.gemm = None                       # set by enable_gemm()
        self.strict = os.environ.get("DMB_STRICT_OPS", "0") == "1"
        self._tc_err = torch.zeros(1, dtype=torch.int32, device=self.device)   # raised by the tcgen05 attention kernels
        if os.environ.get("DMB_GEMM", "tcgen05") == "tcgen05":
            from .gemm import Tcgen05Gemm
            self.gemm = Tcgen05Gemm(self.lib, self.device)

    # ---- helpers ---------------------------------------------------------------------------
    def dkv_rows128(self, on=None):
        """The key-side tcgen05 attention backward at head dim 64 streams its readers in tiles of 128 rows (default) or
        of 64 (`on=False`); returns the previous setting.  A process-wide switch of the kernel library."""
        return bool(self.lib.dmb_attn_dkv_rows128(-1 if on is None else int(bool(on))))

    def _fell_back(self, name):
        """A call whose arguments the kernel does not take (layout, dtype, size) runs the torch statement; it is
        counted so that a hot path that silently left the kernels shows up (`fallbacks`, `DMB_STRICT_OPS=1` raises)."""
        self.fallbacks[name] = self.fallbacks.get(name, 0) + 1
        if self.strict:
            raise RuntimeError(f"{name}: arguments not accepted by the sm_100a kernel (DMB_STRICT_OPS=1)")

    def _st(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _ck(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed with code {rc}")
        self.launches += 1

    def _scratch_f32(self, key, n):
        buf = self._scratch.get(key)
        if buf is None or buf.numel() < n:
            buf = torch.empty(n, dtype=F32, device=self.device)
            self._scratch[key] = buf
        return buf

    # ---- GEMMs -------------------------------------------------------------------------------
    # The factor products of a low-rank write law (rank 120-144: an up factor has a reduction of 2.25 k-blocks, a down
    # factor fills half an output tile) are plain bf16 GEMMs outside this kernel's tile shapes; callers mark them
    # `narrow` and they go to the library GEMM (torch.mm: cuBLAS).  Measured at the 1.3B recipe's window of 8192 rows
    # (`bench_ops --only gemm_lora`): own kernel / library = 52.7 / 33.8 us (stacked down factors), 25.8 / 19.8 (one
    # up factor), 24.0 / 17.4 (one down factor), 25.0 / 17.4 and 30.6 / 28.2 (their input gradients).
    # DMB_GEMM_NARROW=own keeps them on the tcgen05 kernel.
    LIB_NARROW = os.environ.get("DMB_GEMM_NARROW", "lib") == "lib"

    def _lib_mm(self, a, b, out, shape):
        """a [M, K] @ b [K, N] through the library into `out` (a [M, N] view with a dense last dim) or a new tensor."""
        self.lib_gemms += 1
        if out is not None:
            return torch.mm(a, b, out=out)
        return torch.mm(a, b).view(shape)

    @staticmethod
    def _rows2d(t):
        if t.dim() == 2:
            return t if t.stride(1) == 1 else None
        return t.reshape(-1, t.shape[-1]) if t.is_contiguous() else None

    def linear(self, x, w, bias=None, out_dtype=None, out=None, narrow=False):
        if (narrow and self.LIB_NARROW and x.is_cuda and x.dtype == BF16 and w.dtype == BF16
                and out_dtype in (None, BF16) and (out is None or out.dtype == BF16)
                and (bias is None or (bias.dtype == BF16 and out is None))):
            x2 = self._rows2d(x)
            if x2 is not None and (out is None or (out.dim() == 2 and out.stride(1) == 1)):
                if bias is not None:
                    self.lib_gemms += 1
                    return torch.addmm(bias, x2, w.t()).view(x.shape[:-1] + (w.shape[0],))
                return self._lib_mm(x2, w.t(), out, x.shape[:-1] + (w.shape[0],))
        if (self.gemm is not None and self.gemm.ok_tn(x, w) and (bias is None or bias.dtype == BF16)
                and (out is None or self.gemm.ok_out(out, x, w.shape[0]))):
            y = self.gemm.linear(x, w, out_dtype or x.dtype, bias=bias, out=out)
            self.launches += 1
            return y
        self._fell_back("linear")
        return super().linear(x, w, bias, out_dtype, out)

    def linear_dx(self, dy, w, out=None, narrow=False):
        if (narrow and self.LIB_NARROW and dy.is_cuda and dy.dtype == BF16 and w.dtype == BF16
                and (out is None or out.dtype == BF16)):
            d2 = self._rows2d(dy)
            if d2 is not None and (out is None or (out.dim() == 2 and out.stride(1) == 1)):
                return self._lib_mm(d2, w, out, dy.shape[:-1] + (w.shape[1],))
        if self.gemm is not None and self.gemm.ok_nn(dy, w) and (out is None or self.gemm.ok_out(out, dy, w.shape[1])):
            self.launches += 1
            return self.gemm.linear_dx(dy, w, out=out)
        self._fell_back("linear_dx")
        return super().linear_dx(dy, w, out)

    def linear_dw_acc(self, dW, dy, x):
        if self.gemm is not None and self.gemm.ok_tn_dw(dW, dy, x):
            self.launches += 1
            return self.gemm.linear_dw_acc(dW, dy, x)
        self._fell_back("linear_dw_acc")
        return super().linear_dw_acc(dW, dy, x)

    # ---- norms ------------------------------------------------------------------------------------
    def rms_fwd(self, x, w, eps=1e-5):
        d = x.shape[-1]
        if x.dtype != BF16 or d % 8:
            self._fell_back("rms_fwd")
            return super().rms_fwd(x, w, eps)
        if not x.is_contiguous():
            x = x.contiguous()
        x2 = x.view(-1, d)
        rows = x2.shape[0]
        y = torch.empty(rows, d, dtype=BF16, device=x.device)
        rstd = torch.empty(rows, dtype=F32, device=x.device)
        self._ck(self.lib.dmb_rms_fwd(x2.data_ptr(), x2.stride(0), w.data_ptr(), y.data_ptr(),
                                      rstd.data_ptr(), rows, d, eps, self._st()), "rms_fwd")
        return y.view(*x.shape), rstd.view(*x.shape[:-1], 1)

    def rms_bwd(self, dy, x, w, rstd, dw_acc, residual=None, out_dtype=F32):
        d = x.shape[-1]
        ok = (x.dtype == BF16 and dy.dtype in (BF16, F32) and out_dtype in (BF16, F32)
              and x.is_contiguous() and dy.is_contiguous()
              and (residual is None or (residual.is_contiguous() and residual.dtype == out_dtype)))
        if not ok:
            self._fell_back("rms_bwd")
            return super().rms_bwd(dy, x, w, rstd, dw_acc, residual, out_dtype)
        rows = x.numel() // d
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        rs = rstd.reshape(-1)
        self._ck(self.lib.dmb_rms_bwd_dx(dy.data_ptr(), int(dy.dtype == F32), x.data_ptr(), d,
                                         w.data_ptr(), rs.data_ptr(),
                                         residual.data_ptr() if residual is not None else None,
                                         out.data_ptr(), int(out_dtype == F32), rows, d, self._st()),
                 "rms_bwd_dx")
        nsplit = max(1, min(64, rows // 64))
        part = self._scratch_f32("col", nsplit * d)
        self._ck(self.lib.dmb_col_reduce_acc(dy.data_ptr(), int(dy.dtype == F32), x.data_ptr(), d,
                                             rs.data_ptr(), part.data_ptr(), nsplit, dw_acc.data_ptr(),
                                             rows, d, self._st()), "rms_bwd_dw")
        self.launches += 1
        return out

    def col_sum_acc(self, out, dy):
        n = dy.shape[-1]
        if dy.dtype not in (BF16, F32) or not dy.is_contiguous():
            self._fell_back("col_sum_acc")
            return super().col_sum_acc(out, dy)
        rows = dy.numel() // n
        nsplit = max(1, min(64, rows // 64))
        part = self._scratch_f32("col", nsplit * n)
        self._ck(self.lib.dmb_col_reduce_acc(dy.data_ptr(), int(dy.dtype == F32), None, 0, None,
                                             part.data_ptr(), nsplit, out.data_ptr(), rows, n,
                                             self._st()), "col_sum")
        self.launches += 1

    def embed_bwd(self, gw, idx, dx):
        d = dx.shape[-1]
        if dx.dtype not in (BF16, F32) or not dx.is_contiguous() or not gw.is_contiguous() or d % 4:
            self._fell_back("embed_bwd")
            return super().embed_bwd(gw, idx, dx)
        tok, order = torch.sort(idx.reshape(-1), stable=True)
        self._ck(self.lib.dmb_embed_bwd_sorted(tok.data_ptr(), order.data_ptr(), dx.data_ptr(), int(dx.dtype == F32),
                                               gw.data_ptr(), tok.numel(), d, self._st()), "embed_bwd")

    def col_dot_acc(self, out, a, b):
        n = a.shape[-1]
        if a.dtype != BF16 or b.dtype != BF16 or not a.is_contiguous() or not b.is_contiguous():
            self._fell_back("col_dot_acc")
            return super().col_dot_acc(out, a, b)
        rows = a.numel() // n
        nsplit = max(1, min(64, rows // 64))
        part = self._scratch_f32("col", nsplit * n)
        ones = self._scratch_f32("ones", rows)
        if not getattr(self, "_ones_rows", 0) >= rows:
            ones.fill_(1.0)
            self._ones_rows = rows
        self._ck(self.lib.dmb_col_reduce_acc(a.data_ptr(), 0, b.data_ptr(), n, ones.data_ptr(), part.data_ptr(), nsplit,
                                             out.data_ptr(), rows, n, self._st()), "col_dot")
        self.launches += 1

    # ---- write law of the mult_res family ---------------------------------------------------------------------
    def _mrk_ok(self, k, raw, *views):
        B, c, d = k.shape
        return (k.dtype == BF16 and raw.dtype == BF16 and raw.is_contiguous()
                and all(_dense_tail(t, 1) for t in (k,) + views))

    def mrk_vin_fwd(self, raw, ssq, o, w_ctx, vgx, lam, out=None):
        B, c, d = o.shape
        h = ssq.shape[-1]
        dh = d // h
        if not (self._mrk_ok(o, raw, vgx) and o.is_contiguous() and ssq.is_contiguous() and w_ctx.dtype == BF16
                and vgx.dtype == BF16 and dh % 16 == 0
                and (out is None or (out.dtype == BF16 and out.is_contiguous() and out.shape == (B, c, d)))):
            self._fell_back("mrk_vin_fwd")
            return super().mrk_vin_fwd(raw, ssq, o, w_ctx, vgx, lam, out)
        vin = out if out is not None else torch.empty(B, c, d, dtype=BF16, device=o.device)
        self._ck(self.lib.dmb_mrk_vin_fwd(raw.data_ptr(), ssq.data_ptr(), o.data_ptr(), w_ctx.data_ptr(), vgx.data_ptr(),
                                          _tv(vgx), vin.data_ptr(), B, c, h, dh, lam, 1e-5, self._st()), "mrk_vin_fwd")
        self.launches += 1
        return vin

    def mrk_vin_bwd(self, dvin, raw, ssq, o, w_ctx, vgx, lam, dcg, dvgx_acc):
        B, c, d = o.shape
        h = ssq.shape[-1]
        dh = d // h
        ok = (self._mrk_ok(o, raw, vgx, dvgx_acc) and dvin.dtype == BF16 and dvin.is_contiguous() and dcg.is_contiguous()
              and dcg.dtype == BF16 and ssq.is_contiguous() and w_ctx.dtype == BF16 and vgx.dtype == BF16
              and dvgx_acc.dtype == F32 and dh % 16 == 0)
        if not ok:
            self._fell_back("mrk_vin_bwd")
            return super().mrk_vin_bwd(dvin, raw, ssq, o, w_ctx, vgx, lam, dcg, dvgx_acc)
        du_hat = torch.empty(B, c, d, dtype=F32, device=o.device)
        self._ck(self.lib.dmb_mrk_vin_bwd(dvin.data_ptr(), raw.data_ptr(), ssq.data_ptr(), w_ctx.data_ptr(), vgx.data_ptr(),
                                          _tv(vgx), dcg.data_ptr(), dvgx_acc.data_ptr(), _tv(dvgx_acc), du_hat.data_ptr(),
                                          B, c, h, dh, lam, 1e-5, self._st()), "mrk_vin_bwd")
        self.launches += 1
        return du_hat

    def mrk_refine_fwd(self, raw, vc, ssq, glx, k, v, cos, sin, h, pin_cols, k_gain, tau, out=None):
        B, c, d = k.shape
        dh = d // h
        ok = (self._mrk_ok(k, raw, glx, v) and vc.dtype == BF16 and vc.is_contiguous() and cos.is_contiguous() and cos.dtype == F32 and sin.dtype == F32
              and ssq.is_contiguous() and k_gain.dtype == F32 and dh % 16 == 0)
        if not ok:
            self._fell_back("mrk_refine_fwd")
            return super().mrk_refine_fwd(raw, vc, ssq, glx, k, v, cos, sin, h, pin_cols, k_gain, tau, out)
        if (out is not None and all(t.dtype == BF16 and _dense_tail(t, 2) for t in out)
                and out[0].stride() == out[1].stride()):
            K_out, V_out = out
        else:
            K_out = torch.empty(B, c, h, dh, dtype=BF16, device=k.device)
            V_out = torch.empty(B, c, h, dh, dtype=BF16, device=k.device)
        self._ck(self.lib.dmb_mrk_refine_fwd(raw.data_ptr(), vc.data_ptr(), ssq.data_ptr(), glx.data_ptr(), _tv(glx),
                                             k.data_ptr(), _tv(k), v.data_ptr(), _tv(v), cos.data_ptr(), sin.data_ptr(),
                                             k_gain.data_ptr(), K_out.data_ptr(), V_out.data_ptr(), _tv(K_out), B, c, h, dh,
                                             pin_cols, float(tau or 0.0), 1e-5, self._st()), "mrk_refine_fwd")
        self.launches += 1
        if out is not None and K_out is not out[0]:
            out[0].copy_(K_out)
            out[1].copy_(V_out)
            return out
        return K_out, V_out

    def mrk_refine_bwd(self, dK_out, dV_out, raw, vc, ssq, o, glx, k, v, cos, sin, pin_cols, k_gain, tau,
                       dk_acc, dv_acc, dglx_acc, dcg_out, uhat_out, dvc_out, dkg_out):
        B, c, d = k.shape
        h = dK_out.shape[2]
        dh = d // h
        views = (glx, v, dk_acc, dv_acc) + ((dglx_acc,) if dglx_acc is not None else ())
        ok = (self._mrk_ok(k, raw, *views) and vc.dtype == BF16 and vc.is_contiguous()
              and o.dtype == BF16 and o.is_contiguous() and dK_out.dtype == F32 and dV_out.dtype == F32
              and _dense_tail(dK_out, 2) and dK_out.stride() == dV_out.stride() and ssq.is_contiguous()
              and all(t.is_contiguous() and t.dtype == BF16 for t in (dcg_out, uhat_out, dvc_out))
              and dkg_out.is_contiguous() and dkg_out.dtype == F32 and k_gain.dtype == F32
              and cos.is_contiguous() and cos.dtype == F32 and sin.dtype == F32 and dh % 16 == 0)
        if not ok:
            self._fell_back("mrk_refine_bwd")
            return super().mrk_refine_bwd(dK_out, dV_out, raw, vc, ssq, o, glx, k, v, cos, sin, pin_cols, k_gain, tau,
                                          dk_acc, dv_acc, dglx_acc, dcg_out, uhat_out, dvc_out, dkg_out)
        self._ck(self.lib.dmb_mrk_refine_bwd(
            dK_out.data_ptr(), dV_out.data_ptr(), _tv(dK_out), raw.data_ptr(), vc.data_ptr(), ssq.data_ptr(), o.data_ptr(),
            glx.data_ptr(), _tv(glx), k.data_ptr(), _tv(k), v.data_ptr(), _tv(v), cos.data_ptr(), sin.data_ptr(),
            k_gain.data_ptr(), dcg_out.data_ptr(), uhat_out.data_ptr(), dvc_out.data_ptr(), dkg_out.data_ptr(),
            dk_acc.data_ptr(), _tv(dk_acc), dv_acc.data_ptr(), _tv(dv_acc),
            dglx_acc.data_ptr() if dglx_acc is not None else None,
            _tv(dglx_acc) if dglx_acc is not None else TView(0, 0),
            B, c, h, dh, pin_cols, float(tau or 0.0), 1e-5, self._st()), "mrk_refine_bwd")
        self.launches += 1

    # ---- rope -----------------------------------------------------------------------------------------
    def _rope(self, x, cos, sin, sign, out_dtype):
        B, T, H, DH = x.shape
        if (x.dtype not in (BF16, F32) or not _dense_tail(x, 2) or not cos.is_contiguous() or not sin.is_contiguous()
                or cos.dtype != F32 or sin.dtype != F32):
            return None
        out = torch.empty(B, T, H, DH, dtype=out_dtype, device=x.device)
        self._ck(self.lib.dmb_rope(x.data_ptr(), int(x.dtype == F32), x.stride(0), x.stride(1),
                                   cos.data_ptr(), sin.data_ptr(), out.data_ptr(),
                                   int(out_dtype == F32), B, T, H, DH, sign, self._st()), "rope")
        return out

    def rope(self, x, cos, sin):
        out = self._rope(x, cos, sin, 1.0, x.dtype) if x.is_cuda else None
        return out if out is not None else super().rope(x, cos, sin)

    def unrope(self, x, cos, sin):
        out = self._rope(x, cos, sin, -1.0, x.dtype) if x.is_cuda else None
        return out if out is not None else super().unrope(x, cos, sin)

    # ---- swiglu ------------------------------------------------------------------------------------------
    def swiglu_fwd(self, h1, h3):
        if h1.dtype != BF16 or not (h1.is_contiguous() and h3.is_contiguous()) or h1.numel() % 8:
            self._fell_back("swiglu_fwd")
            return super().swiglu_fwd(h1, h3)
        g = torch.empty_like(h1)
        self._ck(self.lib.dmb_swiglu_fwd(h1.data_ptr(), h3.data_ptr(), g.data_ptr(), h1.numel(),
                                         self._st()), "swiglu_fwd")
        return g

    def swiglu_bwd(self, dg, h1, h3):
        if h1.dtype != BF16 or dg.dtype != BF16 or h1.numel() % 8 or not (
                dg.is_contiguous() and h1.is_contiguous() and h3.is_contiguous()):
            self._fell_back("swiglu_bwd")
            return super().swiglu_bwd(dg, h1, h3)
        d1, d3 = torch.empty_like(h1), torch.empty_like(h3)
        self._ck(self.lib.dmb_swiglu_bwd(dg.data_ptr(), h1.data_ptr(), h3.data_ptr(), d1.data_ptr(),
                                         d3.data_ptr(), h1.numel(), self._st()), "swiglu_bwd")
        return d1, d3

    # ---- CE ---------------------------------------------------------------------------------------------------
    def ce_chunk(self, logits, targets, inv_n):
        if logits.dtype != BF16 or not logits.is_contiguous() or not torch.is_tensor(inv_n):
            self._fell_back("ce_chunk")
            return super().ce_chunk(logits, targets, inv_n)
        n, V = logits.shape
        row_loss = torch.empty(n, dtype=F32, device=logits.device)
        dlog = torch.empty_like(logits)
        inv = inv_n.to(F32).reshape(1)
        self._ck(self.lib.dmb_ce(logits.data_ptr(), targets.contiguous().data_ptr(), inv.data_ptr(),
                                 row_loss.data_ptr(), dlog.data_ptr(), n, V, self._st()), "ce")
        return row_loss.sum(), dlog

    # ---- cell ops ------------------------------------------------------------------------------------------------
    @staticmethod
    def _cell_ok(q_r):
        B, c, h, dh = q_r.shape
        return q_r.dtype == BF16 and dh in (64, 128) and c in (16, 32, 64)

    def prefix_fwd(self, q_r, Kc, Vc, pos0, scale, window=0, out=None, qoff=0):
        from ..engines.fused_math import prefix_lo
        B, c, h, dh = q_r.shape
        lo = prefix_lo(pos0, window, qoff)
        if not self._cell_ok(q_r) or pos0 - lo <= 0 or not (_dense_tail(q_r, 2) and _dense_tail(Kc, 2)):
            self._fell_back("prefix_fwd")
            return super().prefix_fwd(q_r, Kc, Vc, pos0, scale, window, out, qoff)
        if out is not None and out[0].is_contiguous() and out[1].is_contiguous() and out[0].dtype == F32:
            o_c, lse_c = out
        else:
            o_c = torch.empty(B, c, h, dh, dtype=F32, device=q_r.device)
            lse_c = torch.empty(B, c, h, dtype=F32, device=q_r.device)
        if self._tc("fwd") and c == 64 and self._tc_ok(q_r, Kc, Vc):
            self.attn_fwd_tc(q_r, Kc, Vc, lo, pos0, pos0 + qoff, scale, window, Lq=c, bm=64, out=(o_c, lse_c))
            if out is not None and o_c is not out[0]:
                out[0].copy_(o_c)
                out[1].copy_(lse_c)
                return out
            return o_c, lse_c
        self._ck(self.lib.dmb_prefix_fwd(q_r.data_ptr(), _tv(q_r), Kc.data_ptr(), Vc.data_ptr(), _tv(Kc),
                                         o_c.data_ptr(), lse_c.data_ptr(), B, c, h, dh, lo, pos0,
                                         scale, window, 1, 0, qoff, self._st()), "prefix_fwd")
        if out is not None and o_c is not out[0]:
            out[0].copy_(o_c)
            out[1].copy_(lse_c)
            return out
        return o_c, lse_c

    # Which of the 64-row tape reads (a cell's prefix read, the wavefront's far and near reads) and their
    # backward sides go through the tcgen05 kernels of csrc/attn_tc.cu instead of the warp-MMA kernels.
    # Default: all three; measured at the 340M cell shape (32 sequences x 16 heads of 64, 1024 keys / later
    # queries), tcgen05 against warp MMA: forward 47 vs 66 us, key side 59 vs 109 us, query side 64 vs 90 us (the
    # backward sides with their 128-row streamed tiles; with 64-row tiles the query side was slower than warp MMA).
    # DMB_ATTN_TC: comma list of fwd / dq / dkv, "1" or "all" = all, "0" = none.
    _tc_env = os.environ.get("DMB_ATTN_TC", "all").lower()
    ATTN_TC = (frozenset(("fwd", "dq", "dkv")) if _tc_env in ("1", "all") else
               frozenset() if _tc_env in ("0", "", "none") else frozenset(x.strip() for x in _tc_env.split(",")))

    # near reads of a window with two chunks per 128-row tile (the union of their key ranges streams through, each half
    # masks to its own): measured no faster than one chunk per 64-row tile at the 1.3B recipe's window (192 vs 184 us),
    # so off by default
    NEAR_PAIRS = os.environ.get("DMB_NEAR_PAIRS", "0") == "1"

    def _tc(self, side):
        """ATTN_TC may also be set to True / False on an instance (tests, benchmarks): all sides / none."""
        a = self.ATTN_TC
        return a if isinstance(a, bool) else side in a

    def attn_fwd_tc(self, q, Kc, Vc, lo, hi, qbase, scale, window=0, causal=False, causal_excl=1, Lq=None, G=1,
                    grow=0, bm=None, out_dtype=F32, out=None, pair_shift=0):
        """Attention forward on tcgen05 (csrc/attn_tc.cu).  q: [B, rows, h, dh] bf16 view; group z (of G) takes
        its rows [z*grow, z*grow + Lq), sits at positions qbase + z*grow + i and reads the tape rows
        max(0, lo + z*grow) <= j < hi + z*grow of Kc / Vc [B, T, h, dh], under the causal rule
        j <= position - causal_excl and the sliding window j > position - window.  `pair_shift` (with Lq = bm = 128):
        each group is two 64-row groups sharing a tile; the second one's key range is shifted by pair_shift rows.
        Returns (o [B, G, Lq, h, dh] in out_dtype, lse [B, G, Lq, h] fp32)."""
        B, rows, h, dh = q.shape
        Lq = rows if Lq is None else Lq
        bm = bm or (128 if Lq >= 128 else 64)
        if out is not None:                                  # dense buffers of B*G*Lq rows
            o, lse = out
            out_dtype = o.dtype
        else:
            o = torch.empty(B, G, Lq, h, dh, dtype=out_dtype, device=q.device)
            lse = torch.empty(B, G, Lq, h, dtype=F32, device=q.device)
        self._ck(self.lib.dmb_attn_fwd_tc(
            q.data_ptr(), _tv(q), rows, Kc.data_ptr(), Vc.data_ptr(), _tv(Kc), Kc.shape[1], o.data_ptr(),
            int(out_dtype == BF16), lse.data_ptr(), B, G, Lq, h, dh, lo, hi, qbase, grow, scale, window,
            int(causal), causal_excl, bm, pair_shift, self._tc_err.data_ptr(), self._st()), "attn_fwd_tc")
        return o, lse

    def attn_dq_tc(self, q, do_c, Kc, Vc, lo, hi, qbase, scale, window, lse, corr, dq, G=1, grow=0, accumulate=True):
        """Query side of a tape read's backward on tcgen05: dq [B, G*64, h, dh] fp32 (dense) += dS K, with
        dS = exp(s - lse) (d o . v - corr) scale; group z reads tape rows max(0, lo + z*grow) <= j < hi + z*grow.
        lse, corr: dense [B, G*64, h] fp32."""
        B, rows, h, dh = q.shape
        self._ck(self.lib.dmb_attn_dq_tc(
            q.data_ptr(), _tv(q), do_c.data_ptr(), _tv(do_c), rows, Kc.data_ptr(), Vc.data_ptr(), _tv(Kc), Kc.shape[1],
            lse.data_ptr(), corr.data_ptr(), dq.data_ptr(), _tv(dq), B, G, h, dh, lo, hi, qbase, grow, scale, window,
            int(accumulate), self._tc_err.data_ptr(), self._st()), "attn_dq_tc")

    def attn_dkv_tc(self, q_all, doc_all, corr_all, lse_all, Kc, Vc, pos0, q_start, q_end, scale, window=0, G=1,
                    grow=0, span=1 << 30, out=None, accumulate=False):
        """Key side on tcgen05: (dK, dV) [B, G*64, h, dh] fp32 of the tape rows [pos0 + z*grow, +64) gathered
        over the query positions [max(q_start, chunk end), min(q_end, chunk start + span))."""
        B, T, h, dh = q_all.shape
        if out is None:
            out = (torch.empty(B, G * 64, h, dh, dtype=F32, device=q_all.device),
                   torch.empty(B, G * 64, h, dh, dtype=F32, device=q_all.device))
        self._ck(self.lib.dmb_attn_dkv_tc(
            q_all.data_ptr(), doc_all.data_ptr(), corr_all.data_ptr(), lse_all.data_ptr(), T, Kc.data_ptr(),
            Vc.data_ptr(), _tv(Kc), Kc.shape[1], out[0].data_ptr(), out[1].data_ptr(), _tv(out[0]), int(accumulate),
            B, G, h, dh, pos0, q_start, q_end, grow, span, scale, window, self._tc_err.data_ptr(), self._st()),
            "attn_dkv_tc")
        return out

    @staticmethod
    def _tc_ok(q, Kc, Vc):
        """Operands the tensor maps can describe: bf16, 16-byte aligned, rows of h*dh dense elements, strides in
        whole 16-byte units, K and V tapes laid out alike."""
        def ok(t):
            return (t.dtype == BF16 and t.dim() == 4 and t.data_ptr() % 16 == 0 and _dense_tail(t, 2)
                    and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0)
        return (ok(q) and ok(Kc) and ok(Vc) and q.shape[3] in (64, 128) and Kc.stride() == Vc.stride()
                and Kc.shape == Vc.shape)

    def tc_check(self):
        """Host read of the tcgen05 attention kernels' error flag (a pipeline wait that ran out)."""
        if self._tc_err.item() != 0:
            raise RuntimeError("tcgen05 attention: a pipeline wait ran out (kernel aborted its tile loop)")

    def prefix_dq(self, q_r, Kc, Vc, pos0, scale, window, lse_c, do_c, corr, dq_acc, qoff=0):
        from ..engines.fused_math import prefix_lo
        B, c, h, dh = q_r.shape
        lo = prefix_lo(pos0, window, qoff)
        if pos0 - lo <= 0:
            return
        ok = (self._cell_ok(q_r) and do_c.dtype == BF16 and dq_acc.dtype == F32 and _dense_tail(dq_acc, 2)
              and _dense_tail(q_r, 2) and _dense_tail(do_c, 2) and _dense_tail(Kc, 2))
        if not ok:
            self._fell_back("prefix_dq")
            return super().prefix_dq(q_r, Kc, Vc, pos0, scale, window, lse_c, do_c, corr, dq_acc, qoff)
        lse_c, corr = lse_c.contiguous(), corr.contiguous()
        if (self._tc("dq") and c == 64 and self._tc_ok(q_r, Kc, Vc)
                and self._tc_ok(do_c, Kc, Vc)):
            return self.attn_dq_tc(q_r, do_c, Kc, Vc, lo, pos0, pos0 + qoff, scale, window, lse_c, corr, dq_acc)
        self._ck(self.lib.dmb_prefix_dq(q_r.data_ptr(), _tv(q_r), do_c.data_ptr(), _tv(do_c), Kc.data_ptr(),
                                        Vc.data_ptr(), _tv(Kc), lse_c.data_ptr(), corr.data_ptr(),
                                        dq_acc.data_ptr(), _tv(dq_acc), B, c, h, dh, lo, pos0, scale, window, 1, 0, qoff,
                                        self._st()), "prefix_dq")

    def prefix_dkv(self, q_all, doc_all, corr_all, lsec_all, Kc, Vc, pos0, c, q_start, scale, window=0, q_end=None,
                   out=None, accumulate=False):
        B, T, h, dh = q_all.shape
        q_end = T if q_end is None else min(q_end, T)
        ok = (q_all.dtype == BF16 and doc_all.dtype == BF16 and dh in (64, 128) and c in (16, 32, 64)
              and q_all.is_contiguous() and doc_all.is_contiguous() and corr_all.is_contiguous()
              and lsec_all.is_contiguous() and _dense_tail(Kc, 2) and (out is None or self._dkv_view_ok(out)))
        if not ok:
            self._fell_back("prefix_dkv")
            return super().prefix_dkv(q_all, doc_all, corr_all, lsec_all, Kc, Vc, pos0, c, q_start, scale, window, q_end,
                                      out, accumulate)
        if out is not None:
            dK, dV = out
        else:
            dK = torch.empty(B, c, h, dh, dtype=F32, device=q_all.device)
            dV = torch.empty(B, c, h, dh, dtype=F32, device=q_all.device)
            accumulate = False
        if self._tc("dkv") and c == 64 and self._tc_ok(q_all, Kc, Vc):
            return self.attn_dkv_tc(q_all, doc_all, corr_all, lsec_all, Kc, Vc, pos0, q_start, q_end, scale, window,
                                    out=(dK, dV), accumulate=accumulate)
        self._ck(self.lib.dmb_prefix_dkv(q_all.data_ptr(), doc_all.data_ptr(), corr_all.data_ptr(),
                                         lsec_all.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), _tv(Kc),
                                         dK.data_ptr(), dV.data_ptr(), _tv(dK), int(accumulate), B, T, c, h, dh, pos0,
                                         q_start, q_end, scale, window, 1, 0, 1 << 30, self._st()), "prefix_dkv")
        return dK, dV

    def tail_fwd(self, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, scale, window=0):
        if not self._cell_ok(q_r) or not all(_dense_tail(t, 2) for t in (q_r, kself_r, v_raw, K_in, V_in)):
            self._fell_back("tail_fwd")
            return super().tail_fwd(q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, scale, window)
        B, c, h, dh = q_r.shape
        o = torch.empty(B, c, h, dh, dtype=BF16, device=q_r.device)
        lse = torch.empty(B, c, h, dtype=F32, device=q_r.device)
        ssq = torch.empty(B, c, h, dtype=F32, device=q_r.device)
        o_c, lse_c = o_c.contiguous(), lse_c.contiguous()
        self._ck(self.lib.dmb_tail_fwd(q_r.data_ptr(), _tv(q_r), kself_r.data_ptr(), _tv(kself_r),
                                       v_raw.data_ptr(), _tv(v_raw), K_in.data_ptr(), _tv(K_in),
                                       V_in.data_ptr(), _tv(V_in), o_c.data_ptr(), lse_c.data_ptr(),
                                       o.data_ptr(), lse.data_ptr(), ssq.data_ptr(), B, c, h, dh, scale, window,
                                       1, 0, self._st()), "tail_fwd")
        return o, lse, ssq

    def tail_bwd(self, dO, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, o, lse, scale, window,
                 dq_acc, dks_acc, dv_acc, doc_acc, dlsec_acc, init=0, dkv_out=None):
        ok = (self._cell_ok(q_r) and dO.dtype == F32 and dO.is_contiguous() and o.is_contiguous()
              and doc_acc.is_contiguous() and dlsec_acc.is_contiguous()
              and all(_dense_tail(t, 2) for t in (q_r, kself_r, v_raw, K_in, V_in, dks_acc, dv_acc, dq_acc))
              and (dkv_out is None or self._dkv_view_ok(dkv_out)))
        if not ok:
            self._fell_back("tail_bwd")
            return super().tail_bwd(dO, q_r, kself_r, v_raw, K_in, V_in, o_c, lse_c, o, lse, scale,
                                    window, dq_acc, dks_acc, dv_acc, doc_acc, dlsec_acc, init, dkv_out)
        B, c, h, dh = q_r.shape
        if dkv_out is not None:
            dK_in, dV_in = dkv_out
        else:
            dK_in = torch.empty(B, c, h, dh, dtype=F32, device=q_r.device)
            dV_in = torch.empty(B, c, h, dh, dtype=F32, device=q_r.device)
        o_c, lse_c, lse = o_c.contiguous(), lse_c.contiguous(), lse.contiguous()
        self._ck(self.lib.dmb_tail_bwd(
            dO.data_ptr(), q_r.data_ptr(), _tv(q_r), kself_r.data_ptr(), _tv(kself_r), v_raw.data_ptr(),
            _tv(v_raw), K_in.data_ptr(), _tv(K_in), V_in.data_ptr(), _tv(V_in), o_c.data_ptr(),
            lse_c.data_ptr(), o.data_ptr(), lse.data_ptr(), dq_acc.data_ptr(), _tv(dq_acc), dks_acc.data_ptr(),
            _tv(dks_acc), dv_acc.data_ptr(), _tv(dv_acc), doc_acc.data_ptr(), dlsec_acc.data_ptr(),
            dK_in.data_ptr(), dV_in.data_ptr(), _tv(dK_in), B, c, h, dh, scale, window, 1, 0, int(init), self._st()),
            "tail_bwd")
        return dK_in, dV_in

    def tail_bwd_sweep(self, dO, q_r, kself_r, K_in, V_in, lse_c, o, lse, scale, window, dq_acc, init, scal):
        B, c, h, dh = q_r.shape
        ok = (self._cell_ok(q_r) and dO.dtype == F32 and dO.is_contiguous() and o.is_contiguous()
              and scal.is_contiguous() and scal.dtype == F32 and scal.shape == (3, B, c, h)
              and all(_dense_tail(t, 2) for t in (q_r, kself_r, K_in, V_in, dq_acc)))
        if not ok:
            self._fell_back("tail_bwd_sweep")
            return super().tail_bwd_sweep(dO, q_r, kself_r, K_in, V_in, lse_c, o, lse, scale, window, dq_acc, init, scal)
        dK_in = torch.empty(B, c, h, dh, dtype=F32, device=q_r.device)
        dV_in = torch.empty(B, c, h, dh, dtype=F32, device=q_r.device)
        lse_c, lse = lse_c.contiguous(), lse.contiguous()
        # deferred mode (flag bit 2): the raw value, o_c and the dks / dv / d o_c accumulators are not touched
        self._ck(self.lib.dmb_tail_bwd(
            dO.data_ptr(), q_r.data_ptr(), _tv(q_r), kself_r.data_ptr(), _tv(kself_r), kself_r.data_ptr(),
            _tv(kself_r), K_in.data_ptr(), _tv(K_in), V_in.data_ptr(), _tv(V_in), None,
            lse_c.data_ptr(), o.data_ptr(), lse.data_ptr(), dq_acc.data_ptr(), _tv(dq_acc), None,
            _tv(dq_acc), None, _tv(dq_acc), None, scal.data_ptr(),
            dK_in.data_ptr(), dV_in.data_ptr(), _tv(dK_in), B, c, h, dh, scale, window, 1, 0, 4 | (1 if init else 0),
            self._st()), "tail_bwd_sweep")
        return dK_in, dV_in

    def cell_finish_sweeps(self, dOs, scal, q_r, kself_r, v_raw, o_c, lse_c, dK0, dV0, doc, corr, lsec, dks, dv, dq,
                           scale):
        B, R, h, dh = o_c.shape
        K = len(dOs)
        absf, absb = (dks, dv, dq), (q_r, kself_r, v_raw)
        ok = (dh in (64, 128) and o_c.is_cuda and 1 <= K <= 64 and doc.dtype in (BF16, F32) and _dense_tail(doc, 2)
              and doc.stride(1) == h * dh and scal.is_contiguous() and scal.shape == (K, 3, B, R, h)
              and all(t.is_contiguous() and t.dtype == F32 and t.shape == o_c.shape for t in tuple(dOs) + (o_c, dK0, dV0))
              and lse_c.is_contiguous() and lse_c.dtype == F32
              and all(self._abs_view_ok(t, 2) for t in absf)
              and all(t.dtype == BF16 and _dense_tail(t, 2) for t in absb)
              and all(self._abs_view_ok(t, 1) for t in (corr, lsec)) and corr.stride(0) == lsec.stride(0)
              and len({t.stride(0) for t in absf + (doc,)}) == 1)
        if not ok:
            self._fell_back("cell_finish_sweeps")
            return super().cell_finish_sweeps(dOs, scal, q_r, kself_r, v_raw, o_c, lse_c, dK0, dV0, doc, corr, lsec,
                                              dks, dv, dq, scale)
        cv = torch.empty(B, R, h, dtype=F32, device=o_c.device)
        ptrs = (ctypes.c_void_p * K)(*[t.data_ptr() for t in dOs])
        self._ck(self.lib.dmb_cell_finish_sweeps(
            ctypes.cast(ptrs, ctypes.c_void_p), K, scal.data_ptr(), q_r.data_ptr(), _tv(q_r), kself_r.data_ptr(),
            _tv(kself_r), v_raw.data_ptr(), _tv(v_raw), o_c.data_ptr(),
            lse_c.data_ptr(), dK0.data_ptr(), dV0.data_ptr(), doc.data_ptr(), int(doc.dtype == BF16), corr.data_ptr(),
            cv.data_ptr(), lsec.data_ptr(), dks.data_ptr(), dv.data_ptr(), dq.data_ptr(), scale, dks.stride(0),
            corr.stride(0), B, R, h, dh, self._st()), "cell_finish_sweeps")
        return cv

    @staticmethod
    def _dkv_view_ok(pair):
        a, b = pair
        return (a.dtype == F32 and b.dtype == F32 and _dense_tail(a, 2) and a.stride() == b.stride()
                and a.data_ptr() % 8 == 0 and b.data_ptr() % 8 == 0)

    def win_near_dkv(self, q_all, docn_all, corrn_all, lsen_all, Kc, Vc, j0, G, C, q_lo, q_hi, span, scale, window=0,
                     out=None, accumulate=False):
        B, T, h, dh = q_all.shape
        ok = (q_all.dtype == BF16 and docn_all.dtype == BF16 and dh in (64, 128) and C in (16, 32, 64)
              and q_all.is_contiguous() and docn_all.is_contiguous() and corrn_all.is_contiguous()
              and lsen_all.is_contiguous() and _dense_tail(Kc, 2) and (out is None or self._dkv_view_ok(out)))
        if not ok:
            self._fell_back("win_near_dkv")
            return super().win_near_dkv(q_all, docn_all, corrn_all, lsen_all, Kc, Vc, j0, G, C, q_lo, q_hi, span, scale,
                                        window, out, accumulate)
        if out is not None:
            dK, dV = out
        else:
            dK = torch.empty(B, G * C, h, dh, dtype=F32, device=q_all.device)
            dV = torch.empty(B, G * C, h, dh, dtype=F32, device=q_all.device)
            accumulate = False
        if self._tc("dkv") and C == 64 and self._tc_ok(q_all, Kc, Vc):
            return self.attn_dkv_tc(q_all, docn_all, corrn_all, lsen_all, Kc, Vc, j0 * C, q_lo, min(q_hi, T), scale,
                                    window, G=G, grow=C, span=span, out=(dK, dV), accumulate=accumulate)
        self._ck(self.lib.dmb_prefix_dkv(q_all.data_ptr(), docn_all.data_ptr(), corrn_all.data_ptr(),
                                         lsen_all.data_ptr(), Kc.data_ptr(), Vc.data_ptr(), _tv(Kc), dK.data_ptr(),
                                         dV.data_ptr(), _tv(dK), int(accumulate), B, T, C, h, dh, j0 * C, q_lo,
                                         min(q_hi, T), scale, window, G, C, span, self._st()), "win_near_dkv")
        return dK, dV

    @staticmethod
    def _abs_view_ok(t, n_tail):
        """A [B, R, ...] slice of a contiguous [B, T, ...] buffer: dense rows, only the batch stride differs."""
        return t.dtype == F32 and _dense_tail(t, n_tail) and t.stride(1) == (t.shape[2] * (t.shape[3] if t.dim() == 4 else 1))

    def cell_finish(self, do_c, dlse_c, o_c, lse_c, dK0, dV0, doc, corr, lsec, dks, dv):
        B, R, h, dh = do_c.shape
        ok = (dh in (64, 128) and do_c.is_cuda and doc.dtype in (BF16, F32) and _dense_tail(doc, 2)
              and all(t.is_contiguous() and t.dtype == F32 for t in (do_c, dlse_c, o_c, lse_c, dK0, dV0))
              and all(self._abs_view_ok(t, 2) for t in (dks, dv)) and all(self._abs_view_ok(t, 1) for t in (corr, lsec))
              and doc.stride(1) == h * dh and len({doc.stride(0), dks.stride(0), dv.stride(0)}) == 1
              and corr.stride(0) == lsec.stride(0))
        if not ok:
            self._fell_back("cell_finish")
            return super().cell_finish(do_c, dlse_c, o_c, lse_c, dK0, dV0, doc, corr, lsec, dks, dv)
        cv = torch.empty(B, R, h, dtype=F32, device=do_c.device)
        self._ck(self.lib.dmb_cell_finish(do_c.data_ptr(), dlse_c.data_ptr(), o_c.data_ptr(), lse_c.data_ptr(),
                                          dK0.data_ptr(), dV0.data_ptr(), doc.data_ptr(), int(doc.dtype == BF16),
                                          corr.data_ptr(), cv.data_ptr(), lsec.data_ptr(), dks.data_ptr(), dv.data_ptr(),
                                          doc.stride(0), corr.stride(0), B, R, h, dh, self._st()), "cell_finish")
        return cv

    def merge_partials(self, o_f, lse_f, o_n, lse_n):
        B, R, h, dh = o_n.shape
        ok = (dh in (64, 128) and self._abs_view_ok(o_f, 2) and self._abs_view_ok(lse_f, 1)
              and o_n.is_contiguous() and lse_n.is_contiguous() and o_n.dtype == F32 and o_n.is_cuda)
        if not ok:
            self._fell_back("merge_partials")
            return super().merge_partials(o_f, lse_f, o_n, lse_n)
        o_c, lse_c = torch.empty_like(o_n), torch.empty_like(lse_n)
        w_f, w_n = torch.empty_like(lse_n), torch.empty_like(lse_n)
        self._ck(self.lib.dmb_wave_merge_fwd(o_f.data_ptr(), lse_f.data_ptr(), o_f.stride(0), lse_f.stride(0),
                                             o_n.data_ptr(), lse_n.data_ptr(), o_c.data_ptr(), lse_c.data_ptr(),
                                             w_f.data_ptr(), w_n.data_ptr(), B, R, h, dh, self._st()), "merge_partials")
        return o_c, lse_c, w_f, w_n

    def split_partials(self, do_c, dlse_c, o_f, o_c, o_n, lse_n, w_f, w_n, DOf, DLf, docn, corrn, lsen, corrn_dense=None):
        B, R, h, dh = o_n.shape
        vec = (o_f, DOf)
        ok = (dh in (64, 128) and all(self._abs_view_ok(t, 2) for t in vec) and _dense_tail(docn, 2)
              and docn.dtype in (BF16, F32) and all(self._abs_view_ok(t, 1) for t in (DLf, corrn, lsen))
              and len({o_f.stride(0), DOf.stride(0), docn.stride(0)}) == 1
              and len({DLf.stride(0), corrn.stride(0), lsen.stride(0)}) == 1
              and all(t.is_contiguous() and t.dtype == F32 for t in (do_c, dlse_c, o_c, o_n, lse_n, w_f, w_n))
              and (corrn_dense is None or (corrn_dense.is_contiguous() and corrn_dense.dtype == F32
                                           and corrn_dense.shape == lse_n.shape)))
        if not ok:
            self._fell_back("split_partials")
            return super().split_partials(do_c, dlse_c, o_f, o_c, o_n, lse_n, w_f, w_n, DOf, DLf, docn, corrn, lsen,
                                          corrn_dense)
        self._ck(self.lib.dmb_wave_split_bwd(do_c.data_ptr(), dlse_c.data_ptr(), o_c.data_ptr(), o_n.data_ptr(),
                                             lse_n.data_ptr(), w_f.data_ptr(), w_n.data_ptr(), o_f.data_ptr(),
                                             DOf.data_ptr(), DLf.data_ptr(), docn.data_ptr(), int(docn.dtype == BF16),
                                             corrn.data_ptr(), corrn_dense.data_ptr() if corrn_dense is not None else None,
                                             lsen.data_ptr(), o_f.stride(0), DLf.stride(0), B, R, h, dh,
                                             self._st()), "split_partials")

    def chunk_finish(self, DOf, DLf, o_f, lse_f, dKp, dVp, dks, dv, doc, corr, lsec, sweeps=None, q=None, dglx=None):
        B, R, h, dh = DOf.shape
        vec, sca = (DOf, o_f, dKp, dVp, dks, dv), (DLf, lse_f, corr, lsec)
        sweeps = sweeps or []
        ok = (dh in (64, 128) and DOf.is_cuda and doc.dtype in (BF16, F32) and _dense_tail(doc, 2)
              and doc.stride(1) == h * dh
              and all(self._abs_view_ok(t, 2) and t.dtype == F32 for t in vec)
              and all(self._abs_view_ok(t, 1) and t.dtype == F32 for t in sca)
              and len({t.stride(0) for t in vec + (doc,)}) == 1 and len({t.stride(0) for t in sca}) == 1
              and len(sweeps) <= 64
              and all(self._abs_view_ok(t[0], 2) and t[0].shape == DOf.shape and self._abs_view_ok(t[1], 1)
                      and self._abs_view_ok(t[2], 1) and t[1].shape == DLf.shape and t[1].stride(0) == t[2].stride(0)
                      for t in sweeps)
              and (not sweeps or (q is not None and q.dtype == BF16 and _dense_tail(q, 2) and q.shape == DOf.shape))
              and (dglx is None or (bool(sweeps) and dglx.dtype == F32 and dglx.shape == (B, R, 2 * h * dh)
                                    and _dense_tail(dglx, 2)
                                    and all(len(t) == 4 and t[3].dtype == BF16 and t[3].shape == (B, R, 4 * h * dh)
                                            and _dense_tail(t[3], 2) and t[3].stride(0) == 4 * t[0].stride(0)
                                            for t in sweeps))))
        if not ok:
            self._fell_back("chunk_finish")
            return super().chunk_finish(DOf, DLf, o_f, lse_f, dKp, dVp, dks, dv, doc, corr, lsec, sweeps, q, dglx)
        cv = torch.empty(B, R, h, dtype=F32, device=DOf.device)
        ls = torch.empty(B, R, h, dtype=F32, device=DOf.device)
        K = len(sweeps)
        arr = lambda ty, vals: ctypes.cast((ty * max(K, 1))(*vals), ctypes.c_void_p)
        self._ck(self.lib.dmb_wave_chunk_finish(
            DOf.data_ptr(), DLf.data_ptr(), o_f.data_ptr(), lse_f.data_ptr(), dKp.data_ptr(), dVp.data_ptr(),
            dks.data_ptr(), dv.data_ptr(), doc.data_ptr(), int(doc.dtype == BF16), corr.data_ptr(), lsec.data_ptr(),
            cv.data_ptr(), ls.data_ptr(), DOf.stride(0), DLf.stride(0), B, R, h, dh, K,
            arr(ctypes.c_void_p, [t[0].data_ptr() for t in sweeps]),
            arr(ctypes.c_void_p, [t[1].data_ptr() for t in sweeps]),
            arr(ctypes.c_void_p, [t[2].data_ptr() for t in sweeps]),
            arr(ctypes.c_longlong, [t[0].stride(0) for t in sweeps]),
            arr(ctypes.c_longlong, [t[1].stride(0) for t in sweeps]),
            q.data_ptr() if K else None, _tv(q) if K else TView(0, 0),
            arr(ctypes.c_void_p, [t[3].data_ptr() for t in sweeps]) if dglx is not None else None,
            dglx.data_ptr() if dglx is not None else None, dglx.stride(0) if dglx is not None else 0,
            self._st()), "chunk_finish")
        return cv, ls

    def copy_pair(self, d0, s0, d1, s1):
        """d0 <- s0 and d1 <- s1 in one launch: same shape and dtype, every batch row one contiguous block."""
        B = d0.shape[0]
        row = d0[0].numel() * d0.element_size()
        blk = lambda t: t.dim() >= 2 and t[0].is_contiguous() and t.data_ptr() % 16 == 0
        ok = (d0.is_cuda and all(blk(t) for t in (d0, s0, d1, s1)) and row % 16 == 0
              and d0.shape == s0.shape == d1.shape == s1.shape and d0.dtype == s0.dtype == d1.dtype == s1.dtype
              and s0.stride(0) == s1.stride(0) and d0.stride(0) == d1.stride(0)
              and (s0.stride(0) * s0.element_size()) % 16 == 0 and (d0.stride(0) * d0.element_size()) % 16 == 0)
        if not ok:
            self._fell_back("copy_pair")
            return super().copy_pair(d0, s0, d1, s1)
        es = d0.element_size()
        self._ck(self.lib.dmb_copy_pair(s0.data_ptr(), d0.data_ptr(), s1.data_ptr(), d1.data_ptr(), s0.stride(0) * es,
                                        d0.stride(0) * es, row, B, self._st()), "copy_pair")

    # ---- window ops: G consecutive chunks of the same sequences in one launch ----------------------------
    def _win_ok(self, q_win, C, *views):
        B, rows, h, dh = q_win.shape
        return (q_win.dtype == BF16 and dh in (64, 128) and C in (16, 32, 64) and rows % C == 0
                and all(_dense_tail(t, 2) for t in (q_win,) + views))

    def win_near_fwd(self, q_win, Kc, Vc, pos0, lo, C, scale, window=0):
        if not self._win_ok(q_win, C, Kc):
            self._fell_back("win_near_fwd")
            return super().win_near_fwd(q_win, Kc, Vc, pos0, lo, C, scale, window)
        B, rows, h, dh = q_win.shape
        o_n = torch.empty(B, rows, h, dh, dtype=F32, device=q_win.device)
        lse_n = torch.empty(B, rows, h, dtype=F32, device=q_win.device)
        if self._tc("fwd") and C == 64 and self._tc_ok(q_win, Kc, Vc):
            G = rows // C
            if dh == 64 and G % 2 == 0 and self.NEAR_PAIRS:
                # two window chunks per 128-row tile: their key ranges overlap in all but one chunk each
                self.attn_fwd_tc(q_win, Kc, Vc, lo, pos0, pos0, scale, window, Lq=128, G=G // 2, grow=128, bm=128,
                                 out=(o_n, lse_n), pair_shift=64)
            else:
                self.attn_fwd_tc(q_win, Kc, Vc, lo, pos0, pos0, scale, window, Lq=C, G=G, grow=C, bm=64,
                                 out=(o_n, lse_n))
            return o_n, lse_n
        self._ck(self.lib.dmb_prefix_fwd(q_win.data_ptr(), _tv(q_win), Kc.data_ptr(), Vc.data_ptr(), _tv(Kc),
                                         o_n.data_ptr(), lse_n.data_ptr(), B, C, h, dh, lo, pos0, scale, window,
                                         rows // C, C, 0, self._st()), "win_near_fwd")
        return o_n, lse_n

    def win_near_merged(self, q_win, Kc, Vc, pos0, lo, C, scale, window, o_f, lse_f, keep_near=True):
        """The near read of a window merged with the chunks' far partials in the read kernel's epilogue."""
        B, rows, h, dh = q_win.shape
        G = rows // C
        ok = (self._tc("fwd") and C == 64 and self._win_ok(q_win, C, Kc) and self._tc_ok(q_win, Kc, Vc)
              and self._abs_view_ok(o_f, 2) and self._abs_view_ok(lse_f, 1) and o_f.shape == (B, rows, h, dh))
        if not ok:
            self._fell_back("win_near_merged")
            return super().win_near_merged(q_win, Kc, Vc, pos0, lo, C, scale, window, o_f, lse_f, keep_near)
        dev = q_win.device
        o_c = torch.empty(B, rows, h, dh, dtype=F32, device=dev)
        lse_c, w_f, w_n = (torch.empty(B, rows, h, dtype=F32, device=dev) for _ in range(3))
        o_n = torch.empty(B, rows, h, dh, dtype=F32, device=dev) if keep_near else None
        lse_n = torch.empty(B, rows, h, dtype=F32, device=dev) if keep_near else None
        pair = dh == 64 and G % 2 == 0 and self.NEAR_PAIRS
        Lq, Gz, grow, bm, shift = (128, G // 2, 128, 128, 64) if pair else (C, G, C, 64, 0)
        self._ck(self.lib.dmb_attn_fwd_tc_merged(
            q_win.data_ptr(), _tv(q_win), rows, Kc.data_ptr(), Vc.data_ptr(), _tv(Kc), Kc.shape[1], o_c.data_ptr(), 0,
            lse_c.data_ptr(), B, Gz, Lq, h, dh, lo, pos0, pos0, grow, scale, window, 0, 1, bm, shift,
            o_f.data_ptr(), lse_f.data_ptr(), o_f.stride(0), lse_f.stride(0), w_f.data_ptr(), w_n.data_ptr(),
            o_n.data_ptr() if keep_near else None, lse_n.data_ptr() if keep_near else None,
            self._tc_err.data_ptr(), self._st()), "win_near_merged")
        return o_c, lse_c, w_f, w_n, o_n, lse_n

    def win_near_dq(self, q_win, Kc, Vc, pos0, lo, C, scale, lse_n, do_n, corr_n, dq_acc, window=0):
        ok = (self._win_ok(q_win, C, Kc, do_n) and do_n.dtype == BF16 and dq_acc.dtype == F32 and _dense_tail(dq_acc, 2)
              and lse_n.is_contiguous() and corr_n.is_contiguous())
        if not ok:
            self._fell_back("win_near_dq")
            return super().win_near_dq(q_win, Kc, Vc, pos0, lo, C, scale, lse_n, do_n, corr_n, dq_acc, window)
        B, rows, h, dh = q_win.shape
        if (self._tc("dq") and C == 64 and self._tc_ok(q_win, Kc, Vc)
                and self._tc_ok(do_n, Kc, Vc)):
            return self.attn_dq_tc(q_win, do_n, Kc, Vc, lo, pos0, pos0, scale, window, lse_n, corr_n, dq_acc,
                                   G=rows // C, grow=C)
        self._ck(self.lib.dmb_prefix_dq(q_win.data_ptr(), _tv(q_win), do_n.data_ptr(), _tv(do_n), Kc.data_ptr(),
                                        Vc.data_ptr(), _tv(Kc), lse_n.data_ptr(), corr_n.data_ptr(),
                                        dq_acc.data_ptr(), _tv(dq_acc), B, C, h, dh, lo, pos0, scale, window, rows // C,
                                        C, 0, self._st()), "win_near_dq")

    def win_tail_fwd(self, q_win, ks_win, vr_win, K_in, V_in, o_c, lse_c, C, scale, window=0):
        if not self._win_ok(q_win, C, ks_win, vr_win, K_in, V_in) or not (o_c.is_contiguous() and lse_c.is_contiguous()):
            self._fell_back("win_tail_fwd")
            return super().win_tail_fwd(q_win, ks_win, vr_win, K_in, V_in, o_c, lse_c, C, scale, window)
        B, rows, h, dh = q_win.shape
        o = torch.empty(B, rows, h, dh, dtype=BF16, device=q_win.device)
        lse = torch.empty(B, rows, h, dtype=F32, device=q_win.device)
        ssq = torch.empty(B, rows, h, dtype=F32, device=q_win.device)
        self._ck(self.lib.dmb_tail_fwd(q_win.data_ptr(), _tv(q_win), ks_win.data_ptr(), _tv(ks_win),
                                       vr_win.data_ptr(), _tv(vr_win), K_in.data_ptr(), _tv(K_in),
                                       V_in.data_ptr(), _tv(V_in), o_c.data_ptr(), lse_c.data_ptr(),
                                       o.data_ptr(), lse.data_ptr(), ssq.data_ptr(), B, C, h, dh, scale, window,
                                       rows // C, C, self._st()), "win_tail_fwd")
        return o, lse, ssq

    def win_tail_bwd(self, dO, q_win, ks_win, vr_win, K_in, V_in, o_c, lse_c, o, lse, C, scale,
                     dq_acc, dks_acc, dv_acc, doc_acc, dlsec_acc, window=0, init=0, dkv_out=None, raw_stash=None):
        B, rows, h, dh = q_win.shape
        raw_views = () if raw_stash is not None else (dks_acc, dv_acc)
        ok = (self._win_ok(q_win, C, ks_win, vr_win, K_in, V_in, *raw_views) and dO.dtype == F32
              and all(t.is_contiguous() for t in (dO, o, o_c, lse_c, lse, doc_acc, dlsec_acc))
              and _dense_tail(dq_acc, 2) and (dkv_out is None or self._dkv_view_ok(dkv_out))
              and (raw_stash is None or (raw_stash.is_contiguous() and raw_stash.dtype == F32
                                         and raw_stash.shape == (2, B, rows, h))))
        if not ok:
            self._fell_back("win_tail_bwd")
            return super().win_tail_bwd(dO, q_win, ks_win, vr_win, K_in, V_in, o_c, lse_c, o, lse, C, scale,
                                        dq_acc, dks_acc, dv_acc, doc_acc, dlsec_acc, window, init, dkv_out, raw_stash)
        if dkv_out is not None:
            dK_in, dV_in = dkv_out
        else:
            dK_in = torch.empty(B, rows, h, dh, dtype=F32, device=q_win.device)
            dV_in = torch.empty(B, rows, h, dh, dtype=F32, device=q_win.device)
        self._ck(self.lib.dmb_tail_bwd(
            dO.data_ptr(), q_win.data_ptr(), _tv(q_win), ks_win.data_ptr(), _tv(ks_win), vr_win.data_ptr(),
            _tv(vr_win), K_in.data_ptr(), _tv(K_in), V_in.data_ptr(), _tv(V_in), o_c.data_ptr(),
            lse_c.data_ptr(), o.data_ptr(), lse.data_ptr(), dq_acc.data_ptr(), _tv(dq_acc),
            # raw-row gradients deferred (flag bit 3): the stash [2, B, rows, h] rides in the d k_self slot
            *((raw_stash.data_ptr(), TView(0, 0), None, TView(0, 0)) if raw_stash is not None else
              (dks_acc.data_ptr(), _tv(dks_acc), dv_acc.data_ptr(), _tv(dv_acc))),
            doc_acc.data_ptr(), dlsec_acc.data_ptr(),
            dK_in.data_ptr(), dV_in.data_ptr(), _tv(dK_in), B, C, h, dh, scale, window, rows // C, C,
            int(init) | (8 if raw_stash is not None else 0), self._st()), "win_tail_bwd")
        return dK_in, dV_in

    def refine_fwd(self, raw, ssq, glx, k, v, cos, sin, h, pin_cols=0, out=None):
        B, c, d = k.shape
        dh = d // h
        ok = (k.dtype == BF16 and raw.dtype == BF16 and raw.is_contiguous() and cos.is_contiguous() and cos.dtype == F32 and sin.dtype == F32
              and ssq.is_contiguous() and dh % 16 == 0
              and all(_dense_tail(t, 1) for t in (glx, k, v)))
        if not ok:
            self._fell_back("refine_fwd")
            return super().refine_fwd(raw, ssq, glx, k, v, cos, sin, h, pin_cols, out)
        if (out is not None and all(t.dtype == BF16 and _dense_tail(t, 2) for t in out)
                and out[0].stride() == out[1].stride()):
            K_out, V_out = out                                # e.g. the cell's rows of the tape itself
        else:
            K_out = torch.empty(B, c, h, dh, dtype=BF16, device=k.device)
            V_out = torch.empty(B, c, h, dh, dtype=BF16, device=k.device)
        self._ck(self.lib.dmb_refine_fwd(raw.data_ptr(), ssq.data_ptr(), glx.data_ptr(), _tv(glx), k.data_ptr(),
                                         _tv(k), v.data_ptr(), _tv(v), cos.data_ptr(), sin.data_ptr(),
                                         K_out.data_ptr(), V_out.data_ptr(), _tv(K_out), B, c, h, dh, pin_cols, 1e-5,
                                         self._st()), "refine_fwd")
        if out is not None and K_out is not out[0]:
            out[0].copy_(K_out)
            out[1].copy_(V_out)
            return out
        return K_out, V_out

    def refine_bwd(self, dK_out, dV_out, raw, ssq, o, glx, k, v, cos, sin, pin_cols, dk_acc, dv_acc, dglx_acc,
                   dcg_out, uhat_out):
        B, c, d = k.shape
        h = dK_out.shape[2]
        dh = d // h
        ok = (k.dtype == BF16 and raw.dtype == BF16 and o.dtype == BF16 and dK_out.dtype == F32
              and dV_out.dtype == F32 and _dense_tail(dK_out, 2) and dK_out.stride() == dV_out.stride()
              and raw.is_contiguous() and o.is_contiguous() and ssq.is_contiguous() and cos.is_contiguous() and cos.dtype == F32 and sin.dtype == F32
              and dcg_out.is_contiguous() and uhat_out.is_contiguous() and dcg_out.dtype == BF16
              and dh % 16 == 0
              and all(_dense_tail(t, 1) for t in (glx, k, v, dk_acc, dv_acc))
              and (dglx_acc is None or _dense_tail(dglx_acc, 1)))
        if not ok:
            self._fell_back("refine_bwd")
            return super().refine_bwd(dK_out, dV_out, raw, ssq, o, glx, k, v, cos, sin, pin_cols, dk_acc, dv_acc,
                                      dglx_acc, dcg_out, uhat_out)
        dg_ptr, dg_view = (dglx_acc.data_ptr(), _tv(dglx_acc)) if dglx_acc is not None else (None, TView(0, 0))
        self._ck(self.lib.dmb_refine_bwd(
            dK_out.data_ptr(), dV_out.data_ptr(), _tv(dK_out), raw.data_ptr(), ssq.data_ptr(), o.data_ptr(), glx.data_ptr(),
            _tv(glx), k.data_ptr(), _tv(k), v.data_ptr(), _tv(v), cos.data_ptr(), sin.data_ptr(),
            dcg_out.data_ptr(), uhat_out.data_ptr(), dk_acc.data_ptr(), _tv(dk_acc), dv_acc.data_ptr(),
            _tv(dv_acc), dg_ptr, dg_view, B, c, h, dh, pin_cols, 1e-5, self._st()),
            "refine_bwd")

    def stash_gate_sum(self, dcg_stash, B, T, c, K):
        d = dcg_stash.shape[1] // 4
        if not (dcg_stash.dtype == BF16 and dcg_stash.is_contiguous() and d % 8 == 0 and T % c == 0
                and dcg_stash.shape[0] == (T // c) * K * B * c):
            self._fell_back("stash_gate_sum")
            return super().stash_gate_sum(dcg_stash, B, T, c, K)
        out = torch.empty(B, T, 2 * d, dtype=BF16, device=dcg_stash.device)
        self._ck(self.lib.dmb_stash_gate_sum(dcg_stash.data_ptr(), out.data_ptr(), B, T, c, K, d, self._st()),
                 "stash_gate_sum")
        return out

    def rmsn_bwd(self, du, o, ssq, residual=None, out_dtype=F32, extra=None):
        d = o.shape[-1]
        h = ssq.shape[-1]
        ok = (du.dtype == BF16 and o.dtype == BF16 and du.is_contiguous() and o.is_contiguous()
              and ssq.is_contiguous() and d % 8 == 0 and out_dtype in (BF16, F32)
              and (residual is None or (residual.is_contiguous() and residual.dtype == out_dtype))
              and (extra is None or (extra.is_contiguous() and extra.dtype == F32)))
        if not ok:
            self._fell_back("rmsn_bwd")
            return super().rmsn_bwd(du, o, ssq, residual, out_dtype, extra)
        rows = o.numel() // d
        out = torch.empty(o.shape, dtype=out_dtype, device=o.device)
        self._ck(self.lib.dmb_rmsn_bwd(du.data_ptr(), o.data_ptr(), ssq.data_ptr(),
                                       residual.data_ptr() if residual is not None else None,
                                       extra.data_ptr() if extra is not None else None, out.data_ptr(),
                                       int(out_dtype == F32), rows, d, h, 1e-5, self._st()), "rmsn_bwd")
        return out
