"""Python face of the tcgen05 GEMM (csrc/gemm_tcgen05.cu): the three products a linear layer
needs, each in the operand layout it naturally has, so no transposes are materialised.

  linear        y  = x W^T        A = x  [M,K] K-major,  B = W  [N,K] K-major
  linear_dx     dx = dy W         A = dy [M,N] K-major,  B = W  [N,K] read as [K'][N'] N-major
  linear_dw_acc dW += dy^T x      A = dy [rows,N] M-major, B = x [rows,K] N-major, fp32 accumulate
"""

from __future__ import annotations

import ctypes
import os

import torch

BF16, F32 = torch.bfloat16, torch.float32


def _rows(t):
    """2-D row view (rows, cols, row stride) of a tensor whose last dim is dense and whose leading
    dims collapse to one stride; None otherwise."""
    if t.stride(-1) != 1:
        return None
    if t.dim() == 1:
        return None
    if t.dim() == 2:
        return t.shape[0], t.shape[1], t.stride(0)
    if t.is_contiguous():
        return t.numel() // t.shape[-1], t.shape[-1], t.shape[-1]
    return None


def _aligned(t, ld):
    return t.data_ptr() % 16 == 0 and ld % 8 == 0


def gemm_kernel_for(M, N, K, out_f32, acc, pair, ksplit, sms):
    """Name of the library entry point a problem goes to.  `pair`: False, True (every problem with enough rows and
    columns on CTA pairs) or "narrow" (only bf16 results with too few 256-wide tiles for the SMs, on 256 x 128 pair
    tiles); `ksplit`: bf16 results with at most sms / 2 tiles of 128 x 256 and K >= 2048 split K across the two CTAs of
    a cluster (the input gradient of a sweep: 2048 x 1024 over K = 4096)."""
    tiles = -(-M // 128) * -(-N // 256)
    if pair == "narrow":
        use_pair = not out_f32 and M >= 256 and N >= 128 and K >= 512 and tiles <= sms // 2
    else:
        use_pair = bool(pair) and M >= 512 and N >= 192
    if use_pair:
        return "dmb_gemm_bf16_pair"
    if ksplit and not out_f32 and not acc and K >= 2048 and 2 * tiles <= sms:
        return "dmb_gemm_bf16_ksplit2"
    return "dmb_gemm_bf16"


class Tcgen05Gemm:
    MIN_WORK = 1 << 18          # below this many MACs the launch is not worth a tensor-map encode

    def __init__(self, lib, device):
        self.lib, self.device = lib, torch.device(device)
        p, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.dmb_gemm_bf16.restype = i
        lib.dmb_gemm_bf16.argtypes = [p, p, p, p, i, i, i, ll, ll, ll, i, i, i, i, p, p]
        lib.dmb_gemm_bf16_pair.restype = i
        lib.dmb_gemm_bf16_pair.argtypes = lib.dmb_gemm_bf16.argtypes
        lib.dmb_gemm_pair_bn.argtypes = [i]
        lib.dmb_gemm_bf16_ksplit2.restype = i
        lib.dmb_gemm_bf16_ksplit2.argtypes = lib.dmb_gemm_bf16.argtypes
        # bf16 results with at most SMs / 2 tiles and a long reduction (the input gradient of a sweep): two CTAs of a
        # cluster split the K range of each tile and add their accumulators through shared memory
        self.ksplit = os.environ.get("DMB_GEMM_KSPLIT", "1") != "0"
        # CTA pairs (tcgen05 cta_group::2): DMB_GEMM_PAIR = "1" / True for every problem with enough rows and columns
        # (256 x 256 tiles, or 256 x 128 where those leave SMs idle), "narrow" only for bf16 results with too few
        # 256-wide tiles to fill the SMs (256 x 128 pair tiles instead of 128 x 128 tiles per CTA), "0" never
        mode = os.environ.get("DMB_GEMM_PAIR", "0")
        self.pair = True if mode == "1" else ("narrow" if mode == "narrow" else False)
        self.sms = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        # probe: fails here (not mid-step) if the driver entry point for tensor maps is missing
        a = torch.zeros(128, 64, dtype=BF16, device=self.device)
        w = torch.zeros(256, 64, dtype=BF16, device=self.device)
        self._call(a, w, torch.empty(128, 256, dtype=BF16, device=self.device), None, 128, 256, 64, 64, 64, 256, 0, 0, 0, 0)
        self.check()

    def pair_width(self, bn):
        """Forces the CTA-pair kernel's tile width (128 or 256); 0 gives the choice back to its cost model."""
        self.lib.dmb_gemm_pair_bn(int(bn))

    def check(self):
        if self.err.item() != 0:
            raise RuntimeError("tcgen05 GEMM: a pipeline wait ran out (kernel aborted its tile loop)")

    def _call(self, A, B, C, bias, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_f32, acc):
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        fn = getattr(self.lib, gemm_kernel_for(M, N, K, out_f32, acc, self.pair, self.ksplit, self.sms))
        rc = fn(A.data_ptr(), B.data_ptr(), C.data_ptr(),
                                    bias.data_ptr() if bias is not None else None, M, N, K, lda, ldb, ldc,
                                    a_mn, b_mn, out_f32, acc, self.err.data_ptr(), st)
        if rc != 0:
            raise RuntimeError(f"tcgen05 GEMM launch failed ({rc})")

    # ---- y = x W^T ------------------------------------------------------------------------------
    def ok_tn(self, x, w):
        if x.dtype != BF16 or w.dtype != BF16 or w.dim() != 2 or not w.is_contiguous():
            return False
        r = _rows(x)
        if r is None:
            return False
        M, K, lda = r
        N = w.shape[0]
        return (K == w.shape[1] and N % 8 == 0 and K % 8 == 0 and _aligned(x, lda) and _aligned(w, K)
                and M * N * K >= self.MIN_WORK)

    def ok_out(self, out, x, N):
        """`out`: a 2-D [rows, N] view with a dense last dim (bf16 or fp32), e.g. a column block of a wider
        matrix; its row stride becomes the kernel's ldc."""
        r = _rows(x)
        return (out.dim() == 2 and out.stride(1) == 1 and out.dtype in (BF16, F32) and r is not None
                and out.shape == (r[0], N) and out.data_ptr() % 16 == 0
                and out.stride(0) % (8 if out.dtype == BF16 else 4) == 0)

    def linear(self, x, w, out_dtype=BF16, bias=None, out=None):
        M, K, lda = _rows(x)
        N = w.shape[0]
        if out is not None:
            self._call(x, w, out, bias, M, N, K, lda, K, out.stride(0), 0, 0, int(out.dtype == F32), 0)
            return out
        y = torch.empty(*x.shape[:-1], N, dtype=out_dtype, device=x.device)
        self._call(x, w, y, bias, M, N, K, lda, K, N, 0, 0, int(out_dtype == F32), 0)
        return y

    # ---- dx = dy W --------------------------------------------------------------------------------
    def ok_nn(self, dy, w):
        if dy.dtype != BF16 or w.dtype != BF16 or w.dim() != 2 or not w.is_contiguous():
            return False
        r = _rows(dy)
        if r is None:
            return False
        M, Kd, lda = r
        return (Kd == w.shape[0] and w.shape[1] % 8 == 0 and Kd % 8 == 0 and _aligned(dy, lda)
                and _aligned(w, w.shape[1]) and M * Kd * w.shape[1] >= self.MIN_WORK)

    def linear_dx(self, dy, w, out=None):
        M, Kd, lda = _rows(dy)
        N = w.shape[1]
        if out is not None:
            self._call(dy, w, out, None, M, N, Kd, lda, N, out.stride(0), 0, 1, int(out.dtype == F32), 0)
            return out
        dx = torch.empty(*dy.shape[:-1], N, dtype=BF16, device=dy.device)
        self._call(dy, w, dx, None, M, N, Kd, lda, N, N, 0, 1, 0, 0)
        return dx

    # ---- dW += dy^T x --------------------------------------------------------------------------------
    def ok_tn_dw(self, dW, dy, x):
        if dW.dtype != F32 or dy.dtype != BF16 or x.dtype != BF16 or dW.dim() != 2 or dW.stride(1) != 1:
            return False
        rd, rx = _rows(dy), _rows(x)
        if rd is None or rx is None or rd[0] != rx[0]:
            return False
        rows, M, lda = rd
        _, N, ldb = rx
        return (dW.shape == (M, N) and M % 8 == 0 and N % 8 == 0 and _aligned(dy, lda) and _aligned(x, ldb)
                and dW.data_ptr() % 16 == 0 and dW.stride(0) % 4 == 0 and rows * M * N >= self.MIN_WORK)

    def linear_dw_acc(self, dW, dy, x):
        rows, M, lda = _rows(dy)
        _, N, ldb = _rows(x)
        self._call(dy, x, dW, None, M, N, rows, lda, ldb, dW.stride(0), 1, 1, 1, 1)
