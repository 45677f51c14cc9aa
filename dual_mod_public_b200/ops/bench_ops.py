"""Micro-benchmarks of the sm_100a kernels at the shapes the 340M engine launches them with.

  python -m dual_mod_public_b200.ops.bench_ops                 # every op
  python -m dual_mod_public_b200.ops.bench_ops --only tail_bwd --iters 3 --no-flush   # for a profiler
  python -m dual_mod_public_b200.ops.bench_ops --only tail_fwd,refine_bwd             # several ops (substrings)

Each op is timed with CUDA events on the launching stream after warm-up; between timed
iterations a 512 MB buffer is written twice, so inputs come from HBM, not from the 126 MB L2, and the
GPU is still busy while the host prepares the launch (the interval then holds the kernel, not the
host's launch latency).
Printed per op: microseconds, and the achieved TFLOP/s or GB/s from the op's algorithmic
FLOPs / bytes (with the fraction of the measured peaks when MEASURED_PEAKS.json is found).
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from ..models.rope import build_rope_cache
from .cuda_ops import CudaOps

DEV = "cuda:0"
BF = torch.bfloat16


def peaks():
    here = os.path.dirname(os.path.abspath(__file__))
    p = os.path.join(here, "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "of measured"
    return 6650.0, 1590.0, "of fallback"


class Timer:
    def __init__(self, iters, flush):
        self.iters, self.flush = iters, flush
        self.junk = torch.empty(512 << 20, dtype=torch.uint8, device=DEV) if flush else None

    def __call__(self, fn, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(self.iters):
            if self.junk is not None:
                self.junk.fill_(1)
                self.junk.fill_(2)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / self.iters * 1e3          # microseconds


def rnd(*s, dtype=BF, scale=1.0):
    return (torch.randn(*s, device=DEV) * scale).to(dtype)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--B", type=int, default=32)
    ap.add_argument("--pos0", type=int, default=1024)
    ap.add_argument("--d", type=int, default=1024)
    ap.add_argument("--dh", type=int, default=64)
    args = ap.parse_args()
    ops = CudaOps(torch.device(DEV))
    T = Timer(args.iters, not args.no_flush)
    hbm, tf, tag = peaks()
    B, c, d, dh = args.B, 64, args.d, args.dh
    h = d // dh
    pos0, Tlen = args.pos0, args.pos0 + 64
    scale = dh ** -0.5
    rows = []

    def report(name, us, flops=0.0, bytes_=0.0):
        msg = f"{name:28s} {us:9.1f} us"
        if flops:
            t = flops / us / 1e6
            msg += f"  {t:8.1f} TFLOP/s ({t / tf:5.1%} {tag})"
        if bytes_:
            g = bytes_ / us / 1e3
            msg += f"  {g:8.1f} GB/s ({g / hbm:5.1%} {tag})"
        print(msg, flush=True)
        rows.append((name, us))

    want = lambda n: not args.only or any(o and o in n for o in args.only.split(","))
    # ---- cell tensors
    q, ks, vr = rnd(B, Tlen, h, dh), rnd(B, Tlen, h, dh), rnd(B, Tlen, h, dh)
    Kc, Vc = rnd(B, Tlen, h, dh), rnd(B, Tlen, h, dh)
    r = slice(pos0, pos0 + c)
    qc, ksc, vrc = q[:, r], ks[:, r], vr[:, r]
    K_in, V_in = rnd(B, c, h, dh), rnd(B, c, h, dh)
    o_c, lse_c = ops.prefix_fwd(qc, Kc, Vc, pos0, scale, 0)
    o, lse, ssq = ops.tail_fwd(qc, ksc, vrc, K_in, V_in, o_c, lse_c, scale, 0)
    z = lambda *s: torch.zeros(*s, device=DEV)
    att_f = 4.0 * B * h * c * dh          # flops per key for QK^T + PV

    def both(name, fn, flops):
        """The op through the tcgen05 kernel and through the warp-MMA kernel it replaces."""
        for tag_, flag in (("tcgen05", True), ("mma.sync", False)):
            ops.ATTN_TC = flag
            report(f"{name} [{tag_}]", T(fn), flops=flops)
        ops.ATTN_TC = type(ops).ATTN_TC
        ops.tc_check()

    if want("prefix_fwd"):
        both("prefix_fwd", lambda: ops.prefix_fwd(qc, Kc, Vc, pos0, scale, 0), att_f * pos0)
    if want("tail_fwd"):
        report("tail_fwd", T(lambda: ops.tail_fwd(qc, ksc, vrc, K_in, V_in, o_c, lse_c, scale, 0)), flops=att_f * c / 2)
    dO = rnd(B, c, h, dh, dtype=torch.float32)
    acc = [z(B, c, h, dh), z(B, Tlen, h, dh), z(B, Tlen, h, dh), z(B, c, h, dh), z(B, c, h)]
    if want("tail_bwd"):
        report("tail_bwd", T(lambda: ops.tail_bwd(dO, qc, ksc, vrc, K_in, V_in, o_c, lse_c, o, lse, scale, 0,
                                                  acc[0], acc[1][:, r], acc[2][:, r], acc[3], acc[4])),
               flops=2.5 * att_f * c / 2)
        # the same sweep with the row-scalar x row sums deferred to the end of the cell (4 sweeps per cell)
        scal = torch.empty(4, 3, B, c, h, device=DEV)
        report("tail_bwd_sweep (deferred)", T(lambda: ops.tail_bwd_sweep(dO, qc, ksc, K_in, V_in, lse_c, o, lse, scale, 0,
                                                                       acc[0], False, scal[0])),
               flops=2.5 * att_f * c / 2)
        dOs = [rnd(B, c, h, dh, dtype=torch.float32) for _ in range(4)]
        doc_a, cr_a, ls_a = torch.zeros(B, Tlen, h, dh, device=DEV, dtype=BF), z(B, Tlen, h), z(B, Tlen, h)
        dq_a = z(B, Tlen, h, dh)
        report("cell_finish_sweeps (4 sweeps)", T(lambda: ops.cell_finish_sweeps(
            dOs, scal, qc, ksc, vrc, o_c, lse_c, acc[0], acc[3], doc_a[:, r], cr_a[:, r], ls_a[:, r], acc[1][:, r],
            acc[2][:, r], dq_a[:, r], scale)), bytes_=B * c * h * dh * (4 * 4 + 3 * 2 + 3 * 4 + 3 * 8 + 2))
    if want("prefix_dq"):
        doc_c, corr = rnd(B, c, h, dh), rnd(B, c, h, dtype=torch.float32)
        both("prefix_dq", lambda: ops.prefix_dq(qc, Kc, Vc, pos0, scale, 0, lse_c, doc_c, corr, acc[0]),
             1.5 * att_f * pos0)
    if want("prefix_dkv"):
        Tq = 2048
        qa, da = rnd(B, Tq, h, dh), rnd(B, Tq, h, dh)
        Ka, Va = rnd(B, Tq, h, dh), rnd(B, Tq, h, dh)
        ca, la = rnd(B, Tq, h, dtype=torch.float32), rnd(B, Tq, h, dtype=torch.float32) + 8.0
        p0 = Tq - pos0 - c                       # as many later query rows as `pos0` keys elsewhere
        both("prefix_dkv", lambda: ops.prefix_dkv(qa, da, ca, la, Ka, Va, p0, c, p0 + c, scale, 0),
             2.0 * att_f * (Tq - p0 - c))
        if dh == 64:
            was = ops.dkv_rows128(False)
            ops.ATTN_TC = True
            report("prefix_dkv [tcgen05, 64-reader tiles]",
                   T(lambda: ops.prefix_dkv(qa, da, ca, la, Ka, Va, p0, c, p0 + c, scale, 0)), flops=2.0 * att_f * (Tq - p0 - c))
            ops.ATTN_TC = type(ops).ATTN_TC
            ops.dkv_rows128(was)
            ops.tc_check()
    if want("near"):
        # the near read of a full window of the 1.3B recipe: 16 sequences x 36 heads of 64, 8 chunks of 64 rows, each
        # reading the 7 chunks before it; single chunks per tile against two chunks per 128-row tile, and the merge
        # with the stored far partials as a kernel of its own against the read kernel's epilogue
        Bn, hn, Gn, Kn, Cn = 16, 36, 8, 8, 64
        lo_c = 16
        Tn = (lo_c + Gn) * Cn
        qn, Kt, Vt = rnd(Bn, Tn, hn, 64), rnd(Bn, Tn, hn, 64), rnd(Bn, Tn, hn, 64)
        of_, lf_ = rnd(Bn, Tn, hn, 64, dtype=torch.float32), rnd(Bn, Tn, hn, dtype=torch.float32)
        wn_ = slice(lo_c * Cn, (lo_c + Gn) * Cn)
        a_ = (qn[:, wn_], Kt, Vt, lo_c * Cn, (lo_c - Kn + 1) * Cn, Cn, 0.125, 0)
        fl = 4.0 * Bn * hn * 64 * Gn * Cn * (Kn - 1) * Cn
        for pairs in (False, True):
            ops.NEAR_PAIRS = pairs
            tag2 = "two chunks per tile" if pairs else "one chunk per tile"
            report(f"near read, {tag2}", T(lambda: ops.win_near_fwd(*a_)), flops=fl)
            report(f"near read + merge kernel, {tag2}",
                   T(lambda: ops.merge_partials(of_[:, wn_], lf_[:, wn_], *ops.win_near_fwd(*a_))), flops=fl)
            report(f"near read merged in its epilogue, {tag2}",
                   T(lambda: ops.win_near_merged(*a_, of_[:, wn_], lf_[:, wn_], keep_near=True)), flops=fl)
        ops.NEAR_PAIRS = type(ops).NEAR_PAIRS
        ops.tc_check()
    if want("bar"):
        # one lower-right causal read of a block of 1024 query rows over 4096 tape rows (the window read of a
        # layer-batched wavefront step), next to torch's fused attention backends on the same mask
        import torch.nn.functional as F
        from torch.nn.attention import SDPBackend, sdpa_kernel
        for (Bb, hb, dhb) in ((4, 36, 64), (4, 16, 128)):
            Lq, Lk = 1024, 4096
            qb, Kb, Vb = rnd(Bb, Lq, hb, dhb), rnd(Bb, Lk, hb, dhb), rnd(Bb, Lk, hb, dhb)
            sc = dhb ** -0.5
            fl = 4.0 * Bb * hb * dhb * sum(Lk - Lq + i + 1 for i in range(Lq))
            report(f"attn fwd tcgen05 {Bb}x{hb}x{dhb} {Lq}x{Lk}",
                   T(lambda: ops.attn_fwd_tc(qb, Kb, Vb, 0, Lk, Lk - Lq, sc, 0, True, 0, Lq=Lq, bm=128, out_dtype=BF)),
                   flops=fl)
            qt, kt, vt = (x.transpose(1, 2) for x in (qb, Kb, Vb))
            mask = torch.ones(Lq, Lk, dtype=torch.bool, device=DEV).tril(Lk - Lq)
            for be in (SDPBackend.CUDNN_ATTENTION, SDPBackend.EFFICIENT_ATTENTION):
                try:
                    with sdpa_kernel(be):
                        report(f"  torch sdpa {be.name.lower()} (same mask)",
                               T(lambda: F.scaled_dot_product_attention(qt, kt, vt, attn_mask=mask, scale=sc)), flops=fl)
                except Exception as e:                     # backend not offered for this case
                    print(f"  torch sdpa {be.name.lower()}: not available ({str(e)[:60]})", flush=True)
        ops.tc_check()
    # ---- refine / norms
    cos, sin = build_rope_cache(Tlen, dh, 10000.0, device=DEV)
    cg, glx, k, v = rnd(B, c, 4 * d), rnd(B, Tlen, 2 * d), rnd(B, Tlen, d), rnd(B, Tlen, d)
    N = B * c
    if want("refine_fwd"):
        for nt in (256, 128):
            ops.lib.dmb_refine_fwd_threads(nt)
            report(f"refine_fwd [{nt} threads per block]",
                   T(lambda: ops.refine_fwd(cg, ssq, glx[:, r], k[:, r], v[:, r], cos[r], sin[r], h, 0)), bytes_=N * d * 2 * 10)
    dK, dV = rnd(B, c, h, dh, dtype=torch.float32), rnd(B, c, h, dh, dtype=torch.float32)
    dk_a, dv_a, dg_a = z(B, Tlen, d), z(B, Tlen, d), z(B, Tlen, 2 * d)
    if want("refine_bwd"):
        dcg_o, uh_o, o2 = torch.empty_like(cg), rnd(B, c, d), o.reshape(B, c, d)
        for mb in (3, 4, 5):
            ops.lib.dmb_refine_bwd_minblocks(mb)
            report(f"refine_bwd [{mb} blocks per SM]",
                   T(lambda: ops.refine_bwd(dK, dV, cg, ssq, o2, glx[:, r], k[:, r], v[:, r], cos[r], sin[r], 0,
                                            dk_a[:, r], dv_a[:, r], dg_a[:, r], dcg_o, uh_o)), bytes_=N * d * 68)
        ops.lib.dmb_refine_bwd_minblocks(4)
        du = rnd(B, c, d)
        report("rmsn_bwd", T(lambda: ops.rmsn_bwd(du, o2, ssq)), bytes_=N * d * 8)
    # ---- write law of the mult_res family at the 18 x d2304 recipe's step: 16 sequences x a window of 512 rows, 36 heads
    if want("mrk"):
        Bm, cm, hm = 16, 512, 36
        dm = hm * dh
        Nm = Bm * cm
        cosm, sinm = build_rope_cache(cm, dh, 10000.0, device=DEV)
        raw_m, vc_m, o_m = rnd(Bm, cm, 4 * dm), rnd(Bm, cm, dm), rnd(Bm, cm, dm)
        ssq_m = (o_m.float().view(Bm, cm, hm, dh) ** 2).sum(-1)
        glx_m, k_m, v_m = rnd(Bm, cm, 2 * dm), rnd(Bm, cm, dm), rnd(Bm, cm, dm)
        kg = torch.ones(hm, device=DEV)
        report("mrk_refine_fwd", T(lambda: ops.mrk_refine_fwd(raw_m, vc_m, ssq_m, glx_m, k_m, v_m, cosm, sinm, hm, 0, kg, 1.0)),
               bytes_=Nm * dm * 2 * 11)
        dKm, dVm = rnd(Bm, cm, hm, dh, dtype=torch.float32), rnd(Bm, cm, hm, dh, dtype=torch.float32)
        dka, dva = z(Bm, cm, dm), z(Bm, cm, dm)
        dcg_m, uh_m, dvc_m, dkg_m = torch.empty_like(raw_m), torch.empty_like(o_m), torch.empty_like(o_m), z(Nm, hm)
        for mb in (2, 3, 4):
            ops.lib.dmb_mrk_refine_bwd_minblocks(mb)
            report(f"mrk_refine_bwd [{mb} blocks per SM]",
                   T(lambda: ops.mrk_refine_bwd(dKm, dVm, raw_m, vc_m, ssq_m, o_m, glx_m, k_m, v_m, cosm, sinm, 0, kg, 1.0,
                                                dka, dva, None, dcg_m, uh_m, dvc_m, dkg_m)), bytes_=Nm * dm * 52)
        ops.lib.dmb_mrk_refine_bwd_minblocks(4)
        assert not ops.fallbacks, ops.fallbacks
    if want("chain"):
        # one forward sweep (tail read -> packed GEMM -> refine) and one backward sweep (refine -> GEMM -> norm -> tail)
        # as their launches follow one another in a replayed CUDA graph of 16 sweeps, against the sum of the parts
        Wp = rnd(4 * d, d, scale=0.03)
        o2 = o.reshape(B, c, d)
        dcg_o, uh_o = torch.empty_like(cg), rnd(B, c, d)
        scal = torch.empty(3, B, c, h, device=DEV)

        def fwd_sweep():
            o_, lse_, ssq_ = ops.tail_fwd(qc, ksc, vrc, K_in, V_in, o_c, lse_c, scale, 0)
            raw = ops.linear(o_.reshape(B, c, d), Wp)
            ops.refine_fwd(raw, ssq_, glx[:, r], k[:, r], v[:, r], cos[r], sin[r], h, 0)

        def bwd_sweep():
            ops.refine_bwd(dK, dV, cg, ssq, o2, glx[:, r], k[:, r], v[:, r], cos[r], sin[r], 0, dk_a[:, r], dv_a[:, r],
                           None, dcg_o, uh_o)
            du_ = ops.linear_dx(dcg_o, Wp)
            d_o = ops.rmsn_bwd(du_, o2, ssq)
            ops.tail_bwd_sweep(d_o.view(B, c, h, dh), qc, ksc, K_in, V_in, lse_c, o, lse, scale, 0, acc[0], False, scal)

        for name, fn, n_k in (("forward sweep chain (3 launches)", fwd_sweep, 3), ("backward sweep chain (4 launches)", bwd_sweep, 4)):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for _ in range(16):
                    fn()
            us = T(gr.replay) / 16
            report(name + ", per sweep in a graph", us)
    x2, w = rnd(N, d), rnd(d) + 1
    if want("rms_fwd"):
        report("rms_fwd", T(lambda: ops.rms_fwd(x2, w)), bytes_=N * d * 4)
    y, rstd = ops.rms_fwd(x2, w)
    dwa = z(d)
    if want("rms_bwd"):
        report("rms_bwd (+dw)", T(lambda: ops.rms_bwd(x2, x2, w, rstd, dwa)), bytes_=N * d * (2 + 2 + 4 + 4))
    if want("ce"):
        lg, tg = rnd(4096, 32000), torch.randint(0, 32000, (4096,), device=DEV)
        inv = torch.tensor(1.0 / 4096, device=DEV)
        report("ce slab 4096x32000", T(lambda: ops.ce_chunk(lg, tg, inv)), bytes_=4096 * 32000 * 2 * 2)
    # ---- GEMMs: ours (128 x BN tiles per CTA, and 256 x 256 / 256 x 128 tiles on CTA pairs) vs torch.matmul (cuBLAS)
    if want("gemm") and ops.gemm is not None:
        g = ops.gemm

        def trio(name, fn, ref, flops):
            for tag_, flag, bn in (("1 CTA", False, 0), ("CTA pair 256x256", True, 256), ("CTA pair 256x128", True, 128)):
                g.pair = flag
                g.pair_width(bn)
                report(f"gemm {name} [{tag_}]", T(fn), flops=flops)
            g.pair = False
            g.pair_width(0)
            if g.ksplit:
                g.ksplit = False
                report(f"gemm {name} [1 CTA per tile, no K split across a CTA pair]", T(fn), flops=flops)
                g.ksplit = True
            report(f"  cublas {name}", T(ref), flops=flops)

        shapes = [("sweep y=uW^T", 2048, 4096, 1024), ("qkv", 65536, 1024, 1024), ("mlp up", 65536, 2816, 1024),
                  ("mlp down", 65536, 1024, 2816), ("head", 4096, 32000, 1024)]
        for name, M, Nn, K in shapes:
            a, wt = rnd(M, K), rnd(Nn, K)
            trio("tn " + name, lambda: g.linear(a, wt), lambda: a @ wt.t(), 2.0 * M * Nn * K)
        dy, wt = rnd(2048, 4096), rnd(4096, 1024)
        f = 2.0 * 2048 * 4096 * 1024
        trio("nn sweep du", lambda: g.linear_dx(dy, wt), lambda: dy @ wt, f)
        dyl, wl = rnd(65536, 2816), rnd(2816, 1024)
        trio("nn layer dx", lambda: g.linear_dx(dyl, wl), lambda: dyl @ wl, 2.0 * 65536 * 2816 * 1024)
        dW, xx = z(4096, 1024), rnd(2048, 1024)
        trio("dw sweep", lambda: g.linear_dw_acc(dW, dy, xx),
             lambda: dW.add_(torch.mm(dy.t(), xx, out_dtype=torch.float32)), f)
        dyb, xb, dWb = rnd(65536, 1024), rnd(65536, 1024), z(1024, 1024)
        trio("dw layer", lambda: g.linear_dw_acc(dWb, dyb, xb),
             lambda: dWb.add_(torch.mm(dyb.t(), xb, out_dtype=torch.float32)), 2.0 * 65536 * 1024 * 1024)
        dyp, xp, dWp = rnd(262144, 4096), rnd(262144, 1024), z(4096, 1024)
        trio("dw packed (262144 rows)", lambda: g.linear_dw_acc(dWp, dyp, xp),
             lambda: dWp.add_(torch.mm(dyp.t(), xp, out_dtype=torch.float32)), 2.0 * 262144 * 4096 * 1024)
        g.check()
    # ---- the skinny GEMMs of the rank-144 factored write law (18 x d2304 recipe: 8192 window rows per step)
    if want("gemm_lora") and ops.gemm is not None:
        g = ops.gemm
        M, dm, rk, nop = 8192, 2304, 144, 4
        u, t_all, raw = rnd(M, dm), rnd(M, nop * rk), rnd(M, 4 * dm)
        D_all, U = rnd(nop * rk, dm), rnd(dm, rk)
        t1, raw1 = t_all[:, rk:2 * rk], raw[:, dm:2 * dm]
        f = 2.0 * M * dm * nop * rk
        report("gemm tn down (4 operators)", T(lambda: g.linear(u, D_all, BF, out=t_all)), flops=f)
        report("  cublas down", T(lambda: torch.mm(u, D_all.t(), out=t_all)), flops=f)
        f1 = 2.0 * M * dm * rk
        report("gemm tn up (one operator)", T(lambda: g.linear(t1, U, BF, out=raw1)), flops=f1, bytes_=M * dm * 2)
        report("  cublas up", T(lambda: torch.mm(t1, U.t(), out=raw1)), flops=f1, bytes_=M * dm * 2)
        Dv, tv = rnd(rk, dm), rnd(M, rk)
        report("gemm tn down (one operator)", T(lambda: g.linear(u, Dv, BF, out=tv)), flops=f1, bytes_=M * dm * 2)
        report("  cublas down one", T(lambda: torch.mm(u, Dv.t(), out=tv)), flops=f1, bytes_=M * dm * 2)
        report("gemm nn d(down out) (one operator)", T(lambda: g.linear_dx(raw1, U, out=t1)), flops=f1, bytes_=M * dm * 2)
        report("  cublas d(down out)", T(lambda: torch.mm(raw1, U, out=t1)), flops=f1, bytes_=M * dm * 2)
        du = rnd(M, dm)
        report("gemm nn d(read) (4 operators)", T(lambda: g.linear_dx(t_all, D_all, out=du)), flops=f)
        report("  cublas d(read)", T(lambda: torch.mm(t_all, D_all, out=du)), flops=f)
        # the deferred weight gradients of the factors over all steps of a layer (71 steps x 8192 rows)
        rows_l = 71 * M
        dcg_l, t_l, u_l = rnd(rows_l, 4 * dm), rnd(rows_l, nop * rk), rnd(rows_l, dm)
        dU, dD = z(dm, rk), z(nop * rk, dm)
        fu, fd = 2.0 * rows_l * dm * rk, 2.0 * rows_l * nop * rk * dm
        report("gemm dw up factor (581 632 rows)", T(lambda: g.linear_dw_acc(dU, dcg_l[:, dm:2 * dm], t_l[:, rk:2 * rk])), flops=fu)
        report("  cublas dw up factor", T(lambda: dU.add_(torch.mm(dcg_l[:, dm:2 * dm].t(), t_l[:, rk:2 * rk], out_dtype=torch.float32))), flops=fu)
        report("gemm dw stacked down factors", T(lambda: g.linear_dw_acc(dD, t_l, u_l)), flops=fd)
        report("  cublas dw stacked down factors", T(lambda: dD.add_(torch.mm(t_l.t(), u_l, out_dtype=torch.float32))), flops=fd)
        g.check()
    return rows


if __name__ == "__main__":
    main()
