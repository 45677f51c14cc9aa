"""Numerics of every sm_100a kernel against the plain-torch fp32 statement of the
same op (engines/fused_math.py), on bf16 inputs of engine-like shapes."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from dual_mod_public_b200.engines import fused_math as fm
from dual_mod_public_b200.models import build_rope_cache
from dual_mod_public_b200.ops import TorchOps


@pytest.fixture(scope="module")
def ops():
    from dual_mod_public_b200.ops.cuda_ops import CudaOps
    return CudaOps(torch.device("cuda:0"))


DEV = "cuda:0"
REF = TorchOps()


def rnd(*shape, scale=1.0, dtype=torch.bfloat16, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(DEV).to(dtype)


def close(a, b, rtol=2e-2, atol=2e-2, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"{what}: max err {err:.4g} vs ref scale {ref:.4g}"


def test_library_loaded(ops):
    assert ops.name == "sm100a" and ops.lib is not None


@pytest.mark.parametrize("rows,d", [(4096, 1024), (333, 2304), (64, 128)])
def test_rms_fwd_bwd(ops, rows, d):
    x, w, dy = rnd(rows, d), rnd(d, scale=0.3, seed=1) + 1, rnd(rows, d, seed=2)
    n0 = ops.launches
    y, rstd = ops.rms_fwd(x, w)
    assert ops.launches > n0
    y_ref, rstd_ref = fm.rms_fwd(x.float(), w.float())
    close(y, y_ref, what="rms y")
    close(rstd, rstd_ref, rtol=1e-3, atol=1e-4, what="rstd")
    dw = torch.zeros(d, device=DEV)
    res = rnd(rows, d, seed=3)
    dx = ops.rms_bwd(dy, x, w, rstd, dw, residual=res, out_dtype=torch.bfloat16)
    dx_ref, dw_ref = fm.rms_bwd(dy.float(), x.float(), w.float(), rstd_ref)
    close(dx, dx_ref + res.float(), what="rms dx")
    close(dw, dw_ref, rtol=2e-2, atol=0.05 * dw_ref.abs().mean().item() + 1e-3, what="rms dw")
    dxf = ops.rms_bwd(dy.float(), x, w, rstd, torch.zeros(d, device=DEV))
    close(dxf, dx_ref, rtol=1e-2, atol=1e-2, what="rms dx fp32")


@pytest.mark.parametrize("dh", [64, 128])
def test_rope_roundtrip(ops, dh):
    B, T, H = 2, 96, 4
    cos, sin = build_rope_cache(T, dh, 10000.0, device=DEV)
    full = rnd(B, 128, H, dh)
    x = full[:, 16:16 + T]                                    # batch-strided view
    y = ops.rope(x, cos, sin)
    close(y, fm.rope_tm(x.float(), cos, sin), what="rope")
    xf = rnd(B, T, H, dh, dtype=torch.float32, seed=5)
    close(ops.unrope(ops.rope(xf, cos, sin), cos, sin), xf, rtol=1e-5, atol=1e-5, what="unrope")


def test_swiglu(ops):
    h1, h3, dg = rnd(512, 2816), rnd(512, 2816, seed=1), rnd(512, 2816, seed=2)
    close(ops.swiglu_fwd(h1, h3), fm.swiglu_fwd(h1.float(), h3.float()), what="swiglu")
    d1, d3 = ops.swiglu_bwd(dg, h1, h3)
    r1, r3 = fm.swiglu_bwd(dg.float(), h1.float(), h3.float())
    close(d1, r1, what="dh1")
    close(d3, r3, what="dh3")


def test_ce_slab(ops):
    n, V = 300, 32000
    logits = rnd(n, V, scale=2.0)
    tg = torch.randint(0, V, (n,), device=DEV)
    tg[5] = -1
    inv_n = 1.0 / (tg >= 0).sum().float()
    loss, dl = ops.ce_chunk(logits, tg, inv_n)
    loss_ref, dl_ref = fm.ce_chunk(logits.float(), tg, inv_n)
    assert abs(loss.item() - loss_ref.item()) < 2e-3 * abs(loss_ref.item())
    close(dl, dl_ref, rtol=2e-2, atol=1e-6, what="dlogits")


def _cell_inputs(B, c, H, dh, T, seed=0):
    q = rnd(B, T, H, dh, scale=1.0, seed=seed)
    ks = rnd(B, T, H, dh, seed=seed + 1)
    vr = rnd(B, T, H, dh, seed=seed + 2)
    Kc = rnd(B, T, H, dh, seed=seed + 3)
    Vc = rnd(B, T, H, dh, seed=seed + 4)
    return q, ks, vr, Kc, Vc


@pytest.mark.parametrize("c,dh,pos0,window", [(64, 64, 192, 0), (64, 128, 128, 0), (32, 64, 96, 0),
                                              (16, 64, 48, 0), (64, 64, 192, 100), (64, 64, 0, 0)])
def test_prefix_and_tail_fwd_bwd(ops, c, dh, pos0, window):
    B, H, T = 3, 4, pos0 + c
    scale = dh ** -0.5
    q, ks, vr, Kc, Vc = _cell_inputs(B, c, H, dh, T)
    r = slice(pos0, pos0 + c)
    qc, ksc, vrc = q[:, r], ks[:, r], vr[:, r]
    K_in, V_in = rnd(B, c, H, dh, seed=9), rnd(B, c, H, dh, seed=10)
    f = lambda t: t.float()
    # ---- forward
    o_c, lse_c = ops.prefix_fwd(qc, Kc, Vc, pos0, scale, window)
    o_c_ref, lse_c_ref = fm.prefix_fwd(f(qc), f(Kc), f(Vc), pos0, scale, window)
    close(o_c, o_c_ref, what="o_c")
    live = lse_c_ref > -1e29
    if live.any():
        close(lse_c[live], lse_c_ref[live], rtol=1e-2, atol=2e-2, what="lse_c")
    assert (lse_c[~live] < -1e29).all()
    o, lse, ssq = ops.tail_fwd(qc, ksc, vrc, K_in, V_in, o_c_ref, lse_c_ref, scale, window)
    o_ref, lse_ref, ssq_ref = fm.tail_fwd(f(qc), f(ksc), f(vrc), f(K_in), f(V_in), o_c_ref, lse_c_ref, scale, window)
    close(o, o_ref, what="tail o")
    close(lse, lse_ref, rtol=1e-2, atol=2e-2, what="tail lse")
    close(ssq, ssq_ref, rtol=2e-2, atol=1e-3, what="tail ssq")
    # ---- tail backward
    dO = rnd(B, c, H, dh, dtype=torch.float32, seed=11)
    z = lambda *s: torch.zeros(*s, device=DEV)
    acc = [z(B, c, H, dh), z(B, T, H, dh), z(B, T, H, dh), z(B, c, H, dh), z(B, c, H)]
    dK_in, dV_in = ops.tail_bwd(dO, qc, ksc, vrc, K_in, V_in, o_c_ref, lse_c_ref, o_ref.to(torch.bfloat16),
                                lse_ref, scale, window, acc[0], acc[1][:, r], acc[2][:, r], acc[3], acc[4])
    ref = fm.tail_bwd(dO, f(qc), f(ksc), f(vrc), f(K_in), f(V_in), o_c_ref, lse_c_ref, o_ref, lse_ref,
                      scale, window)
    names = ["dq", "dkself", "dvraw", "dK_in", "dV_in", "do_c", "dlse_c"]
    got = [acc[0], acc[1][:, r], acc[2][:, r], dK_in, dV_in, acc[3], acc[4]]
    for n_, g_, r_ in zip(names, got, ref):
        close(g_, r_, rtol=3e-2, atol=3e-2, what=n_)
    assert acc[1][:, :pos0].abs().max() == 0 if pos0 else True
    # ---- prefix backward, query side
    do_c, dlse_c = ref[5], ref[6]
    corr = (do_c * o_c_ref).sum(-1) - dlse_c
    dq_acc, dq_r = z(B, c, H, dh), z(B, c, H, dh)
    ops.prefix_dq(qc, Kc, Vc, pos0, scale, window, lse_c_ref, do_c.to(torch.bfloat16), corr, dq_acc)
    fm.prefix_dq(f(qc), f(Kc), f(Vc), pos0, scale, window, lse_c_ref, do_c, corr, dq_r)
    close(dq_acc, dq_r, rtol=3e-2, atol=3e-2, what="prefix dq")


@pytest.mark.parametrize("c,dh,window,H,n_sweeps", [(64, 64, 0, 4, 3), (64, 128, 0, 3, 2), (32, 64, 20, 5, 4), (16, 64, 0, 4, 1)])
def test_deferred_sweeps_equal_per_sweep_accumulation(ops, c, dh, window, H, n_sweeps):
    """`tail_bwd_sweep` per sweep + `cell_finish_sweeps` once per cell against the per-sweep fp32 statement
    (`tail_bwd` accumulating every sweep, then `cell_finish`)."""
    B, pos0 = 2, 2 * c
    T = pos0 + 2 * c
    scale = dh ** -0.5
    q, ks, vr, Kc, Vc = _cell_inputs(B, c, H, dh, T)
    r = slice(pos0, pos0 + c)
    qc, ksc, vrc = q[:, r], ks[:, r], vr[:, r]
    f = lambda t: t.float()
    o_c, lse_c = fm.prefix_fwd(f(qc), f(Kc), f(Vc), pos0, scale, window)
    z = lambda *s: torch.zeros(*s, device=DEV)
    sweeps = []
    for s_ in range(n_sweeps):
        K_in, V_in = rnd(B, c, H, dh, seed=20 + s_), rnd(B, c, H, dh, seed=40 + s_)
        o, lse, _ = fm.tail_fwd(f(qc), f(ksc), f(vrc), f(K_in), f(V_in), o_c, lse_c, scale, window)
        sweeps.append((K_in, V_in, o.to(torch.bfloat16), lse, rnd(B, c, H, dh, dtype=torch.float32, seed=60 + s_)))
    dK0, dV0 = rnd(B, c, H, dh, dtype=torch.float32, seed=5), rnd(B, c, H, dh, dtype=torch.float32, seed=6)

    def arrays():      # doc, corr, lsec, dks, dv, dq by absolute position (dks / dv / dq start non-zero)
        return [torch.zeros(B, T, H, dh, device=DEV, dtype=torch.bfloat16), z(B, T, H), z(B, T, H),
                rnd(B, T, H, dh, dtype=torch.float32, seed=7), rnd(B, T, H, dh, dtype=torch.float32, seed=8),
                rnd(B, T, H, dh, dtype=torch.float32, seed=9)]
    # statement: every sweep accumulates, then cell_finish
    a = arrays()
    do_c, dlse_c = z(B, c, H, dh), z(B, c, H)
    dq_cell = z(B, c, H, dh)
    for K_in, V_in, o, lse, dO in reversed(sweeps):
        REF.tail_bwd(dO, f(qc), f(ksc), f(vrc), f(K_in), f(V_in), o_c, lse_c, o.float(), lse, scale, window,
                     dq_cell, a[3][:, r], a[4][:, r], do_c, dlse_c)
    a[5][:, r] = dq_cell                      # the first sweep processed writes the cell's d q
    cv_ref = REF.cell_finish(do_c, dlse_c, o_c, lse_c, dK0, dV0, a[0][:, r], a[1][:, r], a[2][:, r], a[3][:, r], a[4][:, r])
    # kernels: deferred
    b_ = arrays()
    scal = torch.empty(n_sweeps, 3, B, c, H, device=DEV)
    outs = []
    for s_ in range(n_sweeps - 1, -1, -1):
        K_in, V_in, o, lse, dO = sweeps[s_]
        outs.append(ops.tail_bwd_sweep(dO, qc, ksc, K_in, V_in, lse_c, o, lse, scale, window, b_[5][:, r],
                                       s_ == n_sweeps - 1, scal[s_]))
        ref = fm.tail_bwd(dO, f(qc), f(ksc), f(vrc), f(K_in), f(V_in), o_c, lse_c, o.float(), lse, scale, window)
        close(outs[-1][0], ref[3], rtol=3e-2, atol=3e-2, what="dK_in")
        close(outs[-1][1], ref[4], rtol=3e-2, atol=3e-2, what="dV_in")
    cv = ops.cell_finish_sweeps([t[4] for t in sweeps], scal, qc, ksc, vrc, o_c, lse_c, dK0, dV0, b_[0][:, r],
                                b_[1][:, r], b_[2][:, r], b_[3][:, r], b_[4][:, r], b_[5][:, r], scale)
    close(cv, cv_ref, rtol=3e-2, atol=3e-2, what="corr")
    for x, y, n_ in zip(b_, a, ("doc", "corr", "lsec", "dks", "dv", "dq")):
        close(x, y, rtol=3e-2, atol=3e-2, what=n_)
    out = torch.ones(T, dtype=torch.bool, device=DEV)
    out[r] = False
    fresh = arrays()
    for x, y in zip(b_, fresh):
        assert torch.equal(x[:, out], y[:, out])


@pytest.mark.parametrize("c,dh,pos0,T,window", [(64, 64, 128, 512, 0), (64, 128, 64, 300, 0), (32, 64, 32, 200, 0),
                                                (16, 64, 48, 128, 0), (64, 64, 128, 512, 150), (64, 64, 448, 512, 0)])
def test_prefix_dkv_owner_computes(ops, c, dh, pos0, T, window):
    B, H = 2, 4
    scale = dh ** -0.5
    q, doc = rnd(B, T, H, dh), rnd(B, T, H, dh, seed=1)
    Kc, Vc = rnd(B, T, H, dh, seed=2), rnd(B, T, H, dh, seed=3)
    corr = rnd(B, T, H, dtype=torch.float32, seed=4)
    # a plausible lse_c per row: log-sum-exp of that row's scores over its whole prefix
    s = torch.einsum("bthd,bjhd->bhtj", q.float(), Kc.float()) * scale
    lsec = torch.logsumexp(s, dim=-1).permute(0, 2, 1).contiguous() + 1.0
    q_start = pos0 + c
    dK, dV = ops.prefix_dkv(q, doc, corr, lsec, Kc, Vc, pos0, c, q_start, scale, window)
    dK_r, dV_r = fm.prefix_dkv(q.float(), doc.float(), corr, lsec, Kc.float(), Vc.float(), pos0, c, q_start,
                               scale, window)
    close(dK, dK_r, rtol=3e-2, atol=3e-2, what="dK")
    close(dV, dV_r, rtol=3e-2, atol=3e-2, what="dV")


@pytest.mark.parametrize("pin", [0, 64])
def test_refine_fwd_bwd(ops, pin):
    B, c, H, dh, T = 2, 64, 16, 64, 128
    d = H * dh
    cos, sin = build_rope_cache(T, dh, 10000.0, device=DEV)
    r = slice(64, 128)
    raw, o = rnd(B, c, 4 * d, scale=2.0), rnd(B, c, d, scale=1.5, seed=7)
    ssq = o.float().view(B, c, H, dh).square().sum(-1)
    glx, k, v = rnd(B, T, 2 * d, seed=1), rnd(B, T, d, seed=2), rnd(B, T, d, seed=3)
    f = lambda t: t.float()
    K_out, V_out = ops.refine_fwd(raw, ssq, glx[:, r], k[:, r], v[:, r], cos[r], sin[r], H, pin)
    Kr, Vr = fm.refine_fwd(f(raw), ssq, f(glx[:, r]), f(k[:, r]), f(v[:, r]), cos[r], sin[r], H, pin)
    close(K_out, Kr, what="K''")
    close(V_out, Vr, what="V''")
    dK, dV = rnd(B, c, H, dh, dtype=torch.float32, seed=4), rnd(B, c, H, dh, dtype=torch.float32, seed=5)
    z = lambda *s: torch.zeros(*s, device=DEV)
    dk_acc, dv_acc, dg_acc = z(B, T, d), z(B, T, d), z(B, T, 2 * d)
    dcg = torch.empty(B, c, 4 * d, dtype=torch.bfloat16, device=DEV)
    uhat = torch.empty(B, c, d, dtype=torch.bfloat16, device=DEV)
    ops.refine_bwd(dK, dV, raw, ssq, o, glx[:, r], k[:, r], v[:, r], cos[r], sin[r], pin,
                   dk_acc[:, r], dv_acc[:, r], dg_acc[:, r], dcg, uhat)
    dcg_r, dk_r, dv_r, uh_r = fm.refine_bwd(dK, dV, f(raw), ssq, f(o), f(glx[:, r]), f(k[:, r]), f(v[:, r]),
                                            cos[r], sin[r], pin)
    close(dcg, dcg_r, what="dcg")
    close(uhat, uh_r, what="uhat")
    close(dk_acc[:, r], dk_r, what="dk")
    close(dv_acc[:, r], dv_r, what="dv")
    close(dg_acc[:, r], dcg_r[..., 2 * d:], what="dglx")
    assert dk_acc[:, :64].abs().max() == 0
    du, res = rnd(B, c, d, seed=8), rnd(B, c, d, dtype=torch.float32, seed=9)
    close(ops.rmsn_bwd(du, o, ssq, residual=res), fm.rmsn_bwd(f(du), f(o), ssq) + res, what="rmsn_bwd")
    close(ops.rmsn_bwd(du, o, ssq, out_dtype=torch.bfloat16), fm.rmsn_bwd(f(du), f(o), ssq), what="rmsn_bwd bf16")


@pytest.mark.parametrize("H", [16, 8])
def test_norm_backward_at_the_sweep_shape(ops, H):
    """d = 1024, 2048 rows and a ragged 1001, both result types, with and without the residual."""
    from dual_mod_public_b200.engines import fused_math as fm
    d = 1024
    for rows in (2048, 1001):
        du, o = rnd(1, rows, d, seed=21), rnd(1, rows, d, seed=22)
        ssq = (o.float().view(1, rows, H, d // H) ** 2).sum(-1)
        res = rnd(1, rows, d, dtype=torch.float32, seed=23)
        ref = fm.rmsn_bwd(du.float(), o.float(), ssq)
        close(ops.rmsn_bwd(du, o, ssq), ref, what="fp32 out")
        close(ops.rmsn_bwd(du, o, ssq, residual=res), ref + res, what="fp32 out + residual")
        close(ops.rmsn_bwd(du, o, ssq, out_dtype=torch.bfloat16), ref, what="bf16 out")
        rb = res.bfloat16()
        close(ops.rmsn_bwd(du, o, ssq, residual=rb, out_dtype=torch.bfloat16), ref + rb.float(), what="bf16 out + residual")
    assert "rmsn_bwd" not in ops.fallbacks


def test_col_sum(ops):
    x = rnd(1000, 2048, dtype=torch.float32)
    out = torch.ones(2048, device=DEV)
    ops.col_sum_acc(out, x)
    close(out, 1 + x.sum(0), rtol=1e-4, atol=1e-3, what="colsum")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_embedding_backward_is_exact_and_repeatable(ops, dtype):
    """Sorted-run scatter: fp32 sums of the rows per id, the same bits on every call."""
    V, d, n = 97, 256, 5000
    idx = torch.randint(0, V, (n,), device=DEV)
    idx[:1500] = 3                                  # one long run
    dx = rnd(n, d, dtype=dtype)
    ref = torch.ones(V, d, device=DEV, dtype=torch.float64)
    ref.index_add_(0, idx, dx.double())
    outs = []
    for _ in range(2):
        gw = torch.ones(V, d, device=DEV)
        ops.embed_bwd(gw, idx, dx)
        outs.append(gw)
    close(outs[0], ref.float(), rtol=1e-5, atol=1e-4, what="embed_bwd")
    assert torch.equal(outs[0], outs[1])


@pytest.mark.parametrize("dh,C,G,lo_chunk,K", [(64, 64, 3, 2, 4), (128, 64, 2, 0, 4), (64, 32, 4, 5, 3)])
def test_window_ops_match_per_chunk_statement(ops, dh, C, G, lo_chunk, K):
    """The group-dimension launches (G window chunks at once) against the per-chunk torch statement."""
    B, H = 2, 4
    T = (lo_chunk + G + 1) * C
    scale = dh ** -0.5
    q, ks, vr, Kc, Vc = _cell_inputs(B, C, H, dh, T)
    w = slice(lo_chunk * C, (lo_chunk + G) * C)
    f = lambda t: t.float()
    pos0, lo = lo_chunk * C, (lo_chunk - K + 1) * C
    # near read
    o_n, lse_n = ops.win_near_fwd(q[:, w], Kc, Vc, pos0, lo, C, scale)
    o_nr, lse_nr = REF.win_near_fwd(f(q[:, w]), f(Kc), f(Vc), pos0, lo, C, scale)
    close(o_n, o_nr, what="near o")
    live = lse_nr > -1e29
    close(lse_n[live], lse_nr[live], rtol=1e-2, atol=2e-2, what="near lse")
    assert (lse_n[~live] < -1e29).all()
    # merge with a far partial stored by absolute position
    ofar, lsefar = rnd(B, T, H, dh, dtype=torch.float32, seed=21), rnd(B, T, H, dtype=torch.float32, seed=22) + 3.0
    got = ops.merge_partials(ofar[:, w], lsefar[:, w], o_nr, lse_nr)
    ref = REF.merge_partials(ofar[:, w], lsefar[:, w], o_nr, lse_nr)
    for a, b_, n_ in zip(got, ref, ("o_c", "lse_c", "w_f", "w_n")):
        close(a, b_, rtol=1e-4, atol=1e-4, what=n_)
    o_c, lse_c, w_f, w_n = ref
    # tail forward / backward over the window
    o, lse, ssq = ops.win_tail_fwd(q[:, w], ks[:, w], vr[:, w], Kc[:, w], Vc[:, w], o_c, lse_c, C, scale)
    o_r, lse_r, ssq_r = REF.win_tail_fwd(f(q[:, w]), f(ks[:, w]), f(vr[:, w]), f(Kc[:, w]), f(Vc[:, w]), o_c, lse_c, C, scale)
    close(o, o_r, what="win tail o")
    close(lse, lse_r, rtol=1e-2, atol=2e-2, what="win tail lse")
    dO = rnd(B, G * C, H, dh, dtype=torch.float32, seed=23)
    z = lambda *s: torch.zeros(*s, device=DEV)
    acc = [z(B, G * C, H, dh), z(B, T, H, dh), z(B, T, H, dh), z(B, G * C, H, dh), z(B, G * C, H)]
    accr = [t.clone() for t in acc]
    dK, dV = ops.win_tail_bwd(dO, q[:, w], ks[:, w], vr[:, w], Kc[:, w], Vc[:, w], o_c, lse_c, o_r.to(torch.bfloat16),
                              lse_r, C, scale, acc[0], acc[1][:, w], acc[2][:, w], acc[3], acc[4])
    dKr, dVr = REF.win_tail_bwd(dO, f(q[:, w]), f(ks[:, w]), f(vr[:, w]), f(Kc[:, w]), f(Vc[:, w]), o_c, lse_c, o_r,
                                lse_r, C, scale, accr[0], accr[1][:, w], accr[2][:, w], accr[3], accr[4])
    for a, b_, n_ in zip([dK, dV] + acc, [dKr, dVr] + accr, ("dK_in", "dV_in", "dq", "dks", "dv", "do_c", "dlse_c")):
        close(a, b_, rtol=3e-2, atol=3e-2, what=n_)
    # the same launch with the raw-row gradients deferred: d k_self / d v_raw untouched, (p_self, dss) stashed
    acc2 = [z(B, G * C, H, dh), torch.full((B, T, H, dh), 3.0, device=DEV), torch.full((B, T, H, dh), 5.0, device=DEV),
            z(B, G * C, H, dh), z(B, G * C, H)]
    stash = torch.empty(2, B, G * C, H, device=DEV)
    dK2, dV2 = ops.win_tail_bwd(dO, q[:, w], ks[:, w], vr[:, w], Kc[:, w], Vc[:, w], o_c, lse_c, o_r.to(torch.bfloat16),
                                lse_r, C, scale, acc2[0], acc2[1][:, w], acc2[2][:, w], acc2[3], acc2[4], raw_stash=stash)
    ps_r, dss_r = fm.tail_self_scalars(dO, f(q[:, w]), f(ks[:, w]), f(vr[:, w]), o_r, lse_r, scale)
    close(stash[0], ps_r, rtol=3e-2, atol=1e-3, what="stash p_self")
    close(stash[1], dss_r, rtol=3e-2, atol=3e-2, what="stash dss")
    assert (acc2[1] == 3.0).all() and (acc2[2] == 5.0).all()
    for a, b_, n_ in zip([dK2, dV2, acc2[0], acc2[3], acc2[4]], [dKr, dVr, accr[0], accr[3], accr[4]],
                         ("dK_in", "dV_in", "dq", "do_c", "dlse_c")):
        close(a, b_, rtol=3e-2, atol=3e-2, what=n_ + " (raw deferred)")
    # split + near backward (query side and key side)
    DOf, DLf = z(B, T, H, dh), z(B, T, H)
    docn, corrn, lsen = torch.zeros(B, T, H, dh, device=DEV, dtype=torch.bfloat16), z(B, T, H), z(B, T, H)
    R_ = [t.clone() for t in (DOf, DLf, docn, corrn, lsen)]
    ops.split_partials(accr[3], accr[4], ofar[:, w], o_c, o_nr, lse_nr, w_f, w_n, DOf[:, w], DLf[:, w], docn[:, w],
                       corrn[:, w], lsen[:, w])
    REF.split_partials(accr[3], accr[4], ofar[:, w], o_c, o_nr, lse_nr, w_f, w_n, R_[0][:, w], R_[1][:, w], R_[2][:, w],
                       R_[3][:, w], R_[4][:, w])
    for a, b_, n_ in zip((DOf, DLf, docn, corrn, lsen), R_, ("DOf", "DLf", "docn", "corrn", "lsen")):
        close(a, b_, rtol=1e-2, atol=1e-3, what=n_)
    # the optional dense copy of corr_n
    dense = torch.full((B, G * C, H), 7.0, device=DEV)
    ops.split_partials(accr[3], accr[4], ofar[:, w], o_c, o_nr, lse_nr, w_f, w_n, DOf[:, w].clone(), DLf[:, w].clone(),
                       docn[:, w], corrn[:, w], lsen[:, w], corrn_dense=dense)
    close(dense, R_[3][:, w], rtol=1e-2, atol=1e-3, what="corrn dense")
    dq, dqr = z(B, G * C, H, dh), z(B, G * C, H, dh)
    ops.win_near_dq(q[:, w], Kc, Vc, pos0, lo, C, scale, lse_nr, R_[2][:, w], R_[3][:, w].contiguous(), dq)
    REF.win_near_dq(f(q[:, w]), f(Kc), f(Vc), pos0, lo, C, scale, lse_nr, R_[2][:, w].float(), R_[3][:, w].contiguous(), dqr)
    close(dq, dqr, rtol=3e-2, atol=3e-2, what="near dq")
    j0 = max(0, lo_chunk - K + 1)
    Gk = lo_chunk + G - 1 - j0
    if Gk > 0:
        lsen_full = torch.where(R_[4] == 0, torch.full_like(R_[4], 5.0), R_[4])
        a = ops.win_near_dkv(q, R_[2], R_[3], lsen_full, Kc, Vc, j0, Gk, C, pos0, (lo_chunk + G) * C, K * C, scale)
        b_ = REF.win_near_dkv(f(q), R_[2].float(), R_[3], lsen_full, f(Kc), f(Vc), j0, Gk, C, pos0, (lo_chunk + G) * C, K * C, scale)
        close(a[0], b_[0], rtol=3e-2, atol=3e-2, what="near dK")
        close(a[1], b_[1], rtol=3e-2, atol=3e-2, what="near dV")


@pytest.mark.parametrize("dh", [64, 128])
def test_cell_finish(ops, dh):
    B, T, c, H, pos0 = 2, 160, 64, 4, 64
    r = slice(pos0, pos0 + c)
    f = lambda *s, seed: rnd(*s, dtype=torch.float32, seed=seed)
    do_c, dlse_c, o_c, lse_c = f(B, c, H, dh, seed=1), f(B, c, H, seed=2), f(B, c, H, dh, seed=3), f(B, c, H, seed=4)
    dK0, dV0 = f(B, c, H, dh, seed=5), f(B, c, H, dh, seed=6)

    def arrays():
        return (torch.zeros(B, T, H, dh, device=DEV, dtype=torch.bfloat16), torch.zeros(B, T, H, device=DEV),
                torch.zeros(B, T, H, device=DEV), f(B, T, H, dh, seed=7), f(B, T, H, dh, seed=8))
    a, b_ = arrays(), arrays()
    cv = ops.cell_finish(do_c, dlse_c, o_c, lse_c, dK0, dV0, a[0][:, r], a[1][:, r], a[2][:, r], a[3][:, r], a[4][:, r])
    cr = REF.cell_finish(do_c, dlse_c, o_c, lse_c, dK0, dV0, b_[0][:, r], b_[1][:, r], b_[2][:, r], b_[3][:, r], b_[4][:, r])
    close(cv, cr, rtol=1e-4, atol=1e-4, what="corr")
    for x, y, n_ in zip(a, b_, ("doc", "corr_all", "lsec", "dks", "dv")):
        close(x, y, rtol=1e-2, atol=1e-4, what=n_)


@pytest.mark.parametrize("dh,doc_dtype", [(64, torch.bfloat16), (128, torch.float32)])
def test_chunk_finish(ops, dh, doc_dtype):
    """End of a wavefront chunk's backward (one launch) against its torch statement, on views by absolute position."""
    B, T, c, H, pos0 = 2, 192, 64, 3, 64
    r = slice(pos0, pos0 + c)
    f = lambda *s, seed: rnd(*s, dtype=torch.float32, seed=seed)

    def arrays():
        # DOf, DLf, o_f, lse_f, dKp, dVp, dks, dv, doc, corr, lsec
        return [f(B, T, H, dh, seed=1), f(B, T, H, seed=2), f(B, T, H, dh, seed=3), f(B, T, H, seed=4),
                f(B, T, H, dh, seed=5), f(B, T, H, dh, seed=6), f(B, T, H, dh, seed=7), f(B, T, H, dh, seed=8),
                torch.zeros(B, T, H, dh, device=DEV, dtype=doc_dtype), torch.zeros(B, T, H, device=DEV),
                torch.zeros(B, T, H, device=DEV)]
    a, b_ = arrays(), arrays()
    before = [t.clone() for t in a]
    cv, ls = ops.chunk_finish(*[t[:, r] for t in a])
    cr, lr = REF.chunk_finish(*[t[:, r] for t in b_])
    close(cv, cr, rtol=1e-4, atol=1e-4, what="corr")
    close(ls, lr, rtol=0, atol=0, what="lse")
    assert cv.is_contiguous() and ls.is_contiguous()
    names = ("DOf", "DLf", "o_f", "lse_f", "dKp", "dVp", "dks", "dv", "doc", "corr", "lsec")
    for x, y, n_ in zip(a, b_, names):
        close(x, y, rtol=1e-2, atol=1e-4, what=n_)
    assert (a[4][:, r] == 0).all() and (a[5][:, r] == 0).all()
    out = torch.ones(T, dtype=torch.bool, device=DEV)
    out[r] = False
    for x, y, n_ in zip(a, before, names):                       # rows of other chunks are untouched
        assert torch.equal(x[:, out], y[:, out]), n_
    # with the raw-row gradients of three sweeps deferred to this kernel (views into windows of different widths), and
    # with the gates' x-logit gradient summed from the sweeps' stashed d(ctx / gate logits) rows
    for with_gates in (False, True):
        a, b_ = arrays(), arrays()
        q = rnd(B, T, H, dh, seed=30)
        d = H * dh
        sweeps = []
        for k, (G, g) in enumerate(((3, 2), (2, 0), (1, 0))):
            d_o, st = f(B, G * c, H, dh, seed=40 + k), f(2, B, G * c, H, seed=50 + k)
            gr = slice(g * c, (g + 1) * c)
            extra = (rnd(B, G * c, 4 * d, seed=60 + k)[:, gr],) if with_gates else ()
            sweeps.append((d_o[:, gr], st[0][:, gr], st[1][:, gr]) + extra)
        gl = [torch.full((B, T, 2 * d), 9.0, device=DEV) for _ in range(2)] if with_gates else [None, None]
        view = lambda t: t[:, r] if t is not None else None
        cv, ls = ops.chunk_finish(*[t[:, r] for t in a], sweeps=sweeps, q=q[:, r], dglx=view(gl[0]))
        cr, lr = REF.chunk_finish(*[t[:, r] for t in b_], sweeps=sweeps, q=q[:, r], dglx=view(gl[1]))
        close(cv, cr, rtol=1e-4, atol=1e-4, what="corr (sweeps)")
        for x, y, n_ in zip(a, b_, names):
            close(x, y, rtol=1e-2, atol=1e-4, what=n_ + " (sweeps)")
        if with_gates:
            close(gl[0], gl[1], rtol=1e-3, atol=1e-3, what="dglx")
            assert (gl[0][:, out] == 9.0).all()
    assert not ops.fallbacks.get("chunk_finish") or DEV == "cpu"


def test_narrow_products_through_the_library_and_the_own_kernel(ops):
    """Factor products marked `narrow` (library GEMM by default) against the tcgen05 kernel and fp32, into column blocks."""
    M, d, r_ = 2048, 768, 144
    u, D, U = rnd(M, d, seed=1), rnd(4 * r_, d, seed=2, scale=0.05), rnd(d, r_, seed=3, scale=0.05)
    raw = torch.zeros(M, 4 * d, device=DEV, dtype=torch.bfloat16)
    outs = {}
    for mode in (True, False):
        ops.LIB_NARROW = mode
        n0 = ops.lib_gemms
        try:
            t = ops.linear(u, D, narrow=True)
            ops.linear(t[:, r_:2 * r_], U, out=raw[:, d:2 * d], narrow=True)
            dt = ops.linear_dx(raw[:, d:2 * d], U, narrow=True)
            du = ops.linear_dx(t, D, narrow=True)
        finally:
            ops.LIB_NARROW = type(ops).LIB_NARROW
        assert (ops.lib_gemms - n0) == (4 if mode else 0)
        outs[mode] = (t.clone(), raw[:, d:2 * d].clone(), dt, du)
        assert (raw[:, :d] == 0).all() and (raw[:, 2 * d:] == 0).all()
    ref_t = u.float() @ D.float().t()
    close(outs[True][0], ref_t, what="t (library)")
    for a, b_, n_ in zip(outs[True], outs[False], ("t", "up", "dt", "du")):
        close(a, b_, rtol=2e-2, atol=2e-2, what=n_ + ": library vs own kernel")


def test_copy_pair(ops):
    B, T, H, dh = 3, 320, 5, 64
    tape = [rnd(B, T, H, dh, seed=i) for i in (1, 2)]
    store = [torch.zeros(B, 192, H, dh, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    w = slice(64, 192)
    ops.copy_pair(store[0][:, :128], tape[0][:, w], store[1][:, :128], tape[1][:, w])
    for i in range(2):
        assert torch.equal(store[i][:, :128], tape[i][:, w]) and (store[i][:, 128:] == 0).all()
    back = [torch.zeros_like(t) for t in tape]
    ops.copy_pair(back[0][:, w], store[0][:, :128], back[1][:, w], store[1][:, :128])
    for i in range(2):
        assert torch.equal(back[i][:, w], tape[i][:, w]) and (back[i][:, :64] == 0).all() and (back[i][:, 192:] == 0).all()
    # a shape the kernel refuses (row bytes not a multiple of 16) falls back to two plain copies
    a, b_ = rnd(2, 3, 5, seed=3), rnd(2, 3, 5, seed=4)
    c, d = torch.zeros_like(a), torch.zeros_like(b_)
    ops.copy_pair(c, a, d, b_)
    assert torch.equal(c, a) and torch.equal(d, b_)


@pytest.mark.parametrize("dh,pin,tau,H", [(64, 64, 0.8, 4), (128, 0, 0.0, 4), (64, 0, 50.0, 4), (64, 64, 0.8, 3),
                                          (64, 64, 150.0, 15)])
def test_mult_res_write_law_kernels(ops, dh, pin, tau, H):
    """The four pointwise kernels of the mult_res family against their fp32 torch statement; head counts
    that are not a multiple of four included (15 heads of 64: the reference's own 340M run)."""
    B, c = 2, 64
    n0 = ops.launches
    d = H * dh
    T = 128
    r = slice(32, 32 + c)
    raw, o, vc = rnd(B, c, 4 * d, seed=1), rnd(B, c, d, seed=2), rnd(B, c, d, seed=3)
    ssq = o.float().view(B, c, H, dh).pow(2).sum(-1)
    glx, k, v, vgx = rnd(B, T, 2 * d, seed=4), rnd(B, T, d, seed=5), rnd(B, T, d, seed=6), rnd(B, T, d, seed=7)
    w_ctx, k_gain = rnd(d, seed=8) * 0.1 + 1, (torch.rand(H, device=DEV) + 0.5)
    cos, sin = build_rope_cache(T, dh, 10000.0, device=DEV)
    lam = 0.7
    f = lambda t: t.float()
    vin = ops.mrk_vin_fwd(raw, ssq, o, w_ctx, vgx[:, r], lam)
    vin_r = REF.mrk_vin_fwd(f(raw), ssq, f(o), f(w_ctx), f(vgx[:, r]), lam)
    close(vin, vin_r, what="v_in")
    K1, V1 = ops.mrk_refine_fwd(raw, vc, ssq, glx[:, r], k[:, r], v[:, r], cos[r], sin[r], H, pin, k_gain, tau)
    K2, V2 = REF.mrk_refine_fwd(f(raw), f(vc), ssq, f(glx[:, r]), f(k[:, r]), f(v[:, r]), cos[r], sin[r], H, pin, k_gain, tau)
    close(K1, K2, what="K")
    close(V1, V2, what="V")
    dK, dV = rnd(B, c, H, dh, dtype=torch.float32, seed=9), rnd(B, c, H, dh, dtype=torch.float32, seed=10)
    z = lambda *s, dt=torch.float32: torch.zeros(*s, device=DEV, dtype=dt)

    def run(o_, fl, dt):
        acc = [z(B, T, d), z(B, T, d), z(B, T, 2 * d)]
        dcg, uh, dvc, dkg = z(B, c, 4 * d, dt=dt), z(B, c, d, dt=dt), z(B, c, d, dt=dt), z(B, c, H)
        o_.mrk_refine_bwd(dK, dV, fl(raw), fl(vc), ssq, fl(o), fl(glx[:, r]), fl(k[:, r]), fl(v[:, r]), cos[r], sin[r], pin,
                          k_gain, tau, acc[0][:, r], acc[1][:, r], acc[2][:, r], dcg, uh, dvc, dkg)
        dvin = fl(rnd(B, c, d, seed=11))
        dvgx = z(B, T, d)
        duh = o_.mrk_vin_bwd(dvin, fl(raw), ssq, fl(o), fl(w_ctx), fl(vgx[:, r]), lam, dcg, dvgx[:, r])
        return acc + [dcg, uh, dvc, dkg, dvgx, duh]
    got = run(ops, lambda t: t, torch.bfloat16)
    ref = run(REF, f, torch.float32)
    for a, b_, n_ in zip(got, ref, ("dk", "dv", "dglx", "dcg", "uhat", "dvc", "dkg", "dvgx", "du_hat")):
        close(a, b_, rtol=3e-2, atol=3e-2, what=n_)
    assert ops.launches - n0 >= 4, "the write-law kernels did not run (fell back to the torch statement)"
    # column dot and the norm backward with the extra term
    a_, b2 = rnd(4096, d, seed=12), rnd(4096, d, seed=13)
    out1, out2 = z(d), z(d)
    ops.col_dot_acc(out1, a_, b2)
    REF.col_dot_acc(out2, a_, b2)
    close(out1, out2, rtol=1e-2, atol=1e-1, what="col_dot")
    du, extra = rnd(B, c, d, seed=14), rnd(B, c, d, dtype=torch.float32, seed=15)
    close(ops.rmsn_bwd(du, o, ssq, extra=extra), REF.rmsn_bwd(f(du), f(o), ssq, extra=extra), what="rmsn extra")


@pytest.mark.parametrize("window", [0, 90])
def test_prefix_read_with_a_gap_between_keys_and_queries(ops, window):
    """Far read of the wavefront engine: keys end at pos0, the query chunk starts qoff rows later."""
    B, H, dh, c, pos0, qoff = 2, 4, 64, 64, 128, 64
    T = pos0 + qoff + c
    scale = dh ** -0.5
    q, ks, vr, Kc, Vc = _cell_inputs(B, c, H, dh, T)
    qc = q[:, pos0 + qoff:pos0 + qoff + c]
    f = lambda t: t.float()
    o, lse = ops.prefix_fwd(qc, Kc, Vc, pos0, scale, window, qoff=qoff)
    o_r, lse_r = fm.prefix_fwd(f(qc), f(Kc), f(Vc), pos0, scale, window, qoff)
    live = lse_r > -1e29
    close(o, o_r, what="o")
    if live.any():
        close(lse[live], lse_r[live], rtol=1e-2, atol=2e-2, what="lse")
    assert (lse[~live] < -1e29).all()
    if window:                                   # rows further than the window from every key see nothing
        assert (~live).any() and live.any()
    do, corr = rnd(B, c, H, dh, seed=3), rnd(B, c, H, dtype=torch.float32, seed=4)
    lse_use = torch.where(live, lse_r, torch.full_like(lse_r, 30.0))
    dq, dq_r = torch.zeros(B, c, H, dh, device=DEV), torch.zeros(B, c, H, dh, device=DEV)
    ops.prefix_dq(qc, Kc, Vc, pos0, scale, window, lse_use, do, corr, dq, qoff=qoff)
    fm.prefix_dq(f(qc), f(Kc), f(Vc), pos0, scale, window, lse_use, f(do), corr, dq_r, qoff)
    close(dq, dq_r, rtol=3e-2, atol=3e-2, what="dq")


def test_kernels_write_only_their_rows(ops):
    """Every output a kernel accepts as a strided view (rows of a per-layer array or of the tape) sits between
    guard rows filled with a sentinel; after the launch the guards still hold it (bounds of the row
    arithmetic, batch strides)."""
    B, c, H, dh, g = 2, 64, 4, 64, 64
    d, T, pos0 = H * dh, 3 * 64, 64
    scale = dh ** -0.5
    SENT = 7.0
    z = lambda *s, dt=torch.float32: torch.zeros(*s, dtype=dt, device=DEV)

    def guarded(*tail, dtype=torch.float32):
        big = torch.full((B, g + c + g) + tail, SENT, dtype=dtype, device=DEV)
        big[:, g:g + c] = 0
        return big, big[:, g:g + c]

    def intact(big, what):
        assert (big[:, :g] == SENT).all() and (big[:, g + c:] == SENT).all(), what

    q, ks, vr, Kc, Vc = _cell_inputs(B, c, H, dh, T)
    r = slice(pos0, pos0 + c)
    qc, ksc, vrc = q[:, r], ks[:, r], vr[:, r]
    K_in, V_in = rnd(B, c, H, dh, seed=9), rnd(B, c, H, dh, seed=10)
    n0 = ops.launches
    o_c, lse_c = ops.prefix_fwd(qc, Kc, Vc, pos0, scale, 0)
    o, lse, ssq = ops.tail_fwd(qc, ksc, vrc, K_in, V_in, o_c, lse_c, scale, 0)
    # tail backward: the raw-row accumulators are rows of per-layer arrays
    (b_ks, v_ks), (b_v, v_v) = guarded(H, dh), guarded(H, dh)
    dO = rnd(B, c, H, dh, dtype=torch.float32, seed=11)
    ops.tail_bwd(dO, qc, ksc, vrc, K_in, V_in, o_c, lse_c, o.to(torch.bfloat16), lse, scale, 0,
                 z(B, c, H, dh), v_ks, v_v, z(B, c, H, dh), z(B, c, H))
    intact(b_ks, "tail_bwd dks"), intact(b_v, "tail_bwd dv")
    assert v_ks.abs().max() > 0 and v_v.abs().max() > 0
    # refine forward into tape rows, refine backward into layer accumulators
    cos, sin = build_rope_cache(T, dh, 10000.0, device=DEV)
    raw, oo = rnd(B, c, 4 * d, scale=2.0), rnd(B, c, d, scale=1.5, seed=7)
    ssq2 = oo.float().view(B, c, H, dh).square().sum(-1)
    glx, k, v = rnd(B, c, 2 * d, seed=1), rnd(B, c, d, seed=2), rnd(B, c, d, seed=3)
    bK, vK = guarded(H, dh, dtype=torch.bfloat16)
    bV, vV = guarded(H, dh, dtype=torch.bfloat16)
    ops.refine_fwd(raw, ssq2, glx, k, v, cos[r], sin[r], H, 0, out=(vK, vV))
    intact(bK, "refine_fwd K"), intact(bV, "refine_fwd V")
    assert vK.float().abs().max() > 0
    acc = [guarded(d), guarded(d), guarded(2 * d)]
    dK, dV = rnd(B, c, H, dh, dtype=torch.float32, seed=4), rnd(B, c, H, dh, dtype=torch.float32, seed=5)
    ops.refine_bwd(dK, dV, raw, ssq2, oo, glx, k, v, cos[r], sin[r], 0, *[a[1] for a in acc],
                   z(B, c, 4 * d, dt=torch.bfloat16), z(B, c, d, dt=torch.bfloat16))
    for i, (b, _) in enumerate(acc):
        intact(b, f"refine_bwd acc {i}")
    # cell end: per-layer arrays by absolute position
    arrs = [guarded(H, dh, dtype=torch.bfloat16), guarded(H), guarded(H), guarded(H, dh), guarded(H, dh)]
    f32 = lambda *s, seed: rnd(*s, dtype=torch.float32, seed=seed)
    ops.cell_finish(f32(B, c, H, dh, seed=1), f32(B, c, H, seed=2), f32(B, c, H, dh, seed=3), f32(B, c, H, seed=4),
                    f32(B, c, H, dh, seed=5), f32(B, c, H, dh, seed=6), *[a[1] for a in arrs])
    for i, (b, _) in enumerate(arrs):
        intact(b, f"cell_finish out {i}")
    assert ops.launches - n0 >= 6, "a torch fallback ran instead of a kernel"


def test_stash_gate_sum_matches_torch_statement(ops):
    """Gradient of the gates' x-logits read back from the layer's stash of d(ctx / gate logits)."""
    B, T, c, K, d = 3, 256, 64, 4, 128
    stash = rnd((T // c) * K * B * c, 4 * d, seed=21)
    got = ops.stash_gate_sum(stash, B, T, c, K)
    ref = REF.stash_gate_sum(stash.float(), B, T, c, K)
    assert got.shape == (B, T, 2 * d) and got.dtype == torch.bfloat16
    close(got, ref, rtol=1e-2, atol=2e-2, what="gate x-logit gradient")
