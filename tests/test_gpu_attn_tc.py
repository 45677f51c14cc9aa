"""tcgen05 attention forward (ops/csrc/attn_tc.cu) against a plain fp32 statement of the same read:
whole-prefix reads of chunk groups (M = 64 tiles), lower-right causal reads of long query blocks
(M = 128 tiles), sliding windows, ragged row / key counts, head dims 64 and 128, and agreement with the
warp-MMA `prefix_fwd` kernel it replaces."""

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from dual_mod_public_b200.ops.cuda_ops import CudaOps
    o = CudaOps(torch.device(DEV))
    o.ATTN_TC = True                 # the ops below go through the tcgen05 kernels whatever the process default is
    return o


def rnd(*s, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed + sum(s))
    return (torch.randn(*s, generator=g) * scale).to(DEV).bfloat16()


def reference(q, K, V, lo, hi, qbase, scale, window, causal, causal_excl, Lq, G, grow):
    """fp32: (o [B,G,Lq,h,dh], lse [B,G,Lq,h]); rows without any allowed key: o = 0, lse = -1e30."""
    B, _, h, dh = q.shape
    o = torch.zeros(B, G, Lq, h, dh, device=q.device)
    lse = torch.full((B, G, Lq, h), -1e30, device=q.device)
    for z in range(G):
        lo_z, hi_z = max(0, lo + z * grow), hi + z * grow
        qz = q[:, z * grow:z * grow + Lq].float()
        if hi_z <= lo_z:
            continue
        Kz, Vz = K[:, lo_z:hi_z].float(), V[:, lo_z:hi_z].float()
        s = torch.einsum("bihd,bjhd->bhij", qz, Kz) * scale
        pos = (qbase + z * grow + torch.arange(Lq, device=q.device))[:, None]
        j = torch.arange(lo_z, hi_z, device=q.device)[None, :]
        ok = torch.ones(Lq, hi_z - lo_z, dtype=torch.bool, device=q.device)
        if causal:
            ok &= j <= pos - causal_excl
        if window:
            ok &= j > pos - window
        s = s.masked_fill(~ok, float("-inf"))
        l = torch.logsumexp(s, dim=-1)                                  # [B,h,Lq]
        p = torch.exp(s - l.masked_fill(l == float("-inf"), 0.0)[..., None])
        p = p.masked_fill(~ok, 0.0)
        o[:, z] = torch.einsum("bhij,bjhd->bihd", p, Vz)
        lse[:, z] = torch.where(l == float("-inf"), torch.full_like(l, -1e30), l).permute(0, 2, 1)
    return o, lse


def check(got, ref, what, tol=2e-2):
    o, lse = got
    o_ref, lse_ref = ref
    live = lse_ref > -1e29
    assert torch.equal(lse > -1e29, live), f"{what}: empty rows differ"
    e_o = (o.float() - o_ref).abs().max().item()
    e_l = (lse - lse_ref)[live].abs().max().item() if live.any() else 0.0
    assert e_o < tol and e_l < tol, f"{what}: |do| {e_o:.4g} |dlse| {e_l:.4g}"


CASES = [
    # B, T, h, dh, Lq, G, grow, lo, hi, qbase, window, causal, excl, bm
    (2, 1024, 4, 64, 64, 1, 0, 0, 640, 640, 0, False, 1, 64),          # a cell's whole-prefix read
    (2, 1024, 4, 64, 64, 3, 64, 0, 200, 200, 0, False, 1, 64),         # three chunk groups, ragged key count
    (2, 1024, 2, 64, 64, 2, 64, 0, 448, 448, 300, False, 1, 64),       # sliding window over the prefix
    (1, 1024, 2, 64, 256, 1, 0, 0, 1024, 768, 0, True, 0, 128),        # lower-right causal, diagonal included
    (2, 768, 2, 64, 200, 1, 0, 0, 700, 500, 0, True, 1, 128),          # ragged rows and keys, strictly causal
    (1, 1024, 2, 64, 256, 1, 0, 0, 1024, 768, 333, True, 0, 128),      # causal + window
    (2, 512, 2, 128, 64, 2, 64, 0, 256, 256, 0, False, 1, 64),         # head dim 128, cells
    (1, 1024, 2, 128, 256, 1, 0, 0, 1024, 768, 0, True, 0, 128),       # head dim 128, long block
    (1, 512, 2, 64, 64, 1, 0, 100, 100, 100, 0, False, 1, 64),         # empty key range
]


@pytest.mark.parametrize("case", CASES)
def test_attn_fwd_tc_matches_fp32(ops, case):
    B, T, h, dh, Lq, G, grow, lo, hi, qbase, window, causal, excl, bm = case
    rows = (G - 1) * grow + Lq
    q = rnd(B, rows, h, dh, seed=1)
    K, V = rnd(B, T, h, dh, seed=2), rnd(B, T, h, dh, seed=3)
    scale = dh ** -0.5
    got = ops.attn_fwd_tc(q, K, V, lo, hi, qbase, scale, window, causal, excl, Lq=Lq, G=G, grow=grow, bm=bm)
    ops.tc_check()
    ref = reference(q, K, V, lo, hi, qbase, scale, window, causal, excl, Lq, G, grow)
    check(got, ref, f"case {case}")
    got16 = ops.attn_fwd_tc(q, K, V, lo, hi, qbase, scale, window, causal, excl, Lq=Lq, G=G, grow=grow, bm=bm,
                            out_dtype=torch.bfloat16)
    check(got16, ref, f"case {case} (bf16 out)", tol=3e-2)


def test_strided_query_view_and_agreement_with_prefix_fwd(ops):
    """q is a chunk slice of a full-sequence tensor (row offset, batch stride of the parent), as the engines
    pass it; the result equals the warp-MMA prefix kernel's."""
    B, T, h, dh, c, pos0 = 4, 512, 4, 64, 64, 320
    q_all = rnd(B, T, h, dh, seed=5)
    K, V = rnd(B, T, h, dh, seed=6), rnd(B, T, h, dh, seed=7)
    scale = dh ** -0.5
    qv = q_all[:, pos0:pos0 + c]
    o_tc, lse_tc = ops.attn_fwd_tc(qv, K, V, 0, pos0, pos0, scale, Lq=c, bm=64)
    ops.tc_check()
    was, ops.ATTN_TC = ops.ATTN_TC, False                  # the warp-MMA kernel behind the same op
    try:
        o_mma, lse_mma = ops.prefix_fwd(qv, K, V, pos0, scale)
    finally:
        ops.ATTN_TC = was
    assert (o_tc[:, 0] - o_mma).abs().max() < 2e-2 and (lse_tc[:, 0] - lse_mma).abs().max() < 2e-2


def _cells(ops, B, T, h, dh, window, seed):
    """Per-cell whole-prefix reads of a random tape and random upstream gradients, laid out by absolute
    position as the engines keep them: q, d o_c (bf16), lse_c, corr (fp32)."""
    from dual_mod_public_b200.ops.torch_ops import TorchOps
    ref = TorchOps()
    c, scale = 64, dh ** -0.5
    q_all, K, V = rnd(B, T, h, dh, seed=seed), rnd(B, T, h, dh, seed=seed + 1), rnd(B, T, h, dh, seed=seed + 2)
    doc_all = rnd(B, T, h, dh, seed=seed + 3, scale=0.1)
    lse_all = torch.zeros(B, T, h, device=DEV)
    corr_all = torch.zeros(B, T, h, device=DEV)
    for pos0 in range(c, T, c):
        r = slice(pos0, pos0 + c)
        o_c, lse_c = ref.prefix_fwd(q_all[:, r], K, V, pos0, scale, window)
        dlse = rnd(B, c, h, seed=seed + pos0, scale=0.1).float()
        lse_all[:, r] = lse_c
        corr_all[:, r] = (doc_all[:, r].float() * o_c).sum(-1) - dlse
    return ref, q_all, K, V, doc_all, lse_all, corr_all, scale


def _close(got, ref, what, tol=2e-2):
    err = (got.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item()
    assert err <= tol * scale + 1e-4, f"{what}: err {err:.4g} scale {scale:.4g}"


@pytest.fixture(params=[True, False], ids=["readers128", "readers64"])
def reader_tiles(request, ops):
    """Both forms of the backward kernels at head dim 64: the streamed side in tiles of 128 rows (default) and of 64."""
    was = ops.dkv_rows128(request.param)
    yield request.param
    ops.dkv_rows128(was)


@pytest.mark.parametrize("dh,window", [(64, 0), (64, 150), (128, 0)])
def test_backward_query_side_matches_torch_statement(ops, dh, window, reader_tiles):
    B, T, h, c = 2, 512, 2, 64
    ref, q_all, K, V, doc_all, lse_all, corr_all, scale = _cells(ops, B, T, h, dh, window, 11)
    for pos0 in (64, 320, 448):
        r = slice(pos0, pos0 + c)
        lse_c, corr = lse_all[:, r].contiguous(), corr_all[:, r].contiguous()
        dq_ref = torch.ones(B, c, h, dh, device=DEV)
        ref.prefix_dq(q_all[:, r], K, V, pos0, scale, window, lse_c, doc_all[:, r], corr, dq_ref)
        dq = torch.ones(B, c, h, dh, device=DEV)
        ops.prefix_dq(q_all[:, r], K, V, pos0, scale, window, lse_c, doc_all[:, r], corr, dq)
        ops.tc_check()
        _close(dq, dq_ref, f"dq at pos0 {pos0}")


@pytest.mark.parametrize("dh,window", [(64, 0), (64, 150), (128, 0)])
def test_backward_key_side_matches_torch_statement(ops, dh, window, reader_tiles):
    B, T, h, c = 2, 512, 2, 64
    ref, q_all, K, V, doc_all, lse_all, corr_all, scale = _cells(ops, B, T, h, dh, window, 21)
    for pos0 in (0, 192, 384):
        dK_ref, dV_ref = ref.prefix_dkv(q_all, doc_all, corr_all, lse_all, K, V, pos0, c, pos0 + c, scale, window)
        dK, dV = ops.prefix_dkv(q_all, doc_all, corr_all, lse_all, K, V, pos0, c, pos0 + c, scale, window)
        ops.tc_check()
        _close(dK, dK_ref, f"dK of chunk at {pos0}")
        _close(dV, dV_ref, f"dV of chunk at {pos0}")
    # a bounded reader range, as the wavefront engine's near reads use it
    dK_ref, dV_ref = ref.prefix_dkv(q_all, doc_all, corr_all, lse_all, K, V, 128, c, 256, scale, window, q_end=400)
    dK, dV = ops.prefix_dkv(q_all, doc_all, corr_all, lse_all, K, V, 128, c, 256, scale, window, q_end=400)
    _close(dK, dK_ref, "dK, bounded readers")
    _close(dV, dV_ref, "dV, bounded readers")


@pytest.mark.parametrize("G,lo_c,K_sw,window", [(2, 4, 3, 0), (4, 5, 8, 0), (8, 8, 8, 0), (4, 6, 4, 150), (6, 3, 8, 0), (2, 0, 3, 0)])
def test_near_read_with_two_chunks_per_tile(ops, G, lo_c, K_sw, window):
    """An even number of window chunks: the near read pairs them into 128-row tiles (the union of the two key
    ranges streams through, each half masks to its own); against the per-chunk statement and the unpaired launch."""
    from dual_mod_public_b200.ops.torch_ops import TorchOps
    ref = TorchOps()
    B, h, dh, C = 2, 3, 64, 64
    T = (lo_c + G) * C
    q_all, K, V = rnd(B, T, h, dh, seed=41), rnd(B, T, h, dh, seed=42), rnd(B, T, h, dh, seed=43)
    scale = dh ** -0.5
    w = slice(lo_c * C, (lo_c + G) * C)
    args = (q_all[:, w], K, V, lo_c * C, (lo_c - K_sw + 1) * C, C, scale, window)
    o_ref, lse_ref = ref.win_near_fwd(*args)
    o1, lse1 = ops.win_near_fwd(*args)
    ops.NEAR_PAIRS = True
    try:
        o, lse = ops.win_near_fwd(*args)
    finally:
        ops.NEAR_PAIRS = type(ops).NEAR_PAIRS
    ops.tc_check()
    _close(o, o_ref, "near o (pairs)")
    live = lse_ref > -1e29
    _close(lse[live], lse_ref[live], "near lse (pairs)")
    assert (lse[~live] < -1e29).all()
    _close(o, o1, "pairs vs single chunks", tol=1e-2)


@pytest.mark.parametrize("G,lo_c,K_sw,keep_near", [(4, 5, 8, True), (3, 4, 3, True), (8, 8, 8, False), (2, 0, 3, True)])
def test_near_read_merged_with_far_partials_in_the_epilogue(ops, G, lo_c, K_sw, keep_near):
    """`win_near_merged` (the read kernel's epilogue merges with stored far partials) against the near read followed
    by the merge statement; even group counts run as pairs, odd ones as single chunks."""
    from dual_mod_public_b200.ops.torch_ops import TorchOps
    ref = TorchOps()
    B, h, dh, C = 2, 3, 64, 64
    T = (lo_c + G + 1) * C
    q_all, K, V = rnd(B, T, h, dh, seed=51), rnd(B, T, h, dh, seed=52), rnd(B, T, h, dh, seed=53)
    ofar = rnd(B, T, h, dh, seed=54).float()
    lsefar = rnd(B, T, h, seed=55).float() + 2.0
    lsefar[:, :C] = -1e30                                    # chunks without a far prefix carry an empty partial
    scale = dh ** -0.5
    w = slice(lo_c * C, (lo_c + G) * C)
    args = (q_all[:, w], K, V, lo_c * C, (lo_c - K_sw + 1) * C, C, scale, 0, ofar[:, w], lsefar[:, w])
    want = ref.win_near_merged(*args, keep_near=keep_near)
    ops.NEAR_PAIRS = G % 2 == 0
    try:
        got = ops.win_near_merged(*args, keep_near=keep_near)
    finally:
        ops.NEAR_PAIRS = type(ops).NEAR_PAIRS
    ops.tc_check()
    assert not ops.fallbacks.get("win_near_merged")
    names = ("o_c", "lse_c", "w_f", "w_n", "o_n", "lse_n")
    for a, b_, n_ in zip(got, want, names):
        if b_ is None:
            assert a is None, n_
            continue
        if n_.startswith("lse"):
            live = b_ > -1e29
            _close(a[live], b_[live], n_)
            assert (a[~live] < -1e29).all(), n_
        else:
            _close(a, b_, n_)


def test_window_group_launches_match_the_per_chunk_statement(ops, reader_tiles):
    """The wavefront engine's one-launch-per-window forms (grid z = chunk of the window)."""
    from dual_mod_public_b200.ops.torch_ops import TorchOps
    ref = TorchOps()
    B, T, h, dh, C, G = 2, 640, 2, 64, 64, 3
    q_all, K, V = rnd(B, T, h, dh, seed=31), rnd(B, T, h, dh, seed=32), rnd(B, T, h, dh, seed=33)
    scale, lo_c, K_sw = dh ** -0.5, 4, 3
    w = slice(lo_c * C, (lo_c + G) * C)
    o_ref, lse_ref = ref.win_near_fwd(q_all[:, w], K, V, lo_c * C, (lo_c - K_sw + 1) * C, C, scale)
    o, lse = ops.win_near_fwd(q_all[:, w], K, V, lo_c * C, (lo_c - K_sw + 1) * C, C, scale)
    ops.tc_check()
    _close(o, o_ref, "near o")
    _close(lse, lse_ref, "near lse")
    do_n = rnd(B, G * C, h, dh, seed=34, scale=0.1)
    corr = ((do_n.float() * o_ref).sum(-1) - rnd(B, G * C, h, seed=35, scale=0.1).float()).contiguous()
    dq_ref, dq = torch.zeros(B, G * C, h, dh, device=DEV), torch.zeros(B, G * C, h, dh, device=DEV)
    ref.win_near_dq(q_all[:, w], K, V, lo_c * C, (lo_c - K_sw + 1) * C, C, scale, lse_ref, do_n, corr, dq_ref)
    ops.win_near_dq(q_all[:, w], K, V, lo_c * C, (lo_c - K_sw + 1) * C, C, scale, lse_ref.contiguous(), do_n, corr, dq)
    ops.tc_check()
    _close(dq, dq_ref, "near dq")
    doc_all, lse_all, corr_all = torch.zeros_like(q_all), torch.zeros(B, T, h, device=DEV), torch.zeros(B, T, h, device=DEV)
    doc_all[:, w], lse_all[:, w], corr_all[:, w] = do_n, lse_ref, corr
    j0, Gk = lo_c - K_sw + 1, G + K_sw - 2
    dK_ref, dV_ref = ref.win_near_dkv(q_all, doc_all, corr_all, lse_all, K, V, j0, Gk, C, lo_c * C, (lo_c + G) * C, K_sw * C, scale)
    dK, dV = ops.win_near_dkv(q_all, doc_all, corr_all, lse_all, K, V, j0, Gk, C, lo_c * C, (lo_c + G) * C, K_sw * C, scale)
    ops.tc_check()
    _close(dK, dK_ref, "near dK")
    _close(dV, dV_ref, "near dV")


def test_backward_outputs_into_windows_of_longer_arrays(ops, reader_tiles):
    """The engines hand the backward kernels windows of [B, T, h, dh] gradient arrays: dq added in place, the
    key side added to the pending gradient of its rows."""
    B, T, h, dh, c = 2, 512, 2, 64, 64
    ref, q_all, K, V, doc_all, lse_all, corr_all, scale = _cells(ops, B, T, h, dh, 0, 41)
    pos0 = 256
    r = slice(pos0, pos0 + c)
    dq_ref = torch.full((B, T, h, dh), 0.5, device=DEV)
    dq = dq_ref.clone()
    lse_c, corr = lse_all[:, r].contiguous(), corr_all[:, r].contiguous()
    ref.prefix_dq(q_all[:, r], K, V, pos0, scale, 0, lse_c, doc_all[:, r], corr, dq_ref[:, r])
    ops.prefix_dq(q_all[:, r], K, V, pos0, scale, 0, lse_c, doc_all[:, r], corr, dq[:, r])
    _close(dq, dq_ref, "dq into a window")
    pend_ref = (torch.full((B, T, h, dh), 0.25, device=DEV), torch.full((B, T, h, dh), -0.25, device=DEV))
    pend = (pend_ref[0].clone(), pend_ref[1].clone())
    ref.prefix_dkv(q_all, doc_all, corr_all, lse_all, K, V, pos0, c, pos0 + c, scale, 0,
                   out=(pend_ref[0][:, r], pend_ref[1][:, r]), accumulate=True)
    ops.prefix_dkv(q_all, doc_all, corr_all, lse_all, K, V, pos0, c, pos0 + c, scale, 0,
                   out=(pend[0][:, r], pend[1][:, r]), accumulate=True)
    ops.tc_check()
    _close(pend[0], pend_ref[0], "dK added to a window")
    _close(pend[1], pend_ref[1], "dV added to a window")
    # the same through the warp-MMA kernels
    was, ops.ATTN_TC = ops.ATTN_TC, False
    try:
        pend2 = (torch.full((B, T, h, dh), 0.25, device=DEV), torch.full((B, T, h, dh), -0.25, device=DEV))
        ops.prefix_dkv(q_all, doc_all, corr_all, lse_all, K, V, pos0, c, pos0 + c, scale, 0,
                       out=(pend2[0][:, r], pend2[1][:, r]), accumulate=True)
        dq2 = torch.full((B, T, h, dh), 0.5, device=DEV)
        ops.prefix_dq(q_all[:, r], K, V, pos0, scale, 0, lse_c, doc_all[:, r], corr, dq2[:, r])
    finally:
        ops.ATTN_TC = was
    _close(pend2[0], pend_ref[0], "dK added to a window (warp MMA)")
    _close(dq2, dq_ref, "dq into a window (warp MMA)")
