"""Chunk-cell and engine exactness on CPU in fp32, against the sequential scan.

cell == per-position steps; a layer cut into cells == the scan; after s sweeps
the first s chunk rows are exact and K = c is exact; rows are written once with
the key rotated at write and never outside [pos0, pos0+c); engine loss and
gradients at K = c match autograd through the scan; for K < c the hand-derived
backward matches autograd through the same approximate forward."""

import pytest
import torch

from dual_mod_public_b200 import DualModConfig
from dual_mod_public_b200.engines import cell as gcell
from dual_mod_public_b200.engines.schedule import (WaveScanSchedule, exact_sequential,
                                                   uniform_chunks)
from dual_mod_public_b200.engines.wavescan import WaveScanEngine
from dual_mod_public_b200.models import DualModLM, build_rope_cache
from dual_mod_public_b200.ops import TorchOps

from helpers import perturb

TOL = 1e-5


def cfg_small(**kw):
    d = dict(d_model=64, n_layers=2, n_heads=4, vocab_size=61, max_seq_len=64, gate_bias_init=0.0,
             checkpoint_chunk=0, ctx_proj_init_std=0.02, dtype="fp32")
    d.update(kw)
    return DualModConfig(**d)


def build(**kw):
    torch.manual_seed(0)
    cfg = cfg_small(**kw)
    m = DualModLM(cfg).eval()
    perturb(m)
    return cfg, m


def inputs(cfg, B, T, seed=1):
    g = torch.Generator().manual_seed(seed)
    xhat = torch.randn(B, T, cfg.d_model, generator=g)
    cos, sin = build_rope_cache(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta)
    return xhat, cos, sin


def relerr(a, b):
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def prefix_by_scan(attn, xhat, cos, sin, a):
    B = xhat.shape[0]
    empty = xhat.new_zeros(B, attn.n_heads, 0, attn.head_dim)
    if a == 0:
        return empty, empty.clone()
    _, K, V = gcell.eager_cell(attn, xhat[:, :a], cos[:a], sin[:a], empty, empty.clone())
    return K, V


@pytest.mark.parametrize("c,a", [(1, 0), (1, 17), (8, 0), (8, 24), (16, 8)])
@pytest.mark.parametrize("window", [0, 6])
def test_cell_equals_per_position_steps(c, a, window):
    cfg, m = build(local_window=window)
    attn = m.blocks[0].attn
    xhat, cos, sin = inputs(cfg, 3, a + c)
    with torch.no_grad():
        K_comm, V_comm = prefix_by_scan(attn, xhat, cos, sin, a)
        o_ref, K_ref, V_ref = gcell.eager_cell(attn, xhat[:, a:], cos[a:a + c], sin[a:a + c], K_comm, V_comm)
        o, K_rows, V_rows = gcell.chunk_cell_forward(attn, xhat[:, a:], cos[a:a + c], sin[a:a + c],
                                                     K_comm, V_comm, n_sweeps=c)
    assert relerr(attn._split(o), o_ref) < TOL
    assert relerr(K_rows, K_ref) < TOL and relerr(V_rows, V_ref) < TOL


def _offset_schedule(T):
    return [(0, 3, 3)] + [(p + 3, c, k) for p, c, k in uniform_chunks(T - 3, 8)]


@pytest.mark.parametrize("sched", [exact_sequential, lambda T: uniform_chunks(T, 4),
                                   lambda T: uniform_chunks(T, 8), _offset_schedule])
def test_layer_in_cells_equals_scan(sched):
    cfg, m = build()
    attn = m.blocks[0].attn
    B, T = 2, 48
    xhat, cos, sin = inputs(cfg, B, T)
    Kc = torch.zeros(B, cfg.n_heads, cfg.max_seq_len, cfg.head_dim)
    Vc = torch.zeros_like(Kc)
    with torch.no_grad():
        o = gcell.layer_forward(attn, xhat, cos[:T], sin[:T], sched(T), Kc, Vc)
        o_ref, K_ref, V_ref = gcell.eager_layer(attn, xhat, cos[:T], sin[:T])
    assert relerr(o, attn._merge(o_ref)) < TOL
    assert relerr(Kc[:, :, :T], K_ref) < TOL and relerr(Vc[:, :, :T], V_ref) < TOL


@pytest.mark.parametrize("c", [4, 8, 16])
def test_sweep_frontier_and_nilpotency(c):
    cfg, m = build()
    attn = m.blocks[0].attn
    a = 12
    xhat, cos, sin = inputs(cfg, 2, a + c, seed=3)
    with torch.no_grad():
        K_comm, V_comm = prefix_by_scan(attn, xhat, cos, sin, a)
        o_ex, K_ex, V_ex = gcell.eager_cell(attn, xhat[:, a:], cos[a:a + c], sin[a:a + c], K_comm, V_comm)
        for s in range(1, c + 1):
            o_s, K_s, V_s = gcell.chunk_cell_forward(attn, xhat[:, a:], cos[a:a + c], sin[a:a + c],
                                                     K_comm, V_comm, n_sweeps=s)
            assert relerr(attn._split(o_s)[:, :, :s], o_ex[:, :, :s]) < TOL
            assert relerr(K_s[:, :, :s], K_ex[:, :, :s]) < TOL
    assert relerr(attn._split(o_s), o_ex) < TOL and relerr(V_s, V_ex) < TOL


def test_rows_written_once_inside_bounds():
    cfg, m = build()
    attn = m.blocks[0].attn
    B, T, Tmax = 2, 40, 64
    xhat, cos, sin = inputs(cfg, B, T)
    Kc = torch.full((B, cfg.n_heads, Tmax, cfg.head_dim), 7.0)
    Vc = torch.full_like(Kc, 7.0)
    snaps = []
    with torch.no_grad():
        for cell in uniform_chunks(T, 8):
            gcell.layer_forward(attn, xhat, cos, sin, [cell], Kc, Vc)
            snaps.append(Kc.clone())
    assert (Kc[:, :, T:] == 7.0).all() and (Vc[:, :, T:] == 7.0).all()
    for i, (pos0, c, _) in enumerate(uniform_chunks(T, 8)):
        assert torch.equal(snaps[i][:, :, :pos0 + c], snaps[-1][:, :, :pos0 + c])  # append-only


def _oracle_grads(model, idx, tgt):
    model.zero_grad(set_to_none=True)
    model.cfg.attn_mode = "sequential"
    model.train()
    _, loss = model(idx, targets=tgt)
    loss.backward()
    model.eval()
    return loss.detach(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


def _engine_grads(model, eng, idx, tgt, sid=0):
    eng.zero_grads()
    eng.pack()
    loss = eng.train_step(idx, tgt, sid=sid).clone()
    return loss, {n: eng.grads.get(p).clone() for n, p in model.named_parameters()}


ENGINE_VARIANTS = [
    ("fused", dict()),
    ("fused", dict(local_window=7)),
    ("fused", dict(kmod_vraw_heads=1)),
    ("fused", dict(gate_rank=8, ctx_rank=8)),
    ("generic", dict()),
    ("generic", dict(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms",
                     kmod_vraw_heads=1, v_clamp_tau=0.8)),
    # outside the packed family the kernel backend runs the write law as module code per sweep
    ("fused", dict(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms",
                   kmod_vraw_heads=1, v_clamp_tau=0.8)),
    ("fused", dict(ctx_mod="fusion", gate_type_v="independent", v_ctx_norm="rms")),
    ("fused", dict(gate_input="u", enable_key_mod=False)),
]


@pytest.mark.parametrize("backend,kw", ENGINE_VARIANTS)
def test_engine_exact_schedule_matches_scan(backend, kw):
    cfg, m = build(**kw)
    B, T = 2, 24
    g = torch.Generator().manual_seed(5)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    tgt[0, 3] = -1
    loss_ref, g_ref = _oracle_grads(m, idx, tgt)
    sched = [(0, 5, 5)] + [(p + 5, c, k) for p, c, k in uniform_chunks(T - 5, 8)]
    eng = WaveScanEngine(m, [sched], B, T, backend=backend, ops=TorchOps(), loss_rows=16)
    loss, g_eng = _engine_grads(m, eng, idx, tgt)
    assert abs(loss.item() - loss_ref.item()) < 1e-5
    for n, gr in g_ref.items():
        assert relerr(g_eng[n], gr) < 1e-4, n
    assert eng.debug_scan() == []


@pytest.mark.parametrize("kw", [dict(), dict(local_window=7), dict(kmod_vraw_heads=1)])
def test_fused_backward_matches_autograd_for_few_sweeps(kw):
    cfg, m = build(**kw)
    B, T = 2, 32
    g = torch.Generator().manual_seed(6)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    sched = uniform_chunks(T, 8, 3)
    e_f = WaveScanEngine(m, [sched], B, T, backend="fused", ops=TorchOps())
    e_g = WaveScanEngine(m, [sched], B, T, backend="generic", ops=TorchOps())
    lf, gf = _engine_grads(m, e_f, idx, tgt)
    lg, gg = _engine_grads(m, e_g, idx, tgt)
    assert abs(lf.item() - lg.item()) < 1e-5
    for n in gg:
        assert relerr(gf[n], gg[n]) < 1e-4, n


def test_write_law_families():
    from dual_mod_public_b200 import preset
    from dual_mod_public_b200.engines.wavescan import refine_family
    assert refine_family(cfg_small()) == "packed"
    assert refine_family(cfg_small(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms", kmod_vraw_heads=1,
                                   v_clamp_tau=0.8)) == "mrk"
    assert refine_family(preset("hero_1p3b")) == "mrk"
    assert refine_family(cfg_small(ctx_mod="fusion", gate_type_v="independent", v_ctx_norm="rms")) == "module"


def test_kept_sweep_states_equal_recompute():
    """Keeping every sweep's state from the forward (all layers, one layer, none) gives the same
    gradients as re-running the sweeps in the reverse scan."""
    cfg, m = build(local_window=7)
    B, T = 2, 32
    g = torch.Generator().manual_seed(8)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    sched = uniform_chunks(T, 8, 3)
    out = []
    for keep in (0, 1, "auto"):
        eng = WaveScanEngine(m, [sched], B, T, backend="fused", ops=TorchOps(), keep_sweeps=keep)
        assert eng.keep_layers == {0: 0, 1: 1, "auto": cfg.n_layers}[keep]
        out.append(_engine_grads(m, eng, idx, tgt))
        l2, g2 = _engine_grads(m, eng, idx, tgt)                 # second step reuses the slots
        assert torch.equal(l2, out[-1][0]) and all(torch.equal(g2[n], out[-1][1][n]) for n in g2)
    for l, gr in out[1:]:
        assert torch.equal(l, out[0][0])
        for n in gr:
            assert torch.equal(gr[n], out[0][1][n]), n


def test_saturating_carry_and_rho_signal():
    """A loose cap changes nothing and fills the governor's signal; a tight cap bounds the gradient that
    later cells hand to earlier rows (finite, smaller, different)."""
    cfg, m = build()
    B, T = 2, 32
    g = torch.Generator().manual_seed(9)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    sched = uniform_chunks(T, 8, 3)
    base = WaveScanEngine(m, [sched], B, T, backend="fused", ops=TorchOps())
    l0, g0 = _engine_grads(m, base, idx, tgt)
    assert base.chain_rho_max.item() == 0.0
    loose = WaveScanEngine(m, [sched], B, T, backend="fused", ops=TorchOps(), sat_tau=1e6)
    l1, g1 = _engine_grads(m, loose, idx, tgt)
    assert loose.chain_rho_max.item() > 0 and all(torch.allclose(g1[n], g0[n], rtol=1e-5, atol=1e-8) for n in g0)
    tight = WaveScanEngine(m, [sched], B, T, backend="fused", ops=TorchOps(), sat_tau=1e-3)
    l2, g2 = _engine_grads(m, tight, idx, tgt)
    n = "blocks.0.attn.wk.weight"
    assert torch.isfinite(g2[n]).all() and not torch.allclose(g2[n], g0[n], rtol=1e-3, atol=1e-9)
    assert torch.equal(l0, l2)


def test_explicit_dlogits_backward_and_accumulation():
    cfg, m = build()
    B, T = 2, 16
    g = torch.Generator().manual_seed(7)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    sched = uniform_chunks(T, 8)
    for backend in ("fused", "generic"):
        eng = WaveScanEngine(m, [sched], B, T, backend=backend, ops=TorchOps(), keep_logits=True)
        l1, g1 = _engine_grads(m, eng, idx, tgt)
        eng.zero_grads()
        eng.forward(idx)
        logits = eng.logits.clone().requires_grad_(True)
        loss = torch.nn.functional.cross_entropy(logits.view(-1, cfg.vocab_size), tgt.view(-1))
        (dl,) = torch.autograd.grad(loss, logits)
        eng.backward(d_logits=dl)
        for n, p in m.named_parameters():
            assert relerr(eng.grads.get(p), g1[n]) < 1e-4, (backend, n)
        eng.forward(idx)
        eng.backward(d_logits=dl)                      # second micro-batch accumulates
        n0, p0 = next(iter(m.named_parameters()))
        assert relerr(eng.grads.get(p0), 2 * g1[n0]) < 1e-4


def test_schedule_pool_covers_sequence():
    pool = WaveScanSchedule(seed=3).draw_pool(100)
    assert len(pool) == 8
    for sched in pool:
        assert sum(c for _, c, _ in sched) == 100
        assert all(1 <= k <= c for _, c, k in sched)


@pytest.mark.parametrize("kw", [dict(gate_rank=8, ctx_rank=8),
                                dict(ctx_mod="mult_res", gate_rank=8, ctx_rank=16, k_ctx_norm="rms", kmod_vraw_heads=1,
                                     v_clamp_tau=0.8)])
def test_factored_write_law_equals_composed_matrices(kw, monkeypatch):
    """With every operator of the write law factored, the sweeps apply the factors (down GEMM onto the
    stacked ranks, one narrow up GEMM per operator) and accumulate the factors' gradients directly; the
    result equals the path through the composed d x d matrices and autograd through the same forward."""
    cfg, m = build(**kw)
    B, T = 2, 32
    g = torch.Generator().manual_seed(6)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    sched = uniform_chunks(T, 8, 3)
    e_f = WaveScanEngine(m, [sched], B, T, backend="fused", ops=TorchOps())
    assert e_f.factored and e_f.packs[0].W_pack is None
    lf, gf = _engine_grads(m, e_f, idx, tgt)
    monkeypatch.setenv("DMB_DENSE_WRITE_LAW", "1")
    e_d = WaveScanEngine(m, [sched], B, T, backend="fused", ops=TorchOps())
    assert not e_d.factored and e_d.packs[0].W_pack is not None
    ld, gd = _engine_grads(m, e_d, idx, tgt)
    e_g = WaveScanEngine(m, [sched], B, T, backend="generic", ops=TorchOps())
    lg, gg = _engine_grads(m, e_g, idx, tgt)
    assert abs(lf.item() - ld.item()) < 1e-5 and abs(lf.item() - lg.item()) < 1e-5
    for n in gg:
        assert relerr(gf[n], gd[n]) < 1e-4, n
        assert relerr(gf[n], gg[n]) < 1e-4, n


def test_odd_head_count_of_the_d960_recipe():
    """15 heads at d = 960 in the reference's 340M run: a head count that is not a multiple of 4, with factored
    mult_res operators.  Scaled down (3 heads of 32), fused statement against autograd."""
    from dual_mod_public_b200 import preset
    from dual_mod_public_b200.engines.wavescan import refine_family
    full = preset("dm_d960")
    assert full.n_heads == 15 and full.head_dim == 64 and refine_family(full) == "mrk"
    cfg, m = build(d_model=96, n_heads=3, ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms", kmod_vraw_heads=1,
                   v_clamp_tau=2.0)
    B, T = 2, 24
    g = torch.Generator().manual_seed(9)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g)
    sched = uniform_chunks(T, 8, 3)
    e_f = WaveScanEngine(m, [sched], B, T, backend="fused", ops=TorchOps())
    e_g = WaveScanEngine(m, [sched], B, T, backend="generic", ops=TorchOps())
    lf, gf = _engine_grads(m, e_f, idx, tgt)
    lg, gg = _engine_grads(m, e_g, idx, tgt)
    assert e_f.factored and abs(lf.item() - lg.item()) < 1e-5
    for n in gg:
        assert relerr(gf[n], gg[n]) < 1e-4, n
