"""Wavefront engine on CPU (fp32): the fused path (hand-derived backward with far/near split, version
roll-back and pending tape gradients) against autograd through the plain-torch operator, and the
operator against the exact sequential scan once the sweeps cover the dependency depth."""

import pytest
import torch

from dual_mod_public_b200.engines.wave3d import Wave3DEngine, wavefront_model_forward
from dual_mod_public_b200.ops.torch_ops import TorchOps
from test_engine_cpu import build, relerr


def _data(cfg, B, T, seed):
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, cfg.vocab_size, (B, T), generator=g),
            torch.randint(0, cfg.vocab_size, (B, T), generator=g))


def _autograd(model, idx, tgt, C, K):
    model.zero_grad(set_to_none=True)
    logits = wavefront_model_forward(model, idx, C, K)
    loss = torch.nn.functional.cross_entropy(logits.float().view(-1, logits.shape[-1]), tgt.view(-1))
    loss.backward()
    return loss.detach(), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}


def _engine(model, eng, idx, tgt, sid=0):
    eng.zero_grads()
    eng.pack()
    loss = eng.train_step(idx, tgt, sid=sid).clone()
    return loss, {n: eng.grads.get(p).clone() for n, p in model.named_parameters()}


@pytest.mark.parametrize("K,C,T", [(1, 4, 16), (2, 4, 24), (3, 4, 32), (4, 8, 32), (6, 4, 16)])
@pytest.mark.parametrize("kw", [dict(), dict(kmod_vraw_heads=1), dict(local_window=7), dict(local_window=13, kmod_vraw_heads=1),
                                dict(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms", kmod_vraw_heads=1,
                                     v_clamp_tau=0.8)])
def test_fused_wavefront_matches_autograd(K, C, T, kw):
    cfg, m = build(**kw)
    idx, tgt = _data(cfg, 2, T, 3)
    l_ref, g_ref = _autograd(m, idx, tgt, C, K)
    eng = Wave3DEngine(m, [K], 2, T, C=C, backend="fused", ops=TorchOps(), loss_rows=16)
    l, g = _engine(m, eng, idx, tgt)
    assert abs(l.item() - l_ref.item()) < 1e-5
    for n, gr in g_ref.items():
        assert relerr(g[n], gr) < 1e-4, n
    l2, g2 = _engine(m, eng, idx, tgt)                              # buffers are reusable
    assert torch.equal(l, l2) and all(torch.equal(g[n], g2[n]) for n in g)


def test_kept_far_partials_change_nothing():
    """The backward's forward re-run reuses the far partials the training forward left per layer (`keep_far`) or
    computes them again: bitwise the same loss and gradients; an evaluation forward in between invalidates them."""
    cfg, m = build(n_layers=2)
    idx, tgt = _data(cfg, 2, 32, 5)
    mk = lambda keep: Wave3DEngine(m, [3], 2, 32, C=4, backend="fused", ops=TorchOps(), loss_rows=16, keep_far=keep)
    e1, e0 = mk(True), mk(False)
    assert e1.keep_far and not e0.keep_far and len(e1._far) == 2 and len(e0._far) == 1
    (l1, g1), (l0, g0) = _engine(m, e1, idx, tgt), _engine(m, e0, idx, tgt)
    assert torch.equal(l1, l0) and all(torch.equal(g1[n], g0[n]) for n in g0)
    calls = []
    orig = e1.ops.prefix_fwd
    e1.ops.prefix_fwd = lambda *a, **k: (calls.append(1), orig(*a, **k))[1]
    e1.zero_grads()
    e1.train_step(idx, tgt)
    n_train = len(calls)                       # forward only: the re-run inside the backward adds none
    e1.forward(idx, tgt, train=True)
    assert len(calls) == 2 * n_train
    e1.forward(idx, tgt)                       # an evaluation forward: the kept partials are no longer the training ones
    e1.backward()
    assert len(calls) == 4 * n_train           # eval forward + far reads of the re-run
    del e1.ops.prefix_fwd


def test_windowed_wavefront_reaches_the_windowed_scan():
    """With a sliding window the operator still converges to the exact scan of the windowed model."""
    cfg, m = build(local_window=6)
    T, C = 16, 4
    idx, tgt = _data(cfg, 2, T, 6)
    m.cfg.attn_mode = "sequential"
    with torch.no_grad():
        ref, _ = m(idx)
        got = wavefront_model_forward(m, idx, C, 13)
    assert (got - ref).abs().max().item() < 1e-5


def test_generic_backend_and_ladder():
    cfg, m = build(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms", kmod_vraw_heads=1, v_clamp_tau=0.8)
    T, C = 16, 4
    idx, tgt = _data(cfg, 2, T, 4)
    eng = Wave3DEngine(m, [1, 2], 2, T, C=C, backend="generic", ops=TorchOps())
    for sid, K in enumerate([1, 2]):
        l_ref, g_ref = _autograd(m, idx, tgt, C, K)
        l, g = _engine(m, eng, idx, tgt, sid=sid)
        assert abs(l.item() - l_ref.item()) < 1e-5
        for n, gr in g_ref.items():
            assert relerr(g[n], gr) < 1e-4, (K, n)


def test_wavefront_reaches_the_exact_scan():
    """Position p is exact once p + 1 steps have run, and chunk i is swept at steps i .. i+K-1, so
    K >= T - T/C + 1 sweeps reproduce the sequential scan; fewer sweeps are an approximation (K = C is
    NOT exact for this operator, unlike the cell engine, because a chunk starts while its predecessors
    are still moving)."""
    cfg, m = build()
    T, C = 16, 4
    idx, tgt = _data(cfg, 2, T, 5)
    m.cfg.attn_mode = "sequential"
    with torch.no_grad():
        ref, _ = m(idx)
        errs = []
        for K in (1, 2, 4, 13):
            errs.append((wavefront_model_forward(m, idx, C, K) - ref).abs().max().item())
    assert errs[-1] < 1e-5, errs
    assert errs[2] < 0.5 * errs[0] and errs[2] > 1e-4, errs


def test_make_engine_surface_of_the_reference():
    """`make_engine(model, B, T, engine="x", **kw)` with the reference's keyword arguments, then its calls:
    forward at a sweep count K (one outside the ladder becomes a new rung), `forward_logits`, `mem`, stats."""
    from dual_mod_public_b200.engines.wave3d import make_engine
    cfg, m = build()
    idx, tgt = _data(cfg, 2, 16, 5)
    eng = make_engine(m, 2, 16, engine="x", C=4, ladder=(2, 3), graphs=True, attn_impl="cudnn_fe", stash_attn=True,
                      fused_refine=True, raw_diag=True, keep_logits=True, ops=TorchOps())
    eng.pack()
    assert eng.ladder == [2, 3] and eng.set_compile("all") is eng
    loss3 = eng.forward_K(idx, tgt, 3).clone()
    ref = wavefront_model_forward(m, idx, 4, 3)
    ref_loss = torch.nn.functional.cross_entropy(ref.float().view(-1, ref.shape[-1]), tgt.view(-1))
    assert abs(float(loss3) - float(ref_loss.detach())) < 1e-5
    logits5 = eng.forward_logits(idx, 5)                      # K = 5 is not on the ladder
    assert eng.ladder == [2, 3, 5]
    assert relerr(logits5, wavefront_model_forward(m, idx, 4, 5)) < 1e-5
    assert eng.wave_stats(3) == {"steps": 6, "max_active": 3, "rows_per_step": 24, "layers": cfg.n_layers, "chunks": 4}
    assert isinstance(eng.mem, dict)
