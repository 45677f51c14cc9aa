"""This repository against the reference's own code (the unmodified tree under baseline/_ref; every test
here is skipped when it is not installed).

CPU, fp32: a state dict of this repository's model loaded into the reference's `DualModLM` gives the same
logits, loss and parameter gradients across the write-law variants (ctx_mod, gate type / input / rank,
norms, clamp, raw-pinned heads, sliding window), so the two models are one function of one checkpoint.

GPU, fp32: this repository's cell engine against the reference's `WaveScanEngine` (plain cells, no CUDA
graphs) on the same weights and schedule, and this repository's wavefront engine against the reference's
`make_engine(..., attn_impl="mathk", raw_diag=True)` at K < C and K = C (the reference accepts only its
mult_res / LoRA configuration family there)."""

import os
import sys

import pytest
import torch

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")
have_ref = os.path.isdir(os.path.join(REF, "models", "dualmod"))
pytestmark = pytest.mark.skipif(not have_ref, reason="baseline/_ref (the reference install) is absent")

from dual_mod_public_b200 import DualModConfig
from dual_mod_public_b200.models import DualModLM

from helpers import perturb


def _ref_modules():
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from models.dualmod.config import DualModConfig as RefConfig
    from models.dualmod.model import DualModLM as RefLM
    return RefConfig, RefLM


BASE = dict(d_model=64, n_layers=2, n_heads=4, vocab_size=97, max_seq_len=32, attn_mode="sequential",
            checkpoint_chunk=0, dtype="fp32")
VARIANTS = [
    dict(),
    dict(ctx_mod="mult"), dict(ctx_mod="mult_res", mult_res_lambda=0.9), dict(ctx_mod="fusion"), dict(ctx_mod="vmlp"),
    dict(ctx_mod="kmlp"), dict(ctx_mod="puremlp"), dict(ctx_mod="puremlp_hw"), dict(ctx_mod="linpoint"), dict(ctx_mod="glu"),
    dict(gate_type="independent"), dict(gate_type="unbounded"), dict(gate_type_v="independent"),
    dict(gate_input="u"), dict(gate_input="x"), dict(gate_rank=8, ctx_rank=8),
    dict(v_norm="rms"), dict(v_ctx_norm="rms"), dict(k_ctx_norm="rms"), dict(rmsnorm_on_o=False),
    dict(kmod_vraw_heads=1), dict(kmod_vraw_heads=1, kmod_mode="gated_norm"), dict(kmod_vraw_heads=1, kmod_vraw_bound="tanh"),
    dict(v_clamp_tau=0.5), dict(local_window=7), dict(use_rope=False), dict(attn_logn_ref=16),
    dict(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms", kmod_vraw_heads=1, v_clamp_tau=0.8),
    dict(enable_key_mod=False), dict(enable_value_mod=False), dict(attn_mode="vanilla"), dict(attn_mode="deq", deq_sweeps=3),
    dict(attn_mode="static"),
]


@pytest.mark.parametrize("kw", VARIANTS, ids=lambda kw: ",".join(f"{k}={v}" for k, v in kw.items()) or "default")
def test_one_checkpoint_one_function(kw):
    RefConfig, RefLM = _ref_modules()
    try:
        cfg = DualModConfig(**{**BASE, **kw})
    except (AssertionError, ValueError, TypeError) as e:
        pytest.skip(f"combination refused by this repository's config: {e}")
    try:
        rcfg = RefConfig(**cfg.to_dict())
    except (AssertionError, ValueError, TypeError) as e:
        pytest.skip(f"combination refused by the reference's config: {e}")
    torch.manual_seed(0)
    ours = DualModLM(cfg)
    perturb(ours)
    theirs = RefLM(rcfg)
    theirs.load_state_dict(ours.state_dict(), strict=True)
    g = torch.Generator().manual_seed(5)
    idx = torch.randint(0, cfg.vocab_size, (2, 24), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (2, 24), generator=g)
    la, loss_a = ours(idx, tgt)
    lb, loss_b = theirs(idx, tgt)
    assert (la - lb).abs().max() < 1e-5, float((la - lb).abs().max())
    assert abs(float(loss_a.detach()) - float(loss_b.detach())) < 1e-6
    loss_a.backward()
    loss_b.backward()
    ga = {n: p.grad for n, p in ours.named_parameters() if p.grad is not None}
    gb = {n: p.grad for n, p in theirs.named_parameters() if p.grad is not None}
    assert set(ga) == set(gb)
    for n in ga:
        err = float((ga[n] - gb[n]).abs().max())
        assert err < 1e-5 * max(1.0, float(gb[n].abs().max())), f"{n}: {err}"


def test_decode_matches_the_reference_decode():
    RefConfig, RefLM = _ref_modules()
    cfg = DualModConfig(**BASE)
    torch.manual_seed(0)
    ours = DualModLM(cfg).eval()
    perturb(ours)
    theirs = RefLM(RefConfig(**cfg.to_dict())).eval()
    theirs.load_state_dict(ours.state_dict())
    idx = torch.randint(0, cfg.vocab_size, (2, 12), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        ca, cb = ours.decode_init(), theirs.decode_init()
        for t in range(idx.shape[1]):
            a = ours.decode_step(idx[:, t:t + 1], t, ca)
            b = theirs.decode_step(idx[:, t:t + 1], t, cb)
            assert (a - b).abs().max() < 1e-5


# ---- engines (GPU, fp32) ---------------------------------------------------------------------------------
def _gpu_model(kw, T):
    cfg = DualModConfig(d_model=128, n_layers=2, n_heads=4, vocab_size=257, max_seq_len=T, gate_bias_init=0.0,
                        ctx_proj_init_std=0.02, **kw)
    torch.manual_seed(0)
    m = DualModLM(cfg)
    perturb(m)
    return cfg, m.cuda()


def _rel(a, b):
    a, b = a.flatten().double(), b.flatten().double()
    return float((a - b).norm() / (b.norm() + 1e-30))


@pytest.mark.gpu
@pytest.mark.parametrize("K", [2, 16])
def test_cell_engine_matches_the_reference_engine(K):
    """fp32, chunk 16: sweeps K = 2 (approximate operator) and K = 16 = c (exact); loss and every gradient group."""
    RefConfig, RefLM = _ref_modules()
    from engines.wavescan.engine.graphs import WaveScanEngine as RefEngine
    from engines.wavescan.engine.schedule import uniform_chunks as ref_chunks

    from dual_mod_public_b200.engines.schedule import uniform_chunks
    from dual_mod_public_b200.engines.wavescan import WaveScanEngine
    from dual_mod_public_b200.ops import TorchOps
    B, T, c = 2, 64, 16
    cfg, m = _gpu_model(dict(), T)
    theirs = RefLM(RefConfig(**cfg.to_dict())).cuda()
    theirs.load_state_dict(m.state_dict())
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g).cuda()
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g).cuda()
    eng = WaveScanEngine(m, [uniform_chunks(T, c, K)], B, T, autocast_bf16=False, backend="fused", ops=TorchOps())
    eng.zero_grads()
    eng.pack()
    loss = float(eng.train_step(idx, tgt))
    ref = RefEngine(theirs, [ref_chunks(T, c, K)], B, T, autocast_bf16=False, use_graphs=False, fused_sweep=False)
    ref_loss = float(ref.train_step(idx, tgt, 0))
    ref.finish_grads(world_size=1)
    assert abs(loss - ref_loss) < 1e-5, (loss, ref_loss)
    theirs_g = dict(theirs.named_parameters())
    for n, p in m.named_parameters():
        rg = theirs_g[n].grad
        if rg is None:
            continue
        assert _rel(eng.grads.get(p), rg) < 1e-4, f"{n}: {_rel(eng.grads.get(p), rg):.3g}"


@pytest.mark.gpu
@pytest.mark.parametrize("K", [2, 16])
def test_wavefront_engine_matches_the_reference_wavefront(K):
    """The wavefront operator of this repository against the reference's engine with its fp32 attention twin
    and the raw diagonal, on its own configuration family, at K < C and at K = C (logits and loss)."""
    RefConfig, RefLM = _ref_modules()
    from engines.wave3d.wave3d import make_engine as ref_make

    from dual_mod_public_b200.engines.wave3d import Wave3DEngine
    from dual_mod_public_b200.ops import TorchOps
    B, T, C = 2, 64, 16
    cfg, m = _gpu_model(dict(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms", kmod_vraw_heads=1,
                             v_clamp_tau=2.0), T)
    theirs = RefLM(RefConfig(**cfg.to_dict())).cuda()
    theirs.load_state_dict(m.state_dict())
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, cfg.vocab_size, (B, T), generator=g).cuda()
    tgt = torch.randint(0, cfg.vocab_size, (B, T), generator=g).cuda()
    eng = Wave3DEngine(m, [K], B, T, C=C, autocast_bf16=False, backend="fused", ops=TorchOps(), keep_logits=True)
    eng.pack()
    loss = float(eng.forward(idx, tgt, sid=0, train=False))
    ref = ref_make(theirs, B, T, engine="x", C=C, attn_impl="mathk", raw_diag=True, fused_refine=False, graphs=False)
    with torch.no_grad():
        ref_logits = ref.forward_logits(idx, K).float()
    ref_loss = float(torch.nn.functional.cross_entropy(ref_logits.view(-1, ref_logits.shape[-1]), tgt.view(-1)))
    err = float((eng.logits.float() - ref_logits).abs().max())
    assert err < 1e-4 and abs(loss - ref_loss) < 1e-5, (err, loss, ref_loss)
