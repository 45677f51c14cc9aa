"""Model-level exactness (fp32, tol 1e-5): the scan equals a vanilla Transformer
when modulation is off or the gates are closed, decode equals teacher forcing,
K parallel sweeps are exact on the first K positions, the model is causal, and
span re-materialisation does not change gradients."""

import pytest
import torch

from helpers import make_model, perturb, rand_idx, small_cfg

DEVICES = ["cpu"]
TOL = 1e-5


def _logits(model, idx, mode):
    model.cfg.attn_mode = mode
    with torch.no_grad():
        return model(idx)[0]


@pytest.mark.parametrize("B,T,chunk", [(2, 16, 0), (3, 32, 0), (2, 31, 5), (1, 8, 3)])
def test_scan_equals_vanilla_without_modulation(B, T, chunk):
    cfg = small_cfg(enable_key_mod=False, enable_value_mod=False, checkpoint_chunk=chunk)
    model = make_model(cfg)
    idx = rand_idx(cfg, B, T)
    assert (_logits(model, idx, "sequential") - _logits(model, idx, "vanilla")).abs().max() < TOL


def test_gates_closed_equals_vanilla():
    cfg = small_cfg()
    model = make_model(cfg)
    with torch.no_grad():
        for blk in model.blocks:
            for gate, ctx in (("w_gk", "w_kctx"), ("w_gv", "w_vctx")):
                getattr(blk.attn, gate).bias.fill_(20.0)
                getattr(blk.attn, gate).weight.zero_()
                getattr(blk.attn, ctx).weight.normal_(0, 0.5)
    idx = rand_idx(cfg, 2, 24)
    assert (_logits(model, idx, "sequential") - _logits(model, idx, "vanilla")).abs().max() < TOL


VARIANTS = [
    dict(),
    dict(enable_key_mod=False),
    dict(enable_value_mod=False),
    dict(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms", kmod_vraw_heads=1,
         v_clamp_tau=0.8),
    dict(ctx_mod="mult", mult_res_lambda=0.97),
    dict(ctx_mod="fusion", v_norm="rms", v_ctx_norm="rms"),
    dict(ctx_mod="vmlp", gate_type_v="independent"),
    dict(ctx_mod="kmlp", gate_input="u"),
    dict(ctx_mod="puremlp", gate_input="x"),
    dict(ctx_mod="linpoint", gate_type="independent"),
    dict(ctx_mod="glu", gate_type="unbounded"),
    dict(kmod_vraw_heads=2, kmod_mode="gated_norm", v_norm="rms"),
    dict(kmod_vraw_heads=1, kmod_vraw_bound="tanh"),
    dict(local_window=5),
    dict(attn_logn_ref=8),
    dict(use_rope=False),
    dict(gate_bias_init_k="ugi", gate_bias_init_v="band"),
    dict(gate_bias_init_k="committed", key_frontier_pairs=2),
]


@pytest.mark.parametrize("kw", VARIANTS, ids=lambda k: ",".join(f"{a}={b}" for a, b in k.items()) or "default")
def test_decode_equals_teacher_forcing(kw):
    cfg = small_cfg(**kw)
    model = make_model(cfg)
    perturb(model)
    B, T = 2, 24
    idx = rand_idx(cfg, B, T)
    with torch.no_grad():
        teacher, _ = model(idx)
        caches = model.decode_init()
        dec = torch.cat([model.decode_step(idx[:, t:t + 1], t, caches) for t in range(T)], dim=1)
    assert (teacher - dec).abs().max() < TOL


def test_deq_exact_when_sweeps_equal_length_and_frontier():
    T = 8
    cfg = small_cfg(max_seq_len=T, deq_sweeps=T)
    model = make_model(cfg)
    perturb(model)
    idx = rand_idx(cfg, 2, T)
    seq = _logits(model, idx, "sequential")
    assert (seq - _logits(model, idx, "deq")).abs().max() < TOL
    for m in range(1, T + 1):
        cfg.deq_sweeps = m
        part = _logits(model, idx, "deq")
        assert (seq[:, :m] - part[:, :m]).abs().max() < TOL, f"frontier broken at {m} sweeps"


def test_static_mode_runs_and_is_causal_shape():
    cfg = small_cfg(attn_mode="static")
    model = make_model(cfg)
    perturb(model)
    idx = rand_idx(cfg, 2, 12)
    logits, _ = model(idx)
    assert logits.shape == (2, 12, cfg.vocab_size) and torch.isfinite(logits).all()


@pytest.mark.parametrize("mode", ["sequential", "deq", "static", "vanilla"])
def test_causality(mode):
    cfg = small_cfg(attn_mode=mode)
    model = make_model(cfg)
    if mode != "vanilla":
        perturb(model)
    B, T, t = 2, 16, 7
    idx = rand_idx(cfg, B, T)
    emb = model.tok_emb(idx).detach().requires_grad_(True)
    logits, _ = model(inputs_embeds=emb)
    grad, = torch.autograd.grad(logits[:, t].sum(), emb)
    assert grad[:, t + 1:].abs().max() == 0.0
    assert grad[:, :t + 1].abs().max() > 0.0


@pytest.mark.parametrize("chunk", [5, 8])
def test_rematerialised_spans_keep_gradients(chunk):
    cfg = small_cfg()
    idx, tgt = rand_idx(cfg, 2, 24), rand_idx(cfg, 2, 24, seed=100)
    grads = {}
    for c in (0, chunk):
        model = make_model(cfg)
        perturb(model)
        model.train()
        cfg.checkpoint_chunk = c
        model(idx, targets=tgt)[1].backward()
        grads[c] = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    assert grads[0].keys() == grads[chunk].keys()
    for n in grads[0]:
        assert (grads[0][n] - grads[chunk][n]).abs().max() < 1e-6, n


def test_generate_and_accounting():
    cfg = small_cfg()
    model = make_model(cfg)
    out = model.generate(rand_idx(cfg, 2, 5), 6, temperature=0.8, top_k=10)
    assert out.shape == (2, 11)
    bd = model.param_breakdown()
    assert bd["base"] + bd["dualmod_extra"] == bd["total"]
    assert model.num_params() == bd["total"] - model.tok_emb.weight.numel()


def test_config_validation():
    from dual_mod_public_b200 import DualModConfig
    with pytest.raises(AssertionError):
        DualModConfig(attn_mode="bogus")
    with pytest.raises(AssertionError):
        DualModConfig(n_kv_heads=2)           # GQA is vanilla-only
    with pytest.raises(AssertionError):
        DualModConfig(gate_rank=8, gate_bias_init_k="ugi")
    cfg = DualModConfig(d_model=1024, n_heads=16)
    assert cfg.mlp_hidden == 2752 and cfg.head_dim == 64 and cfg.gate_in_dim == 2048
    assert DualModConfig.from_dict({**cfg.to_dict(), "unknown_knob": 1}).d_model == 1024
