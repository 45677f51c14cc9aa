"""Shared fixtures for the exactness tests: a tiny fp32 model and a weight
perturbation that moves it away from the near-vanilla init (gates around 0.5,
ctx branch live), so a test that passes is testing genuinely non-vanilla math."""

import torch

from dual_mod_public_b200 import DualModConfig
from dual_mod_public_b200.models import DualModLM


def small_cfg(**kw):
    base = dict(d_model=64, n_layers=2, n_heads=4, vocab_size=97, max_seq_len=32,
                attn_mode="sequential", checkpoint_chunk=0, dtype="fp32")
    base.update(kw)
    return DualModConfig(**base)


def make_model(cfg, device="cpu", seed=1234):
    torch.manual_seed(seed)
    return DualModLM(cfg).to(device).eval()


def _randomise(mod, std):
    for p in mod.parameters():
        if p.dim() >= 2:
            p.normal_(0, std)


def perturb(model, seed=7, gate_bias=0.0, ctx_std=0.05):
    torch.manual_seed(seed)
    with torch.no_grad():
        for blk in model.blocks:
            a = blk.attn
            for gate, ctx in (("w_gk", "w_kctx"), ("w_gv", "w_vctx")):
                if hasattr(a, ctx):
                    getattr(a, gate).bias.fill_(gate_bias)
                    _randomise(getattr(a, gate), 0.05 if model.cfg.gate_rank == 0 else 0.2)
                    _randomise(getattr(a, ctx), ctx_std if model.cfg.ctx_rank == 0 else 0.2)
            for extra in ("v_pre", "k_pre", "v_gate", "v_map"):
                if hasattr(a, extra):
                    _randomise(getattr(a, extra), 0.05 if model.cfg.ctx_rank == 0 else 0.2)
            for gain in ("k_gain", "v_gain", "ctx_gain"):
                if hasattr(a, gain):
                    getattr(a, gain).uniform_(0.5, 1.5)
            if hasattr(a, "norm_ctx"):
                a.norm_ctx.weight.uniform_(0.5, 1.5)


def rand_idx(cfg, B, T, device="cpu", seed=99):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (B, T), generator=g).to(device)


def free_port():
    """A TCP port nobody listens on right now (bound to 0 and released), for the rendezvous of spawned ranks."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sk:
        sk.bind(("127.0.0.1", 0))
        return sk.getsockname()[1]
