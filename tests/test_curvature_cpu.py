import torch

from dual_mod_public_b200.train.curvature import ctx_params, ctx_top_eig, layer_grad_norms
from test_engine_cpu import build


def test_ctx_top_eig_matches_dense_hessian():
    cfg, m = build(d_model=32, n_heads=2, n_layers=1)
    g = torch.Generator().manual_seed(1)
    x = torch.randint(0, cfg.vocab_size, (2, 8), generator=g)
    y = torch.randint(0, cfg.vocab_size, (2, 8), generator=g)
    params = ctx_params(m)
    assert len(params) == 2
    flags = [p.requires_grad for p in m.parameters()]
    eig = ctx_top_eig(m, x, y, params, n_iter=60)
    assert [p.requires_grad for p in m.parameters()] == flags and not m.training
    # dense Hessian of the same restricted problem
    sizes = [p.numel() for p in params]
    base = [p.detach().clone() for p in params]

    def loss_of(flat):
        parts = flat.split(sizes)
        with torch.no_grad():
            for p, b in zip(params, base):
                p.copy_(b)
        # functional re-evaluation through the module with substituted weights
        from torch.func import functional_call
        names = [n for n, q in m.named_parameters() if any(q is p for p in params)]
        sub = {n: t.view_as(p) for n, t, p in zip(names, parts, params)}
        m.train()
        out = functional_call(m, sub, (x,), {"targets": y})[1]
        m.eval()
        return out
    H = torch.autograd.functional.hessian(loss_of, torch.cat([b.flatten() for b in base]))
    ev = torch.linalg.eigvalsh(0.5 * (H + H.t()))
    top = ev[ev.abs().argmax()].item()
    assert abs(eig - top) < 5e-2 * abs(top) + 1e-6, (eig, top)


def test_layer_grad_norms():
    cfg, m = build()
    from dual_mod_public_b200.engines.gradbuf import GradBuffers
    G = GradBuffers(list(m.parameters()))
    for p in m.parameters():
        G.get(p).fill_(1.0)
    out = layer_grad_norms(m, G)
    n0 = sum(p.numel() for p in m.blocks[0].parameters())
    assert set(out) == {"gradnorm/L00", "gradnorm/L01"} and abs(out["gradnorm/L00"] - n0 ** 0.5) < 1e-3
