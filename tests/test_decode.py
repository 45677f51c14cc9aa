"""Static-tape decoder == eager decode_step == teacher forcing (CPU, fp32), greedy
generation shapes, the vanilla control, and the GPU kernel read against the torch read."""

import pytest
import torch

from dual_mod_public_b200.eval.graph_decode import GraphDecoder

from helpers import make_model, perturb, rand_idx, small_cfg


@pytest.mark.parametrize("kw", [dict(), dict(local_window=6), dict(attn_mode="vanilla"),
                                dict(ctx_mod="mult_res", k_ctx_norm="rms", kmod_vraw_heads=1)])
def test_static_tape_decoder_equals_teacher_forcing(kw):
    cfg = small_cfg(**kw)
    m = make_model(cfg)
    if cfg.attn_mode != "vanilla":
        perturb(m)
    B, T = 2, 20
    idx = rand_idx(cfg, B, T)
    with torch.no_grad():
        teacher = m(idx)[0]
    dec = GraphDecoder(m, B, 32, dtype=torch.float32)
    outs = []
    for t in range(T):
        dec.tok.copy_(idx[:, t:t + 1])
        dec.step()
        outs.append(dec.logits.clone())
    assert (torch.cat(outs, 1) - teacher).abs().max() < 1e-4
    gen, k = dec.generate(idx[:, :5], 6)
    assert gen.shape == (B, 6) and k == 6
    # greedy continuation equals argmax of the eager decode
    caches = m.decode_init()
    for t in range(5):
        lg = m.decode_step(idx[:, t:t + 1], t, caches)
    assert torch.equal(gen[:, 0], lg[:, -1].argmax(-1))


@pytest.mark.gpu
@pytest.mark.parametrize("dh,window", [(64, 0), (128, 0), (64, 50)])
def test_kernel_read_matches_torch_read(dh, window):
    from dual_mod_public_b200 import DualModConfig
    from dual_mod_public_b200.models import DualModLM
    torch.manual_seed(0)
    cfg = DualModConfig(d_model=4 * dh, n_layers=2, n_heads=4, vocab_size=300, max_seq_len=256,
                        gate_bias_init=0.0, local_window=window)
    m = DualModLM(cfg)
    perturb(m)
    m = m.cuda().bfloat16().eval()
    B, T = 3, 150
    idx = torch.randint(0, 300, (B, T), device="cuda")
    d_k = GraphDecoder(m, B, 256).capture()
    d_t = GraphDecoder(m, B, 256, use_kernel=False)
    assert d_k.use_kernel and d_k.graph is not None
    agree = 0
    for t in range(T):
        for d in (d_k, d_t):
            d.tok.copy_(idx[:, t:t + 1])
            d.step()
        assert (d_k.logits - d_t.logits).abs().max() < 0.15, t
        agree += int((d_k.next == d_t.next).all())
    assert agree >= T - 3
    assert d_k.pos.item() == T
