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


def real_disagreements(a, b, tol=0.15):
    """Rows whose greedy tokens differ between two decoders although the reference's logits separate the two
    candidates by more than the logit tolerance (a difference inside it is a tie within bf16 noise)."""
    diff = (a.next != b.next).view(-1)
    if not diff.any():
        return 0
    lb = b.logits.view(b.logits.shape[0], -1)
    rows = diff.nonzero().view(-1)
    gap = lb[rows, b.next.view(-1)[rows]] - lb[rows, a.next.view(-1)[rows]]
    return int((gap > tol).sum())


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
        assert real_disagreements(d_k, d_t) == 0, t
        agree += int((d_k.next == d_t.next).all())
    assert agree >= T - 8                      # the rest are ties inside the logit tolerance
    assert d_k.pos.item() == T


@pytest.mark.gpu
@pytest.mark.parametrize("name,kw", [
    ("packed", dict()),
    ("packed, raw-pinned head, window", dict(kmod_vraw_heads=1, local_window=60)),
    ("mult_res factored", dict(ctx_mod="mult_res", gate_rank=16, ctx_rank=16, k_ctx_norm="rms", kmod_vraw_heads=1,
                               v_clamp_tau=2.0)),
    ("mult_res dense", dict(ctx_mod="mult_res", k_ctx_norm="rms", v_clamp_tau=0.0)),
    ("vanilla", dict(attn_mode="vanilla")),
])
def test_fused_step_matches_the_module_step(name, kw):
    """The decode step on the engines' kernels and weight packs (`fused`) against the same step through the module's
    own code (kernel read only), token by token from the same prompt: logits within bf16 noise, same arg-max."""
    from dual_mod_public_b200 import DualModConfig
    from dual_mod_public_b200.models import DualModLM
    torch.manual_seed(0)
    cfg = DualModConfig(d_model=256, n_layers=2, n_heads=4, vocab_size=300, max_seq_len=256, gate_bias_init=0.0, **kw)
    m = DualModLM(cfg)
    perturb(m)
    m = m.cuda().bfloat16().eval()
    B, T = 3, 130
    idx = torch.randint(0, 300, (B, T), device="cuda")
    d_f = GraphDecoder(m, B, 256, fused=True).capture()
    d_m = GraphDecoder(m, B, 256, fused=False).capture()
    assert d_f.fused and not d_m.fused and d_f.graph is not None
    agree = 0
    for t in range(T):
        for d in (d_f, d_m):
            d.tok.copy_(idx[:, t:t + 1])
            d.step()
        assert (d_f.logits - d_m.logits).abs().max() < 0.15, (name, t)
        assert real_disagreements(d_f, d_m) == 0, (name, t)
        agree += int((d_f.next == d_m.next).all())
    assert agree >= T - 8, (name, agree)
    assert not d_f.ops.fallbacks.get("refine_fwd") and not d_f.ops.fallbacks.get("mrk_refine_fwd"), d_f.ops.fallbacks


@pytest.mark.gpu
def test_graph_generate_matches_the_eager_decoder_on_the_gpu():
    """`GraphDecoder.capture()` + `generate` (CUDA graph, kernel read) against the same decoder run op by op
    with the torch read: the same greedy tokens, except where two logits tie within bf16 noise."""
    from dual_mod_public_b200 import DualModConfig
    from dual_mod_public_b200.models import DualModLM
    torch.manual_seed(0)
    cfg = DualModConfig(d_model=256, n_layers=2, n_heads=4, vocab_size=300, max_seq_len=256, gate_bias_init=0.0)
    m = DualModLM(cfg)
    perturb(m)
    m = m.cuda().bfloat16().eval()
    B, plen, new = 4, 40, 24
    prompt = torch.randint(0, 300, (B, plen), device="cuda")
    g_k, n_k = GraphDecoder(m, B, 256).capture().generate(prompt, new)
    g_t, n_t = GraphDecoder(m, B, 256, use_kernel=False).generate(prompt, new)
    assert n_k == n_t == new and g_k.shape == (B, new)
    assert (g_k == g_t).float().mean() > 0.9
    assert torch.equal(g_k[:, 0], g_t[:, 0])


@pytest.mark.gpu
def test_adapter_generation_on_the_gpu_matches_its_cpu_path(tmp_path):
    """The evaluation adapter's batched greedy generation through the static-tape decoder on a GPU (fixed batch
    of `gen_rows` rows, short batches padded) against its `decode_step` path on the CPU, fp32 weights."""
    import os

    from dual_mod_public_b200 import DualModConfig
    from dual_mod_public_b200.eval.lm_eval_adapter import DualModEval
    from dual_mod_public_b200.models import DualModLM
    from dual_mod_public_b200.utils.checkpoint import save_checkpoint
    torch.manual_seed(0)
    cfg = DualModConfig(d_model=64, n_layers=2, n_heads=4, vocab_size=300, max_seq_len=512, gate_bias_init=0.0,
                        checkpoint_chunk=0, dtype="fp32")
    save_checkpoint(str(tmp_path), DualModLM(cfg).eval(), step=1)
    ck = os.path.join(tmp_path, "ckpt_latest.pt")
    reqs = [("abc", {"until": [], "max_gen_toks": 6}), ("xyz", {"until": [], "max_gen_toks": 6}),
            ("hello", {"until": [], "max_gen_toks": 5})]
    cpu = DualModEval(ck, tokenizer="bytes", device="cpu", max_length=64, gen_rows=2).generate_until(reqs)
    gpu = DualModEval(ck, tokenizer="bytes", device="cuda:0", max_length=64, gen_rows=2).generate_until(reqs)
    assert len(gpu) == len(cpu) == 3 and all(isinstance(t, str) for t in gpu)
    assert sum(a == b for a, b in zip(cpu, gpu)) >= 2          # bf16 ties may flip a late token of one row
