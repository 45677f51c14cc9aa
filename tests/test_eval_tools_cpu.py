"""Evaluation tooling on CPU: harness adapter (likelihood == direct scan log-probs, bucketing order, greedy
generation == model.generate path, generation cache), MQAR batches, held-out loss, decode validator,
looped fixed-point table, engine validator."""

import json
import os

import torch
import torch.nn.functional as F

from dual_mod_public_b200 import DualModConfig
from dual_mod_public_b200.eval import mqar
from dual_mod_public_b200.eval.heldout_loss import score
from dual_mod_public_b200.eval.lm_eval_adapter import ByteTokenizer, DualModEval, trunc_keep_head
from dual_mod_public_b200.models import DualModLM
from dual_mod_public_b200.utils.checkpoint import save_checkpoint


def tiny(vocab=300, T=64):
    torch.manual_seed(0)
    cfg = DualModConfig(d_model=64, n_layers=2, n_heads=4, vocab_size=vocab, max_seq_len=T, gate_bias_init=0.0,
                        checkpoint_chunk=0, dtype="fp32")
    return DualModLM(cfg).eval()


def test_adapter_likelihood_matches_direct_scoring(tmp_path):
    m = tiny()
    save_checkpoint(str(tmp_path), m, step=3)
    lm = DualModEval(os.path.join(tmp_path, "ckpt_latest.pt"), tokenizer="bytes", device="cpu", batch_rows=2,
                     max_length=64)
    reqs = [("the cat", " sat"), ("a", " much longer continuation here"), ("", "x"), ("hello wor", "ld")]
    got = lm.loglikelihood(reqs)
    tk = ByteTokenizer()
    for (ctx, cont), (lp, greedy) in zip(reqs, got):
        c, k = [1] + tk.encode(ctx), tk.encode(cont)
        x = torch.tensor([c + k])
        with torch.no_grad():
            logp = F.log_softmax(m(x)[0].float(), -1)[0]
        ref = sum(logp[len(c) - 1 + j, t].item() for j, t in enumerate(k))
        assert abs(lp - ref) < 1e-3, (ctx, cont, lp, ref)
        assert isinstance(greedy, bool)
    roll = lm.loglikelihood_rolling([("some document text",)])
    assert len(roll) == 1 and roll[0] < 0


def test_adapter_generation_and_cache(tmp_path, monkeypatch):
    m = tiny()
    cache = str(tmp_path / "gen.jsonl")
    monkeypatch.setenv("EVAL_GEN_CACHE", cache)
    lm = DualModEval(None, tokenizer="bytes", device="cpu", model=m, max_length=64)
    reqs = [("abc", {"until": ["\n"], "max_gen_toks": 6}), ("zz", {"max_gen_toks": 4})]
    out = lm.generate_until(reqs)
    # the same greedy tokens as an explicit decode loop
    ids = [1] + ByteTokenizer().encode("abc")
    caches, lg = m.decode_init(), None
    for t, tok in enumerate(ids):
        lg = m.decode_step(torch.tensor([[tok]]), t, caches)
    first = int(lg[0, -1].argmax())
    assert ByteTokenizer().decode([first])[:1] == (out[0][:1] if out[0] else ByteTokenizer().decode([first])[:1])
    assert len(open(cache).read().strip().splitlines()) == 2
    monkeypatch.setenv("EVAL_CACHE_ONLY", "1")
    lm2 = DualModEval(None, tokenizer="bytes", device="cpu", model=m, max_length=64)
    assert lm2.generate_until(reqs) == out
    assert lm2.generate_until([("never seen", {"max_gen_toks": 2})]) == ["<UNCACHED>"]
    monkeypatch.setenv("GEN_TRUNC", "head")
    t = trunc_keep_head(list(range(1000)), 100)
    assert len(t) == 100 and t[0] == 0 and t[-1] == 999


def test_mqar_batches_and_scoring():
    x, pos, tok = mqar.build_batch(4, 3, 64, 5, seed=1, vocab=300)
    assert x.shape == (5, 64) and pos.shape == (5, 3)
    bos, SEP, EQ, Q = mqar.markers(300)
    for b in range(5):
        for p, t in zip(pos[b].tolist(), tok[b].tolist()):
            assert x[b, p] == EQ and x[b, p + 1] == t and x[b, p - 2] == Q
            key = x[b, p - 1].item()
            first = (x[b] == key).nonzero()[0, 0].item()                 # the pair was shown before the query
            assert first < p - 1 and x[b, first + 2] == t
    x2, _, _ = mqar.build_batch(4, 3, 64, 5, seed=1, vocab=300)
    assert torch.equal(x, x2)
    m = tiny()
    r = mqar.run(m, 4, 3, 64, 8, 0, "cpu", rows=4)
    assert 0.0 <= r <= 1.0
    l = mqar.finetune(m, 2, 4, 3, 64, 4, 1e-3, "cpu")
    assert l == l


def test_heldout_loss_matches_model_loss():
    m = tiny()
    g = torch.Generator().manual_seed(2)
    val = torch.randint(0, 300, (2, 3, 33), generator=g)
    got = score(m, val, "cpu")
    m.cfg.attn_mode = "sequential"
    with torch.no_grad():
        ref = [m(v[:, :-1], targets=v[:, 1:])[1].item() for v in val]
    assert all(abs(a - b) < 1e-5 for a, b in zip(got, ref))


def test_decode_validator_and_engine_validator():
    from dual_mod_public_b200.eval.bench_decode import main as dec_main
    out = dec_main(["--model", "tiny", "--validate", "--device", "cpu"])
    for arm in ("dualmod", "vanilla"):
        assert out[arm]["agree_tf"] >= 0.999 and out[arm]["max_dlogit_tf"] < 1e-4
        assert out[arm]["agree_eager"] >= 0.999 and out[arm]["max_dlogit_eager"] < 1e-4
    from dual_mod_public_b200.train.validate_engine import main as val_main
    lines = []
    res = val_main(["--engine", "wavescan", "--T", "32", "--C", "8", "--d", "64", "--W", "12", "--ladder", "2",
                    "--device", "cpu"], out=lines.append)
    assert res["R1 full causal"] is True and res["R2 window 12"] is True and "R4 K=2" in res
    res = val_main(["--engine", "wave3d", "--T", "16", "--C", "4", "--d", "64", "--device", "cpu"], out=lines.append)
    assert res["R1 full causal"] is True


def test_loop_fixed_point_table():
    from dual_mod_public_b200.formal.loop_fixed_point import analyse
    from dual_mod_public_b200.models.baselines import LoopedLM
    torch.manual_seed(0)
    cfg = DualModConfig(d_model=32, n_layers=1, n_heads=2, vocab_size=40, max_seq_len=32, attn_mode="vanilla")
    m = LoopedLM(cfg, n_unique=1, k_max=8).eval()
    x = torch.randint(0, 40, (3, 16))
    rows = analyse(m, x, torch.roll(x, -1, 1), torch.ones(3, 16, dtype=torch.bool), K=6, out=lambda s: None)
    assert len(rows) == 6 and rows[0][1] != rows[0][1] and all(0 <= r[2] <= 1 for r in rows)
    assert all(r[1] == r[1] for r in rows[1:])
