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
        assert out[arm]["accept"] and out[arm]["identical_continuations"] == out[arm]["continuations"]
        assert len(out[arm]["drift_by_octile"]) == 8
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


def test_engine_scoring_and_generation_at_exact_k_match_the_scan(tmp_path, monkeypatch):
    from dual_mod_public_b200.eval.lm_eval_adapter import WavefrontEval
    m = tiny()
    save_checkpoint(str(tmp_path), m, step=3, extra={"engine_kwargs": {"C": 16}})
    ck = os.path.join(tmp_path, "ckpt_latest.pt")
    monkeypatch.setenv("EVAL_LEN_QUANT", "16")
    ref = DualModEval(ck, tokenizer="bytes", device="cpu", batch_rows=2, max_length=48)
    # 48 positions in chunks of 16: the wavefront is exact from K = 48 - 3 + 1 sweeps on
    for engine, K in (("wave3d", 46), ("wavescan", 16)):
        lm = WavefrontEval(ck, K, T_eval=48, C=16, engine=engine, gen_rows=2, tokenizer="bytes", device="cpu",
                           batch_rows=2)
        reqs = [("the cat", " sat"), ("a", " much longer continuation"), ("", "x"), ("hello wor", "ld"), ("ab", "c")]
        for (lp, g), (lp_r, g_r) in zip(lm.loglikelihood(reqs), ref.loglikelihood(reqs)):
            assert abs(lp - lp_r) < 2e-3 and g == g_r, (engine, lp, lp_r)
        gen = [("abc", {"until": [], "max_gen_toks": 5}), ("hello there", {"until": [], "max_gen_toks": 5}),
               ("x", {"until": [], "max_gen_toks": 3})]
        assert lm.generate_until(gen) == ref.generate_until(gen), engine
    # an approximate operator (few sweeps) still scores, and differs
    few = WavefrontEval(ck, 2, T_eval=48, C=16, tokenizer="bytes", device="cpu", batch_rows=2)
    a, b = few.loglikelihood(reqs[:2]), ref.loglikelihood(reqs[:2])
    assert all(abs(x[0] - y[0]) < 5.0 for x, y in zip(a, b)) and any(abs(x[0] - y[0]) > 1e-6 for x, y in zip(a, b))
    # per-rank generation cache
    monkeypatch.setenv("GEN_CACHE_DIR", str(tmp_path / "gc"))
    first = few.generate_until(gen[:2])
    assert len(os.listdir(tmp_path / "gc")) == 1
    few._generate_engine = None                                     # a second call must not generate
    assert few.generate_until(gen[:2]) == first


def test_recall_and_needle_protocols_run_from_local_files(tmp_path):
    from dual_mod_public_b200.eval import collate, recall_tasks as R
    from dual_mod_public_b200.eval.run_lm_eval import main as eval_main
    tk = ByteTokenizer()
    filler = "lorem ipsum dolor sit amet " * 40
    doc = {"text": filler + "The serial number: QX-7731. " + filler, "key": "serial number", "value": "QX-7731"}
    cut = R.cut_to_answer(doc, "text", ("key", "value"), tk, context_length=300, answer_length=50)
    n = len(tk.encode(cut["text"]))
    assert n <= 250 and "QX-7731" in cut["text"]
    at = cut["text"].lower().index("serial number")
    assert abs(at - 125) < 30                                        # the window is centred on the first match
    head = R.cut_to_answer({"context": filler * 3, "question": "q?", "answers": ["x"]}, "context", (), tk, 300, 50)
    assert head["context"] == (filler * 3).strip()[:250]
    assert R.cut_to_answer({"text": "a b", "key": "k", "value": "7"}, "text", ("value",), tk) is None
    p = R.recall_prompt("fda", {"text": "Device: X9.\nserial number:", "key": "serial number", "value": "X9"}, tk)
    assert p == "Device: X9. Serial number:"
    p = R.recall_prompt("swde", {"text": "Title: Alien. " + R.SUMMARY_MARK + " junk", "key": "title", "value": "Alien"}, tk)
    assert p == "Title: Alien. Title:"
    p = R.recall_prompt("triviaqa", {"context": "[DOC] Paris is in France. Where is Paris?", "question": " Where is Paris? ",
                                     "answers": ["France"]}, tk)
    assert p == "Paris is in France. Where is Paris?"
    assert R.contains_score("it is FRANCE!", ["france", "gaul"]) == 1 and R.contains_score("spain", ["france"]) == 0
    assert R.match_all("keys 12 and 99", ["12", "99", "7"]) == 2 / 3
    assert R.shard(list(range(10)), "1/4") == [1, 5, 9]

    class Echo:                                                      # answers with the tail of the prompt
        tok = tk

        def generate_until(self, reqs):
            return [r[0][-40:] for r in reqs]

    docs = [{"text": "The code is ABC.", "key": "code", "value": "ABC"}, {"text": "Nothing here.", "key": "code", "value": "ZZZ"}]
    dump = str(tmp_path / "s0_TEXT.jsonl")
    assert R.run_recall(Echo(), "fda", docs, tk, dump=dump) == {"contains": 0.5, "n": 2}
    hits, n, lines = collate.pool([dump, dump])
    assert (hits, n) == (2, 4) and lines[-1].startswith("POOLED contains = 50.00")
    root = tmp_path / "ruler"
    os.makedirs(root / "niah_single_1_1024")
    with open(root / "niah_single_1_1024" / "validation.jsonl", "w") as f:
        f.write(json.dumps({"input": "hay needle 4242 hay\n", "outputs": ["4242"], "answer_prefix": " The number is"}) + "\n")
    nd = R.load_needles(str(root), "niah_single_1", [1024, 2048])
    assert nd[0]["gen_prefix"] == "The number is" and R.run_needles(Echo(), nd) == {"1024": 1.0, "n": 1}
    # the driver end to end on a checkpoint, local tasks only (no harness package needed)
    m = tiny()
    run = tmp_path / "runA"
    save_checkpoint(str(run), m, step=7)
    data = str(tmp_path / "fda.jsonl")
    with open(data, "w") as f:
        for d in docs:
            f.write(json.dumps(d) + "\n")
    out = str(tmp_path / "analysis")
    res = eval_main(["--ckpt", str(run / "ckpt_latest.pt"), "--tasks", "jrt_fda,niah_single_1", "--local_data", data,
                     "--ruler_root", str(root), "--ruler_lengths", "1024", "--device", "cpu", "--T_eval", "64",
                     "--out_dir", out, "--tag", "t"])
    assert set(res) == {"jrt_fda", "niah_single_1"} and res["jrt_fda"]["n"] == 2
    files = sorted(os.listdir(out))
    assert any(f.startswith("lmeval_runA_7_") and f.endswith("_t.json") for f in files)
    assert any(f.endswith("_jrt_fda_TEXT.jsonl") for f in files)
    lines = collate.table(out, "runA")
    assert any("jrt_fda" in l for l in lines) and any("niah_single_1" in l for l in lines)


def test_shell_drivers_parse():
    import glob
    import subprocess
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "dual_mod_public_b200")
    scripts = sorted(glob.glob(os.path.join(root, "**", "*.sh"), recursive=True))
    assert len(scripts) >= 7
    for s in scripts:
        assert subprocess.run(["bash", "-n", s], capture_output=True).returncode == 0, s


def test_profile_tool_shapes_are_valid_configs():
    from dual_mod_public_b200.ops import profile_step as P
    for name, sh in P.SHAPES.items():
        cfg = DualModConfig(n_layers=2, vocab_size=32000, gate_bias_init=0.0, **sh["cfg"])
        assert sh["T"] % 64 == 0 and cfg.d_model % cfg.n_heads == 0 and sh["engine"] in ("wavescan", "wave3d"), name


def test_generation_batches_by_prompt_length_and_matches_row_by_row(tmp_path):
    m = tiny()
    save_checkpoint(str(tmp_path), m, step=1)
    ck = os.path.join(tmp_path, "ckpt_latest.pt")
    one = DualModEval(ck, tokenizer="bytes", device="cpu", max_length=64, gen_rows=1)
    many = DualModEval(ck, tokenizer="bytes", device="cpu", max_length=64, gen_rows=3)
    calls = []
    inner = many._greedy_batch
    many._greedy_batch = lambda prompts, max_new, stops: (calls.append(len(prompts)), inner(prompts, max_new, stops))[1]
    reqs = [("abc", {"until": [], "max_gen_toks": 6}), ("xyz", {"until": [], "max_gen_toks": 6}),
            ("hello", {"until": ["e"], "max_gen_toks": 6}), ("qrs", {"until": [], "max_gen_toks": 6}),
            ("tuv", {"until": [], "max_gen_toks": 6}), ("world", {"until": ["e"], "max_gen_toks": 6}),
            ("abc", {"until": [], "max_gen_toks": 4})]
    assert many.generate_until(reqs) == one.generate_until(reqs)
    # four 3-byte prompts with one budget -> batches of 3 + 1; the two 5-byte prompts together; the odd budget alone
    assert sorted(calls) == [1, 1, 2, 3]


def test_step_model_arithmetic():
    from dual_mod_public_b200.ops import step_model as M
    rows = M.model()
    N, d, ffn, K = 32 * 2048, 1024, 2816, 4
    per_layer = 2 * N * (4 * (6 * d * d + 3 * d * ffn) + K * 3 * 4 * d * d)
    assert rows["GEMM (layers)"][0] == per_layer * 24 * 8
    fact = M.model(ranks=(16, 16, 16))
    assert fact["GEMM (layers)"][0] < rows["GEMM (layers)"][0] and fact["attention"] == rows["attention"]
    lines, total = M.report(rows, measured_ms=8000.0)
    assert 1.0 < total < 8.0 and "of it" in lines[-1]


def test_decode_validator_takes_a_checkpoint_and_real_tokens(tmp_path):
    import numpy as np
    from dual_mod_public_b200.eval.bench_decode import main as dec_main
    m = tiny(vocab=300, T=128)
    save_checkpoint(str(tmp_path), m, step=2)
    np.arange(2000, dtype=np.uint16).tofile(tmp_path / "toks.bin")
    out = dec_main(["--ckpt", os.path.join(tmp_path, "ckpt_latest.pt"), "--validate", "--device", "cpu", "--val_len", "40",
                    "--prompt", "32", "--gen", "8", "--tokens_bin", str(tmp_path / "toks.bin")])
    assert "vanilla" not in out and out["dualmod"]["accept"] and out["model"].endswith("ckpt_latest.pt")
