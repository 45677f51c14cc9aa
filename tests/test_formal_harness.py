"""Formal-language trainers end to end on CPU: every task makes a batch the model accepts,
a few eager steps reduce the loss, the engine path agrees with the eager path's loss, and
hand-computed d_logits equal autograd's."""

import torch

from dual_mod_public_b200.formal import harness as H
from dual_mod_public_b200.formal import train_statetrack as TS
from dual_mod_public_b200.formal.tasks import step_rng


def test_every_task_builds_a_batch_within_vocab():
    for task in H.TASK_ID:
        extra = dict(n_ops={"matinv": 3, "match3": 24}.get(task, 6), max_ops=24, cvp_inputs=8, ca_w=8)
        args = H.task_args(task=task, **extra)
        mul, n = H.task_tables(args)
        vocab = H.vocab_of(args, n)
        x, tg, m, d = H.make_batch(args, mul, n, step_rng(H.TASK_ID[task], 0, 1, 0), 4, args.n_ops)
        assert x.max() < vocab and m.any(), task
        if tg is not None:
            assert tg[m].max() < vocab, task


def test_masked_dlogits_matches_autograd():
    torch.manual_seed(0)
    logits = torch.randn(3, 7, 11, requires_grad=True)
    tok = torch.randint(0, 11, (3, 7))
    msk = torch.zeros(3, 7, dtype=torch.bool)
    msk[:, 2::2] = True
    for tgt in (None, torch.randint(0, 11, (3, 7))):
        loss = H.masked_loss(logits, tok, tgt, msk)
        (g,) = torch.autograd.grad(loss, logits)
        l2, d = H.masked_dlogits(logits.detach(), tok, tgt, msk)
        assert abs(loss.item() - l2.item()) < 1e-6 and (g - d).abs().max() < 1e-6


def test_eager_training_reduces_loss(tmp_path):
    final = TS.main(["--task", "group", "--group", "z10", "--format", "tagged", "--n_ops", "8", "--arch", "dualmod",
                     "--n_layers", "1", "--steps", "40", "--bsz", "16", "--lr", "3e-3", "--device", "cpu",
                     "--eval_rows", "32", "--gen_factors", "1,2", "--eval_every", "20", "--out_root", str(tmp_path),
                     "--eval_dump"])
    assert 1 in final and (tmp_path / "analysis").exists()
    ck = torch.load(next((tmp_path / "out" / "statetrack_ckpts").glob("*.pt")), weights_only=False)
    assert set(ck) == {"model", "args"}


def test_baseline_archs_take_a_step(tmp_path):
    for arch, extra in (("vanilla", []), ("lstm", []), ("gdn", []), ("fbt", []),
                        ("looped", ["--loop_k", "3", "--loop_k_min", "1"]),
                        ("looped", ["--loop_huginn", "--loop_k", "4", "--loop_k_mean", "2", "--loop_bp", "2"]),
                        ("fbt", ["--fbt_sched", "3:1,1:2"])):
        TS.main(["--task", "parity", "--n_ops", "6", "--arch", arch, "--n_layers", "1", "--steps", "2", "--bsz", "4",
                 "--device", "cpu", "--eval_rows", "8", "--gen_factors", "1", "--out_root", str(tmp_path)] + extra)


def test_engine_path_trains(tmp_path):
    final = TS.main(["--task", "group", "--group", "z10", "--format", "tagged", "--n_ops", "15", "--arch", "dualmod",
                     "--n_layers", "1", "--steps", "30", "--bsz", "8", "--lr", "3e-3", "--device", "cpu",
                     "--eval_rows", "16", "--gen_factors", "1", "--engine", "wavescan", "--ws_chunk", "8",
                     "--eval_every", "15", "--out_root", str(tmp_path)])
    assert final[1] >= 0.0


def test_warm_starts_keep_the_vocabulary_layout(tmp_path):
    """Keyed K = 2 -> K_max 8: base + key rows stay in place, the 2n group rows move to the new tail, untrained
    key rows start near the mean of the trained ones; a deeper model's extra block starts as identity; the
    body stays frozen for the first steps; cvp grows by moving its 4 value tokens to the new tail."""
    from dual_mod_public_b200.formal import tasks as T
    common = ["--task", "keyed", "--group", "z10", "--D", "2", "--arch", "dualmod", "--bsz", "8", "--lr", "3e-3",
              "--device", "cpu", "--eval_rows", "8", "--gen_factors", "1", "--eval_every", "50",
              "--out_root", str(tmp_path), "--eval_dump"]
    TS.main(common + ["--K", "2", "--K_max", "4", "--n_layers", "1", "--steps", "3", "--tag", "src"])
    src = torch.load(tmp_path / "out" / "statetrack_ckpts" / "src_dualmod.pt", weights_only=False)
    assert src["args"]["K"] == 2 and src["args"]["tag"] == "src"
    n = 10
    args = TS.parse(common + ["--K", "4", "--K_max", "8", "--n_layers", "2", "--newkey_init", "mean", "--init_stack"])
    mul, n_elem = H.task_tables(args)
    model, _ = H.build_model("dualmod", H.vocab_of(args, n_elem), 64, scale=args.scale, n_layers=2)
    before = model.tok_emb.weight.detach().clone()
    TS.load_warm_start(model, str(tmp_path / "out" / "statetrack_ckpts" / "src_dualmod.pt"), args, n_elem)
    W, S = model.tok_emb.weight.detach(), src["model"]["tok_emb.weight"]
    assert S.shape[0] == T.BASE + 4 + 2 * n and W.shape[0] == T.BASE + 8 + 2 * n
    assert torch.equal(W[:T.BASE + 2], S[:T.BASE + 2]) and torch.equal(W[-2 * n:], S[-2 * n:])
    new_keys, trained = W[T.BASE + 2:T.BASE + 8], S[T.BASE:T.BASE + 2]
    assert not torch.equal(new_keys, before[T.BASE + 2:T.BASE + 8])
    assert (new_keys.mean(0) - trained.mean(0)).abs().max() < 3 * trained.std(0).max() + 1e-3
    assert model.blocks[1].attn.wo.weight.abs().max() == 0 and model.blocks[1].mlp.w2.weight.abs().max() == 0
    assert model.blocks[0].attn.wo.weight.abs().max() > 0
    # frozen body (gradients zeroed; no weight decay here): after two steps only the embedding (tied head) has moved
    for engine in ([], ["--engine", "wavescan", "--ws_chunk", "8"]):
        TS.main(common + ["--K", "2", "--K_max", "4", "--n_layers", "1", "--steps", "2", "--freeze_body_steps", "5", "--wd", "0",
                          "--init_from", str(tmp_path / "out" / "statetrack_ckpts" / "src_dualmod.pt"), "--tag", "frz"]
                + engine)
        frz = torch.load(tmp_path / "out" / "statetrack_ckpts" / "frz_dualmod.pt", weights_only=False)["model"]
        assert torch.equal(frz["blocks.0.attn.wq.weight"], src["model"]["blocks.0.attn.wq.weight"]), engine
        assert not torch.equal(frz["tok_emb.weight"], src["model"]["tok_emb.weight"]), engine
    # cvp: 6 -> 12 gates
    cv = ["--task", "cvp", "--cvp_inputs", "4", "--arch", "dualmod", "--n_layers", "1", "--bsz", "4", "--device", "cpu",
          "--eval_rows", "4", "--gen_factors", "1", "--eval_every", "50", "--out_root", str(tmp_path), "--eval_dump"]
    TS.main(cv + ["--n_ops", "6", "--max_ops", "6", "--steps", "2", "--tag", "cv6", "--cvp_leak", "2", "--curriculum"])
    s6 = torch.load(tmp_path / "out" / "statetrack_ckpts" / "cv6_dualmod.pt", weights_only=False)["model"]["tok_emb.weight"]
    a12 = TS.parse(cv + ["--n_ops", "12", "--max_ops", "12"])
    m12, _ = H.build_model("dualmod", H.vocab_of(a12, 0), 128, scale=a12.scale, n_layers=1)
    TS.load_warm_start(m12, str(tmp_path / "out" / "statetrack_ckpts" / "cv6_dualmod.pt"), a12, 0)
    W12 = m12.tok_emb.weight.detach()
    assert W12.shape[0] == s6.shape[0] + 6 and torch.equal(W12[-4:], s6[-4:]) and torch.equal(W12[:s6.shape[0] - 4], s6[:-4])


def test_checkpoint_reevaluation_and_composition_statistics(tmp_path):
    import numpy as np
    from dual_mod_public_b200.formal import analysis as A
    from dual_mod_public_b200.formal import tasks as T
    TS.main(["--task", "group", "--group", "s3", "--format", "tagged", "--n_ops", "8", "--arch", "dualmod", "--n_layers", "1",
             "--steps", "30", "--bsz", "16", "--lr", "3e-3", "--device", "cpu", "--eval_rows", "16", "--gen_factors", "1",
             "--eval_every", "100", "--out_root", str(tmp_path), "--eval_dump", "--tag", "g"])
    ck = str(tmp_path / "out" / "statetrack_ckpts" / "g_dualmod.pt")
    r = A.reeval(ck, factor=2, rows=16)
    assert 0.0 <= r[2] <= 1.0 and r["state_dict_mismatch"] == {"missing": 0, "unexpected": 0} and len(r["x2_by_pos8"]) >= 7
    c = A.composition(ck, rows=16)
    assert c["n_states"] == 6 and c["all"]["n"] == 16 * 8 and 0 <= c["all"]["top1"] <= c["all"]["top5"] <= 1
    assert len(c["octiles"]) == 8 and sum(o["n"] for o in c["octiles"]) == c["all"]["n"]
    # the statistics on made-up logits: gold always second -> rank 1, and a fixed correction element
    mul, n = T.cayley("z5")
    inv = A.inverse_table(np.asarray(mul))
    assert all(mul[g][inv[g]] == 0 for g in range(n))
    gold = np.arange(20) % n
    lg = np.zeros((20, n))
    lg[np.arange(20), gold] = 1.0
    lg[np.arange(20), (gold + 1) % n] = 2.0                      # predicts gold + 1: correction = -1, word length 1
    s = A.composition_stats(lg, gold, np.arange(20), 20, np.asarray(mul))
    assert s["all"]["top1"] == 0.0 and s["all"]["top5"] == 1.0 and s["all"]["mean_rank"] == 1.0
    assert s["all"]["p_wordlen_le2"] == 1.0 and s["all"]["entropy_ratio"] == 0.0 and abs(s["all"]["top5_mass"] - 1.0) < 1e-9


def test_result_tables(tmp_path):
    from dual_mod_public_b200.formal import summarize as S
    for L, seed in ((1, 0), (1, 1), (2, 0)):
        TS.main(["--task", "group", "--group", "z10", "--format", "tagged", "--n_ops", "6", "--arch", "dualmod",
                 "--n_layers", str(L), "--steps", "3", "--bsz", "8", "--device", "cpu", "--eval_rows", "8",
                 "--gen_factors", "1,2", "--eval_every", "50", "--seed", str(seed), "--out_root", str(tmp_path)])
    runs = S.load(str(tmp_path / "analysis"))
    assert len(runs) == 3 and {r["layers"] for r in runs} == {1, 2}
    assert len(S.listing(runs)) == 4 and "x2=" in S.listing(runs)[1]
    grid = S.depth_grid(runs, "z10", solved=0.0)
    assert any("T=6" in l and "2/2" in l and "1/1" in l for l in grid)          # two seeds at depth 1, one at depth 2
    assert "shallowest solving depth: {6: 1}" in grid[-1]
    assert S.by_sidecar(runs, "pos8") and S.main([str(tmp_path / "analysis")])
