"""Loaders are pure functions of (seed, step), rank slices tile the global batch; the
checkpoint layout round-trips and a state dict with the reference's key names loads."""

import os

import numpy as np
import torch

from dual_mod_public_b200.data import PackedLoader, SyntheticStream, memmap_stream, write_corpus
from dual_mod_public_b200.models.telemetry import collect_telemetry, grad_norm_ratios
from dual_mod_public_b200.parallel.fused_optim import FusedDPAdamW, decay_groups, default_buckets
from dual_mod_public_b200.utils.checkpoint import (AsyncCheckpointWriter, build_checkpoint, load_checkpoint,
                                                   model_from_checkpoint, save_checkpoint, save_persist)

from helpers import make_model, perturb, rand_idx, small_cfg


def test_packed_loader_rank_slices_tile_global_batch(tmp_path):
    write_corpus(tmp_path / "train.bin", np.arange(5000) % 997)
    full = PackedLoader(str(tmp_path), "train", 16, 8, data_seed=3)
    parts = [PackedLoader(str(tmp_path), "train", 16, 8, data_seed=3, rank=r, world_size=4) for r in range(4)]
    for step in (0, 7, 60):
        whole = full.train_block(step)
        assert torch.equal(whole, torch.cat([p.train_block(step) for p in parts]))
        x, y = full.train_batch(step)
        assert torch.equal(x[:, 1:], y[:, :-1])
    assert torch.equal(full.train_block(5), PackedLoader(str(tmp_path), "train", 16, 8, data_seed=3).train_block(5))
    assert full.val_block(2).shape == (8, 17)


def test_memmap_stream_resume_and_synthetic(tmp_path):
    write_corpus(tmp_path / "c.bin", np.arange(20000) % 911)
    a = memmap_stream(str(tmp_path / "c.bin"), 32, 4, rank=1, world=2)
    seq = [next(a) for _ in range(5)]
    b = memmap_stream(str(tmp_path / "c.bin"), 32, 4, rank=1, world=2, start_step=3)
    assert torch.equal(next(b), seq[3]) and seq[0].shape == (4, 33)
    s = SyntheticStream(100, 16, 4, rank=2)
    assert torch.equal(s.block(9), SyntheticStream(100, 16, 4, rank=2).block(9))
    assert not torch.equal(s.block(9), s.block(10))


def test_checkpoint_roundtrip_and_reference_keys(tmp_path):
    cfg = small_cfg(ctx_mod="mult_res", gate_rank=8, ctx_rank=8, k_ctx_norm="rms")
    m = make_model(cfg)
    perturb(m)
    opt = FusedDPAdamW(decay_groups(m, 0.1), default_buckets(m), lr=1e-3, use_kernel=False)
    opt.flat_grads.normal_()
    opt.step()
    ck = save_checkpoint(str(tmp_path), m, opt, step=12, applied=11, extra={"gn_ema": {False: 1.0}, "gn_cnt": {False: 3}})
    keys = set(ck["model"])
    for k in ("tok_emb.weight", "blocks.0.attn.w_gk.a.weight", "blocks.0.attn.w_gk.b.bias",
              "blocks.0.attn.w_kctx.down.weight", "blocks.0.attn.w_kctx.up.weight", "blocks.0.attn.k_gain",
              "blocks.0.attn.norm_ctx.weight", "blocks.1.mlp.w3.weight", "norm_f.weight", "lm_head.weight",
              "blocks.0.attn.v_gate.up.bias"):
        assert k in keys, k
    assert not any("rope" in k for k in keys)
    save_checkpoint(str(tmp_path), m, opt, step=13)
    assert os.path.exists(tmp_path / "ckpt_prev.pt")
    ck2 = load_checkpoint(str(tmp_path / "ckpt_latest.pt"))
    assert ck2["step"] == 13 and ck2["model_cfg"]["ctx_mod"] == "mult_res"
    m2 = model_from_checkpoint(ck2, ctx_len=64)
    idx = rand_idx(cfg, 2, 12)
    m.eval()
    assert (m(idx)[0] - m2.eval()(idx)[0]).abs().max() < 1e-6
    assert m2.rope_cos.shape[0] == 64
    # the optimizer entry is a plain torch AdamW state dict
    ref = torch.optim.AdamW([{"params": g["params"], "weight_decay": g["weight_decay"]}
                             for g in decay_groups(m2, 0.1)], lr=1e-3)
    ref.load_state_dict(ck2["optimizer"])
    assert save_persist(str(tmp_path), m, 13, anchor=True).endswith("persist_0000013.pt")


def test_async_writer(tmp_path):
    m = make_model(small_cfg())
    w = AsyncCheckpointWriter()
    w.submit(build_checkpoint(m, step=1), str(tmp_path / "ckpt_latest.pt"))
    w.submit(build_checkpoint(m, step=2), str(tmp_path / "ckpt_latest.pt"))
    w.close()
    assert load_checkpoint(str(tmp_path / "ckpt_latest.pt"))["step"] == 2
    assert load_checkpoint(str(tmp_path / "ckpt_prev.pt"))["step"] == 1


def test_telemetry_runs():
    cfg = small_cfg()
    m = make_model(cfg)
    perturb(m)
    x = rand_idx(cfg, 2, 16)
    fm = torch.zeros(cfg.vocab_size, dtype=torch.bool)
    fm[::3] = True
    scalars, hists = collect_telemetry(m, x, fm)
    assert "telemetry/L0/g_k_mean" in scalars and "telemetry/g_v_mean_all_layers" in scalars
    assert "telemetry/L1/attn_mass_top_decile_1mgk" in scalars and len(hists) > 0
    m.train()
    m(x, targets=x)[1].backward()
    assert "telemetry/L0/gradnorm_ratio_kctx_over_raw" in grad_norm_ratios(m)


def test_corpus_tokeniser_writes_what_the_stream_reads(tmp_path):
    import gzip
    import json
    import numpy as np
    from dual_mod_public_b200.data.packed import memmap_stream
    from dual_mod_public_b200.data.tokenize_corpus import main as tok_main
    docs = [f"document number {i} " + "word " * (5 + i % 7) for i in range(40)]
    with open(tmp_path / "a.jsonl", "w") as f:
        for d in docs[:20]:
            f.write(json.dumps({"text": d}) + "\n")
    with gzip.open(tmp_path / "b.txt.gz", "wt") as f:
        f.write("\n\n".join(docs[20:]) + "\n")
    out, val = str(tmp_path / "train.bin"), str(tmp_path / "val.bin")
    res = tok_main(["--inputs", str(tmp_path / "a.jsonl"), str(tmp_path / "b.txt.gz"), "--out", out, "--val_out", val,
                    "--val_docs", "4", "--vocab_size", "300"])
    assert res["val"][0] == 4 and res["train"][0] == 36
    arr = np.fromfile(out, dtype=np.uint16)
    assert len(arr) == res["train"][1] and json.load(open(out + ".meta.json"))["dtype"] == "uint16"
    first = bytes(int(t) - 3 for t in arr[:len(docs[4].encode())]).decode()
    assert first == docs[4] and arr[len(docs[4].encode())] == 2          # document, then the end-of-sequence id
    two = tok_main(["--inputs", str(tmp_path / "*.jsonl"), str(tmp_path / "*.gz"), "--out", str(tmp_path / "t2.bin"),
                    "--workers", "2", "--vocab_size", "300", "--budget_tokens", "400"])
    a2 = np.fromfile(tmp_path / "t2.bin", dtype=np.uint16)
    n0 = len(docs[0].encode())
    assert 0 < two["train"][1] <= 400 and len(a2) == two["train"][1]
    assert bytes(int(t) - 3 for t in a2[:n0]).decode() == docs[0] and a2[n0] == 2      # input order kept across workers
    blk = next(memmap_stream(out, 16, 2, 0, 1))
    assert blk.shape == (2, 17) and int(blk.max()) < 300
