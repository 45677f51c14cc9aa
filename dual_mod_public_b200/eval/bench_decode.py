"""Incremental-decode benchmark and validator for the static-tape graph decoder.

  python -m dual_mod_public_b200.eval.bench_decode                      # 1.3B shape, B=64, 2048 + 512
  python -m dual_mod_public_b200.eval.bench_decode --validate --model tiny
  python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
      -m dual_mod_public_b200.eval.bench_decode                         # data-parallel: one batch per GPU

Benchmark: random-init weights of the named shape, a prompt of uniform random ids prefilled token by token
through the captured decode graph (the tape is recurrent: row t depends on the read at t), then `gen`
greedy tokens.  The generated tokens are timed with CUDA events around the graph replays (max over
ranks); printed per arm: ms per token, tokens/s (whole job) and the prefill time.  Arms: Dual-Mod, and
the same-shape Transformer++ control (`attn_mode="vanilla"`: `refine_kv` returns the raw key/value, so
the step is a plain KV-cache decoder step).

Validator (`--validate`): graph decode against the eager `decode_step` loop and against one
teacher-forced forward of the exact scan on the same tokens: arg-max agreement and max |delta logit|.

Reference parity: lm/eval/validate_graph_decode.py:40-97 (validation protocol, per-token latency print),
lm/eval/graph_decode.py:97-125 (greedy generate).
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from ..config import DualModConfig, preset
from ..models import DualModLM
from .graph_decode import GraphDecoder


def _dist():
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    return rank, world, local


def build(name, mode, device, max_len):
    cfg = preset(name, max_seq_len=max_len) if name != "tiny" else DualModConfig(
        d_model=128, n_layers=2, n_heads=2, vocab_size=256, max_seq_len=max_len, gate_bias_init=0.0)
    cfg.attn_mode = mode
    torch.manual_seed(1337)
    dt = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
    return cfg, DualModLM(cfg).to(device=device).eval(), dt


def build_reference(name, mode, device, max_len):
    """The unmodified reference model + its GraphDecoder class from `baseline/_ref` (same shape, random init)."""
    import sys
    ref = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "lm", "eval")):
        raise FileNotFoundError("baseline/_ref is not installed")
    sys.path.insert(0, ref)
    from dataclasses import fields

    from lm.eval.graph_decode import GraphDecoder as RefDecoder
    from models.dualmod.config import DualModConfig as RefConfig
    from models.dualmod.model import DualModLM as RefLM
    mine = preset(name, max_seq_len=max_len).to_dict()
    keep = {f.name for f in fields(RefConfig)}
    cfg = RefConfig(**{k: v for k, v in mine.items() if k in keep})
    cfg.attn_mode = mode
    torch.manual_seed(1337)
    return cfg, RefLM(cfg).to(device).eval(), RefDecoder


def time_decode(model, B, prompt_len, gen, dtype, device, rank, world, decoder_cls=None):
    dec = (decoder_cls or GraphDecoder)(model, B, prompt_len + gen, dtype=dtype).capture()
    g = torch.Generator().manual_seed(99 + rank)
    prompt = torch.randint(0, model.cfg.vocab_size, (B, prompt_len), generator=g).to(device)
    cuda = torch.device(device).type == "cuda"
    ev = lambda: torch.cuda.Event(enable_timing=True)
    sync = (lambda: torch.cuda.synchronize()) if cuda else (lambda: None)
    dec.reset()
    sync()
    if cuda:
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
    import time
    t0 = time.perf_counter()
    for p in range(prompt_len):                          # token by token: the tape is recurrent
        dec.tok.copy_(prompt[:, p:p + 1])
        dec.step()
    if cuda:
        e1.record()
    t1 = time.perf_counter()
    for _ in range(gen):
        dec.tok.copy_(dec.next)
        dec.step()
    if cuda:
        e2.record()
    sync()
    t2 = time.perf_counter()
    pre_ms, gen_ms = (e0.elapsed_time(e1), e1.elapsed_time(e2)) if cuda else ((t1 - t0) * 1e3, (t2 - t1) * 1e3)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([pre_ms, gen_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pre_ms, gen_ms = t.tolist()
    return {"ms_per_token": gen_ms / gen, "tokens_per_s": world * B * gen / (gen_ms / 1e3),
            "prefill_ms": pre_ms, "prefill_tokens_per_s": world * B * prompt_len / (pre_ms / 1e3),
            "kernel_read": bool(getattr(dec, "use_kernel", False)), "graph": dec.graph is not None}


@torch.no_grad()
def validate(model, B, L, dtype, device, toks=None, gen=16):
    """Graph decode against eager `decode_step` and against teacher forcing over L positions: arg-max agreement
    and max |dlogit| for both, the drift profile (max |dlogit| vs eager per position octile), and how many of the
    B greedy continuations of `gen` tokens are identical between the graph and the eager decoder.  `accept`
    applies the reference validator's bar (agreement >= 99.9 %, max |dlogit| < 0.1, at least B - 1 identical
    continuations; lm/eval/validate_graph_decode.py:97).  toks: [B, L] prompt ids (default: uniform random)."""
    cfg = model.cfg
    if toks is None:
        g = torch.Generator().manual_seed(5)
        toks = torch.randint(0, cfg.vocab_size, (B, L), generator=g)
    toks = toks[:B, :L].to(device)
    dec = GraphDecoder(model, B, L, dtype=dtype).capture()
    dec.reset()
    lg_graph = []
    for t in range(L):
        dec.tok.copy_(toks[:, t:t + 1])
        dec.step()
        lg_graph.append(dec.logits[:, 0].float().clone())
    lg_graph = torch.stack(lg_graph, 1)
    amp = torch.device(device).type == "cuda"
    with torch.autocast(torch.device(device).type, dtype=torch.bfloat16, enabled=amp):
        caches, lg_eager = model.decode_init(), []
        for t in range(L):
            lg_eager.append(model.decode_step(toks[:, t:t + 1], t, caches)[:, 0].float())
        mode = cfg.attn_mode
        if mode != "vanilla":
            cfg.attn_mode = "sequential"
        lg_tf = model(toks)[0].float()
        cfg.attn_mode = mode
    out = {"agree_tf": (lg_graph.argmax(-1) == lg_tf.argmax(-1)).float().mean().item(),
           "max_dlogit_tf": (lg_graph - lg_tf).abs().max().item()}
    if lg_eager:
        lg_eager = torch.stack(lg_eager, 1)
        diff = (lg_graph - lg_eager).abs().amax(dim=(0, 2))                      # per position
        out.update(agree_eager=(lg_graph.argmax(-1) == lg_eager.argmax(-1)).float().mean().item(),
                   max_dlogit_eager=diff.max().item(),
                   drift_by_octile=[round(c.max().item(), 5) for c in diff.chunk(min(8, L))])
        # greedy continuations: graph decoder vs eager decode_step from the same prompt
        plen = max(1, L - gen)
        g_graph, k = dec.generate(toks[:, :plen], min(gen, L - plen))
        with torch.autocast(torch.device(device).type, dtype=torch.bfloat16, enabled=amp):
            caches, lg = model.decode_init(), None
            for t in range(plen):
                lg = model.decode_step(toks[:, t:t + 1], t, caches)
            g_eager = []
            for j in range(k):
                nxt = lg[:, -1].argmax(-1, keepdim=True)
                g_eager.append(nxt)
                if j < k - 1:
                    lg = model.decode_step(nxt, plen + j, caches)
        same = int((g_graph.to(device) == torch.cat(g_eager, 1)).all(dim=1).sum()) if k else B
        out.update(identical_continuations=same, continuations=B,
                   accept=bool(out["agree_eager"] >= 0.999 and out["max_dlogit_eager"] < 0.1 and same >= B - 1))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dm_1p3b", help="preset name (dm_1p3b, dm_340m, ...) or 'tiny'")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--gen", type=int, default=512)
    ap.add_argument("--validate", action="store_true")
    ap.add_argument("--ckpt", default="", help="validate / time the model of this checkpoint instead of a random-init preset")
    ap.add_argument("--tokens_bin", default="", help="--validate: prompts from this flat token file instead of random ids")
    ap.add_argument("--val_len", type=int, default=96, help="--validate: positions compared")
    ap.add_argument("--device", default="")
    ap.add_argument("--arms", default="dualmod,vanilla")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"],
                    help="reference: the unmodified reference model and GraphDecoder from baseline/_ref")
    args = ap.parse_args(argv)
    rank, world, local = _dist()
    device = args.device or (f"cuda:{local}" if torch.cuda.is_available() else "cpu")
    out = {"metric": "decode_ms_per_token", "model": args.model, "batch_per_gpu": args.batch, "n_gpus": world,
           "prompt": args.prompt, "gen": args.gen, "dtype": "bf16" if "cuda" in device else "fp32",
           "data": "uniform random prompt ids, random-init weights"}
    out["impl"] = args.impl
    for arm in args.arms.split(","):
        mode = "vanilla" if arm == "vanilla" else "sequential"
        dec_cls = None
        if args.impl == "reference":
            try:
                cfg, model, dec_cls = build_reference(args.model, mode, device, args.prompt + args.gen)
                dt = torch.bfloat16
            except Exception as e:
                out = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:300]}
                break
        elif args.ckpt:
            from ..utils.checkpoint import load_checkpoint, model_from_checkpoint
            model = model_from_checkpoint(load_checkpoint(args.ckpt), device=device, ctx_len=args.prompt + args.gen)
            cfg, dt = model.cfg, (torch.bfloat16 if "cuda" in device else torch.float32)
            if mode == "vanilla" and cfg.attn_mode != "vanilla":
                continue                                     # a checkpoint has one operator: no control arm
            out["model"] = args.ckpt
        else:
            cfg, model, dt = build(args.model, mode, device, args.prompt + args.gen)
        if args.validate:
            toks = None
            if args.tokens_bin:
                import numpy as np
                n, L = min(args.batch, 4), min(args.prompt + args.gen, args.val_len)
                arr = np.fromfile(args.tokens_bin, dtype=np.uint16, count=n * L).astype(np.int64)
                toks = torch.from_numpy(arr).view(n, L) % cfg.vocab_size
            out[arm] = validate(model, min(args.batch, 4), min(args.prompt + args.gen, args.val_len), dt, device, toks)
        else:
            out[arm] = {k: (round(v, 4) if isinstance(v, float) else v)
                        for k, v in time_decode(model, args.batch, args.prompt, args.gen, dt, device, rank, world, dec_cls).items()}
        del model
        if "cuda" in device:
            torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return out


if __name__ == "__main__":
    main()
