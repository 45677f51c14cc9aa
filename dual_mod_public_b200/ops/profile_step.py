"""Kernel shares of one training step (or one decode step): which kernels the device time goes to.

  python -m dual_mod_public_b200.ops.profile_step --config 340m     # cell engine, 2 layers of the 340M shape, 32 x 2048 tokens
  python -m dual_mod_public_b200.ops.profile_step --config 1p3b     # wavefront engine K=4, 2 layers d2048 16x128, 16 x 4096
  python -m dual_mod_public_b200.ops.profile_step --config hero     # wavefront engine K=8, 2 layers d2304 36x64 rank 144, 8 x 4096
  python -m dual_mod_public_b200.ops.profile_step --config decode   # one decode step of the 1.3B model, batch 64, position 2300

Runs a two-layer model of the named shape eagerly (no CUDA graphs) under `torch.profiler` with CUDA activity
and prints device time per kernel name, sorted: total, share, launches, mean.  The numbers are for SHARES
only: a run under a profiler is never a timing (time with `bench.py` / `ops/bench_ops.py`).
"""

from __future__ import annotations

import argparse

import torch
from torch.profiler import ProfilerActivity, profile

from ..config import DualModConfig
from ..models import DualModLM

SHAPES = {
    "340m": dict(cfg=dict(d_model=1024, n_heads=16, mlp_hidden_override=2816, max_seq_len=2048), B=32, T=2048, engine="wavescan", K=4),
    "1p3b": dict(cfg=dict(d_model=2048, n_heads=16, mlp_hidden_override=5632, max_seq_len=4096), B=16, T=4096, engine="wave3d", K=4),
    "hero": dict(cfg=dict(d_model=2304, n_heads=36, max_seq_len=4096, ctx_mod="mult_res", gate_rank=144, ctx_rank=144,
                          k_ctx_norm="rms", kmod_vraw_heads=1, v_clamp_tau=150.0), B=8, T=4096, engine="wave3d", K=8),
}


def table(prof, top):
    rows = sorted(((e.self_device_time_total, e.count, e.key) for e in prof.key_averages()
                   if e.self_device_time_total > 0), reverse=True)
    tot = sum(r[0] for r in rows)
    print(f"total device time {tot / 1e3:.1f} ms")
    for t, c, k in rows[:top]:
        print(f"{t / 1e3:9.2f} ms {100 * t / tot:5.1f}% n={c:6d} avg={t / c:8.1f} us  {k[:100]}")
    return rows


def profile_train(name, layers, micro_batch, sweeps, top):
    from ..engines.schedule import uniform_chunks
    from ..engines.wave3d import Wave3DEngine
    from ..engines.wavescan import WaveScanEngine
    sh = SHAPES[name]
    B, T, K = micro_batch or sh["B"], sh["T"], sweeps or sh["K"]
    torch.manual_seed(0)
    cfg = DualModConfig(n_layers=layers, vocab_size=32000, gate_bias_init=0.0, **sh["cfg"])
    m = DualModLM(cfg).cuda()
    if sh["engine"] == "wave3d":
        eng = Wave3DEngine(m, [K], B, T, C=64, autocast_bf16=True, use_graphs=False)
    else:
        eng = WaveScanEngine(m, [uniform_chunks(T, 64, K)], B, T, autocast_bf16=True, use_graphs=False)
    idx = torch.randint(0, 32000, (B, T), device="cuda")
    tgt = torch.randint(0, 32000, (B, T), device="cuda")
    eng.pack()
    for _ in range(2):
        eng.zero_grads()
        eng.train_step(idx, tgt)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        eng.zero_grads()
        eng.train_step(idx, tgt)
        torch.cuda.synchronize()
    return table(prof, top)


def profile_decode(top, batch=64, pos=2300, tape=2560):
    from ..eval.bench_decode import build
    from ..eval.graph_decode import GraphDecoder
    _, m, dt = build("dm_1p3b", "sequential", "cuda:0", tape)
    dec = GraphDecoder(m, batch, tape, dtype=dt)
    for _ in range(2):                                   # the second pass is the profiled state: tape rows live up to `pos`
        dec.pos.fill_(pos)
        dec.pos32.fill_(pos)
        for _ in range(3):
            dec._eager_token()
    dec.pos.fill_(pos)
    dec.pos32.fill_(pos)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        dec._eager_token()
        torch.cuda.synchronize()
    return table(prof, top)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", default="340m", choices=sorted(SHAPES) + ["decode"])
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--micro_batch", type=int, default=0)
    ap.add_argument("--sweeps", type=int, default=0)
    ap.add_argument("--top", type=int, default=36)
    args = ap.parse_args(argv)
    if args.config == "decode":
        return profile_decode(args.top)
    return profile_train(args.config, args.layers, args.micro_batch, args.sweeps, args.top)


if __name__ == "__main__":
    main()
