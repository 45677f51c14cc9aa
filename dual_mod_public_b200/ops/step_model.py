"""Speed-of-light model of one training step of the cell engine: FLOPs and bytes per kernel class, and the
time each class would take at the measured peaks of the machine.

  python -m dual_mod_public_b200.ops.step_model                        # the 340M benchmark shape
  python -m dual_mod_public_b200.ops.step_model --measured_ms 8039     # adds "fraction of the model" for a measured step
  python -m dual_mod_public_b200.ops.step_model --d 2048 --heads 16 --ffn 5632 --T 4096 --B 16 --seqs 256 --K 4

The model counts, per micro-batch of B sequences of T tokens and per layer:

  GEMM          input projection [q k v | gate-x] (5d x d), W_O, the three MLP matrices, and per sweep the packed
                write-law GEMM (4d x d).  Forward once; backward = input gradient + weight gradient (2x forward);
                the layer backward recomputes the projections and the MLP forward; sweep states are kept, so the
                sweeps are not recomputed.  Factored write law: 2 (r_k + r_v + 2 r_g) d per row instead of 4 d^2.
  attention     committed-prefix read of every chunk (T^2 / 2 keys per query overall) and the intra-chunk tail of
                every sweep; backward 2.5x forward.  Tensor-core FLOPs, but these kernels are `mma.sync` code.
  pointwise     bytes moved by the refine chain (forward ~20 B, backward ~68 B per row element and sweep), the
                tail backward (~30 B per row element and sweep, plus the cell-end sums over the sweeps' kept d o:
                ~15 B per sweep + 45 B per cell), norms, RoPE, SwiGLU and the cross-entropy slabs.
  head          unembedding GEMM forward + input / weight gradients.

Times: FLOPs over the sustained bf16 GEMM rate, bytes over the copy bandwidth, both from MEASURED_PEAKS.json
(fallback 1400 TFLOP/s, 6650 GB/s).  The sum is a lower bound of the step with perfect kernels and no launch
gaps; `fraction` = model / measured says how far the measured step is from it.
"""

from __future__ import annotations

import argparse
import json
import os


def peaks():
    p = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops_sustained"] * 1e12, d["hbm_gbs"] * 1e9, "measured"
    return 1400e12, 6650e9, "fallback"


def model(d=1024, heads=16, ffn=2816, vocab=32000, layers=24, T=2048, B=32, seqs=256, c=64, K=4, ranks=(0, 0, 0)):
    """Per optimizer step of `seqs` sequences.  ranks = (r_k, r_v, r_g) of a factored write law, zeros = dense."""
    N = B * T                                               # rows per micro-batch
    micro = seqs // B
    write_law = 4 * d * d if not any(ranks) else 2 * (ranks[0] + ranks[1] + 2 * ranks[2]) * d
    per_row_fwd = 5 * d * d + d * d + 3 * d * ffn          # projections + W_O + MLP
    gemm_layer = 2 * N * (3 * per_row_fwd + per_row_fwd + K * 3 * write_law)       # fwd + 2x bwd + recompute; sweeps fwd + 2x bwd
    head = 2 * N * vocab * d * 3
    dh = d // heads
    att_fwd = 4.0 * B * heads * dh * (T * T / 2 + K * T * c / 2)
    att = att_fwd * 3.5                                      # forward + 2.5x backward
    elem = N * d
    # refine fwd / bwd, tail backward (per sweep: tiles in, d q read-modify-write, dK_in / dV_in out), tail forward;
    # once per cell: the row-scalar sums over the sweeps' kept d o (d v_raw, d k_self, d o_c)
    pointwise = elem * (K * (20 + 68 + 30 + 24) + 15 * K + 45)
    pointwise += elem * (2 * 4 * 4 + 6 * 2 * 3) + N * ffn * 2 * 9    # norms, RoPE, residual adds; SwiGLU fwd + bwd
    ce = N * vocab * 2 * 2
    per_micro = {
        "GEMM (layers)": (layers * gemm_layer, 0.0),
        "GEMM (head)": (head, 0.0),
        "attention": (layers * att, 0.0),
        "pointwise (layers)": (0.0, layers * pointwise),
        "cross-entropy slabs": (0.0, ce),
    }
    return {k: (f * micro, b * micro) for k, (f, b) in per_micro.items()}


def report(rows, measured_ms=0.0):
    flops_s, bytes_s, tag = peaks()
    lines, total = [f"peaks ({tag}): {flops_s / 1e12:.0f} TFLOP/s sustained bf16 GEMM, {bytes_s / 1e9:.0f} GB/s copy"], 0.0
    for name, (f, b) in rows.items():
        t = f / flops_s + b / bytes_s
        total += t
        lines.append(f"{name:22s} {f / 1e12:10.1f} TFLOP {b / 1e9:10.1f} GB {t * 1e3:10.1f} ms")
    lines.append(f"{'model total':22s} {'':10s}       {'':10s}    {total * 1e3:10.1f} ms")
    if measured_ms:
        lines.append(f"measured step {measured_ms:.0f} ms: the model is {total * 1e3 / measured_ms:.1%} of it")
    return lines, total


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    for name, default in (("d", 1024), ("heads", 16), ("ffn", 2816), ("vocab", 32000), ("layers", 24), ("T", 2048),
                          ("B", 32), ("seqs", 256), ("c", 64), ("K", 4)):
        ap.add_argument(f"--{name}", type=int, default=default)
    ap.add_argument("--ranks", default="0,0,0", help="r_k,r_v,r_g of a factored write law")
    ap.add_argument("--measured_ms", type=float, default=0.0)
    a = ap.parse_args(argv)
    rows = model(a.d, a.heads, a.ffn, a.vocab, a.layers, a.T, a.B, a.seqs, a.c, a.K, tuple(int(x) for x in a.ranks.split(",")))
    lines, total = report(rows, a.measured_ms)
    print("\n".join(lines))
    return total


if __name__ == "__main__":
    main()
