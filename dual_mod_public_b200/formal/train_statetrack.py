"""Formal-language trainer: every architecture x every task, eagerly, with length /
depth extrapolation evals.

  python -m dual_mod_public_b200.formal.train_statetrack --task group --group a5 --format tagged \
      --n_ops 16 --arch dualmod --ctx_mod mult_res --n_layers 1 --scale 5m --steps 30 --bsz 16 --lr 4e-4

Prints one `FINAL` line and writes `analysis/statetrack_<tag>_<arch>.json`; `--eval_dump`
also saves `out/statetrack_ckpts/<tag>_<arch>.pt` as {"model", "args"}.  `--engine
wavescan` trains a Dual-Mod model through the chunked engine with an exact schedule
(c = K = --ws_chunk) and hand-computed d_logits instead of the eager scan.

Reference parity: formal_language/harness/train_statetrack.py:239-807 (options,
curricula, loss guard, warm start with vocab growth, looped-K sampling, evaluation
cadence, early stop, dump) and train_statetrack_ws.py (engine path).
"""

from __future__ import annotations

import argparse
import json
import math
import os

import numpy as np
import torch

from . import harness as H
from . import tasks as T
from .tasks import step_rng


def parse(argv=None):
    ap = argparse.ArgumentParser()
    a = ap.add_argument
    a("--task", choices=list(H.TASK_ID), required=True)
    a("--arch", choices=["dualmod", "vanilla", "gdn", "lstm", "looped", "fbt"], required=True)
    a("--scale", choices=list(H.SCALES), default="5m")
    a("--n_layers", type=int, default=0)
    a("--ctx_mod", default="linear")
    a("--deq_sweeps", type=int, default=4)
    a("--nope", action="store_true")
    a("--no_key_mod", action="store_true")
    a("--logn_ref", type=int, default=0)
    a("--steps", type=int, default=1000)
    a("--bsz", type=int, default=64)
    a("--lr", type=float, default=3e-4)
    a("--const_lr", action="store_true")
    a("--wd", type=float, default=0.01)
    a("--seed", type=int, default=0)
    a("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a("--eval_rows", type=int, default=256)
    a("--eval_every", type=int, default=1000)
    a("--gen_factors", default="1,2,4")
    a("--tag_suffix", default="")
    a("--out_root", default=".")
    a("--eval_dump", action="store_true")
    a("--init_from", default=None)
    a("--loss_guard", action="store_true")
    a("--early_stop", type=float, default=0.0)
    a("--snap_interval", type=int, default=0)
    a("--engine", choices=["eager", "wavescan"], default="eager")
    a("--ws_chunk", type=int, default=16)
    a("--no_fused", action="store_true", help="engine path: whole cells under autograd instead of the kernel table")
    a("--tag", default=None, help="run tag (default: built from the task options)")
    a("--eval_bsz", type=int, default=0, help="alias of --eval_rows")
    a("--no_kmod", action="store_true", help="alias of --no_key_mod")
    a("--attn_logn_ref", type=int, default=0, help="alias of --logn_ref")
    # warm starts
    a("--newkey_init", default="none", choices=["none", "mean"],
      help="keyed warm start: key rows beyond the source run's K start from the mean of the trained key rows (+ noise)")
    a("--init_stack", action="store_true", help="warm start from a shallower model: the extra blocks start as identity")
    a("--freeze_body_steps", type=int, default=0, help="warm start: only the embedding / head move for this many steps")
    a("--n_max", type=int, default=0, help="cvp: gates the vocabulary layout has room for (default n_ops x largest factor)")
    a("--cvp_gate", default="xormaj", choices=["xormaj", "copy", "xor2"], help="cvp gate function (control ablations)")
    a("--cvp_leak", type=int, default=0,
      help="cvp curriculum: stage s of cvp_leak + 1 leaks every 2^s-th gate value as an input token, the last stage none")
    # curricula
    a("--curriculum", action="store_true")
    a("--curriculum_start", type=int, default=0)
    a("--curriculum_end", type=int, default=0)
    a("--probe_frac", type=float, default=0.0)
    a("--len_min", type=int, default=0)
    a("--gen_ball", action="store_true")
    a("--K_curriculum", type=int, default=0)
    # looped / fbt
    a("--loop_layers", type=int, default=2)
    a("--loop_k", type=int, default=64)
    a("--loop_k_min", type=int, default=0)
    a("--loop_huginn", action="store_true")
    a("--loop_emb_scale", action="store_true")
    a("--loop_k_mean", type=float, default=32.0)
    a("--loop_bp", type=int, default=8)
    a("--loop_k_per_ops", type=int, default=0)
    a("--eval_loop_ks", default="")
    a("--fbt_sched", default="")
    # task options (defaults = harness.DEFAULTS)
    for k, v in H.DEFAULTS.items():
        if k == "task":
            continue
        if isinstance(v, bool):
            a(f"--{k}", action="store_true")
        else:
            a(f"--{k}", type=type(v), default=v)
    return ap.parse_args(argv)


def run_tag(args):
    if args.tag:
        return args.tag
    t = args.task
    core = {"group": f"{args.group}_{args.format}", "keyed": f"keyed_{args.group}_K{args.K}_D{args.D}",
            "dfa": f"dfa_{args.dfa}", "ca": f"ca{args.ca_rule}_w{args.ca_w}_{args.ca_format}",
            "matinv": f"mi_{args.mi_out}_p{args.mi_p}", "cvp": f"cvp_{args.cvp_format}_m{args.cvp_inputs}"}.get(t, t)
    depth = f"_L{args.n_layers}" if args.n_layers else ""
    return f"{core}_n{args.n_ops}_{args.scale}{depth}_s{args.seed}{args.tag_suffix}"


def word_lengths(mul, n):
    """Word length of every element w.r.t. a small generating set (the first elements that
    generate the group), by breadth-first search on the Cayley graph."""
    gens, reach = [], {0}
    for g in range(1, n):
        if len(reach) == n:
            break
        gens.append(g)
        frontier, reach = [0], {0}
        while frontier:
            nxt = []
            for s in frontier:
                for h in gens:
                    v = int(mul[h, s])
                    if v not in reach:
                        reach.add(v)
                        nxt.append(v)
            frontier = nxt
    dist = np.full(n, -1, dtype=np.int64)
    dist[0], frontier, d = 0, [0], 0
    while frontier:
        d += 1
        nxt = []
        for s in frontier:
            for h in gens:
                v = int(mul[h, s])
                if dist[v] < 0:
                    dist[v] = d
                    nxt.append(v)
        frontier = nxt
    return dist


def load_warm_start(model, path, args=None, n_elem=0):
    """strict=False load of a checkpoint of the same or a smaller problem.  Embedding / head rows grow with
    the vocabulary, keeping the layout: cvp = [ids of inputs and gates | 4 value tokens] (the tail moves to
    the new tail), keyed = [base | keys 0..K_max-1 | 2n group tokens] (likewise, when the source was a keyed
    run), anything else = prefix.  Options of `args`: `newkey_init=mean` (keyed: key rows the source never
    trained start from the mean of its trained key rows + 0.3 sd noise), `init_stack` (blocks the source
    does not have start as identity: zero output projections).
    Reference parity: formal_language/harness/train_statetrack_ws.py:166-215."""
    ck = torch.load(path, map_location="cpu", weights_only=False)
    sd, src_args = dict(ck.get("model", ck)), ck.get("args", {}) or {}
    own = model.state_dict()
    task = getattr(args, "task", None)
    tail = 4 if task == "cvp" else (2 * n_elem if task == "keyed" and "K" in src_args
                                    and src_args.get("task", "keyed") == "keyed" else 0)
    for k, v in list(sd.items()):
        if k not in own or v.shape == own[k].shape:
            continue
        if v.dim() == 2 and v.shape[1] == own[k].shape[1] and v.shape[0] < own[k].shape[0]:
            grown, ns = own[k].clone(), v.shape[0]
            if tail and k in ("tok_emb.weight", "lm_head.weight") and ns > tail:
                grown[:ns - tail] = v[:ns - tail]
                grown[-tail:] = v[-tail:]
            else:
                grown[:ns] = v
            sd[k] = grown
        else:
            del sd[k]
    res = model.load_state_dict(sd, strict=False)
    if args is not None and getattr(args, "newkey_init", "none") == "mean" and task == "keyed":
        K_src, K_max = int(src_args.get("K", 0) or 0), args.K_max or args.K
        if 0 < K_src < K_max:
            with torch.no_grad():
                for name in {"tok_emb.weight", "lm_head.weight"}:
                    W = dict(model.named_parameters()).get(name)
                    if W is None:
                        continue
                    old = W[T.BASE:T.BASE + K_src]
                    mu, sd_ = old.mean(0, keepdim=True), old.std(0, keepdim=True)
                    new = W[T.BASE + K_src:T.BASE + K_max]
                    new.copy_(mu + 0.3 * sd_ * torch.randn_like(new))
    if args is not None and getattr(args, "init_stack", False) and hasattr(model, "blocks"):
        have = {int(k.split(".")[1]) for k in sd if k.startswith("blocks.")}
        with torch.no_grad():
            for i, blk in enumerate(model.blocks):
                if i not in have:
                    blk.attn.wo.weight.zero_()
                    blk.mlp.w2.weight.zero_()
    return res


def freeze_body(model):
    """Zero every gradient but the embedding's and the head's (the first steps of a warm start let new
    vocabulary rows settle before the body moves)."""
    for n, p in model.named_parameters():
        if p.grad is not None and not (n.startswith("tok_emb") or n.startswith("lm_head")):
            p.grad.zero_()


def sample_loop_k(args, kind, n_ops_t):
    if kind == "looped" and args.loop_k_per_ops:
        return max(1, -(-int(n_ops_t) // args.loop_k_per_ops))
    if kind == "looped" and args.loop_huginn:
        tau = math.exp(torch.randn(1).item() * 0.5 + math.log(args.loop_k_mean) - 0.125)
        return int(min(args.loop_k, 1 + torch.poisson(torch.tensor([tau])).item()))
    if kind == "looped" and args.loop_k_min:
        return int(torch.randint(args.loop_k_min, args.loop_k + 1, (1,)))
    if kind == "fbtp":
        ws = [(float(w), int(k)) for w, k in (t.split(":") for t in args.fbt_sched.split(","))]
        return ws[int(torch.multinomial(torch.tensor([w for w, _ in ws]), 1))][1]
    return args.loop_k if kind == "looped" else None


def train_size(args, step):
    """(n_ops for this step, D_override) under the active curriculum."""
    n_ops_t, D_t = args.n_ops, None
    if args.len_min:
        n_ops_t = int(np.random.default_rng(10_000_000 + args.seed * 100_003 + step).integers(args.len_min, args.n_ops + 1))
    if args.curriculum:
        frac = min(1.0, step / max(1, args.curriculum_end or args.steps // 2))
        if args.task == "keyed":
            D_t = max(1, int(round(1 + frac * (args.D - 1))))
        elif args.task == "cvp":
            D_t = frac
        elif args.task == "matinv":
            n0 = args.curriculum_start or 2
            n_ops_t = max(2, int(round(n0 + frac * (args.n_ops - n0))))
        else:
            n_ops_t = max(16, int(16 + frac * (args.n_ops - 16)))
            if args.probe_frac > 0 and (step * args.probe_frac) % 1 > 1 - args.probe_frac:
                n_ops_t = args.n_ops
    return n_ops_t, D_t


def main(argv=None):
    args = parse(argv)
    args.eval_rows = args.eval_bsz or args.eval_rows
    args.no_key_mod = args.no_key_mod or args.no_kmod
    args.logn_ref = args.logn_ref or args.attn_logn_ref
    if args.task == "cvp":
        T.CVP_GATE[0] = args.cvp_gate
    dev = torch.device(args.device)
    torch.manual_seed(args.seed)
    tid = H.TASK_ID[args.task]
    factors = [int(f) for f in args.gen_factors.split(",")]
    args.max_ops = max(args.max_ops, args.n_ops * max(factors), args.n_max)
    mul, n_elem = H.task_tables(args)
    vocab = H.vocab_of(args, n_elem)
    # fixed eval sets (split 0), one per length factor
    evals, max_T = {}, 0
    for f in factors:
        x, tg, m, d = H.make_batch(args, mul, n_elem, step_rng(tid, args.seed, 0, f), args.eval_rows,
                                   args.n_ops * f, evaluating=True)
        evals[f] = (x.to(dev), None if tg is None else tg.to(dev), m.to(dev), d)
        max_T = max(max_T, x.shape[1])
    if args.task == "cvp" and args.cvp_leak:
        max_T += 2 * args.n_ops                               # room for the leaked [id, value] pairs of stage 0
    model, kind = H.build_model(args.arch, vocab, max_T + 8, scale=args.scale, deq_sweeps=args.deq_sweeps,
                                ctx_mod=args.ctx_mod, n_layers=args.n_layers, nope=args.nope,
                                loop_layers=args.loop_layers, loop_k=args.loop_k, key_mod=not args.no_key_mod,
                                logn_ref=args.logn_ref, fbt_sched=args.fbt_sched,
                                loop_emb_scale=args.loop_emb_scale, loop_huginn=args.loop_huginn, loop_bp=args.loop_bp)
    if args.init_from:
        print("warm start:", load_warm_start(model, args.init_from, args, n_elem), flush=True)
    model = model.to(dev)
    n_par = sum(p.numel() for p in model.parameters())
    tag = run_tag(args)
    amp = lambda: torch.autocast(dev.type, dtype=torch.bfloat16, enabled=dev.type == "cuda")
    loop_k = [args.loop_k if kind == "looped" else None]

    engine = None
    if args.engine == "wavescan":
        assert args.arch == "dualmod", "the engine path trains Dual-Mod models"
        from .ws import EngineTrainer
        engine = EngineTrainer(model, args, dev)
    opt = None if engine else torch.optim.AdamW(model.parameters(), lr=args.lr, betas=(0.9, 0.95),
                                                weight_decay=args.wd)

    def predict(x):
        if engine is not None:
            return engine.logits(x)
        with amp():
            return H.logits_of(kind, model, x, K=loop_k[0])

    def acc_eval():
        model.eval()
        if kind in ("looped", "fbtp") and args.eval_loop_ks:
            merged = {}
            for K in [int(k) for k in args.eval_loop_ks.split(",")]:
                loop_k[0] = K
                for f, v in H.evaluate(predict, evals).items():
                    merged[f"K{K}_{f}"] = v
            loop_k[0] = args.loop_k
            firsts = [v for k, v in merged.items() if k.endswith("_1") and isinstance(v, float)]
            merged[1] = merged.get(f"K{args.loop_k}_1", firsts[-1] if firsts else 0.0)
            out = merged
        else:
            out = H.evaluate(predict, evals)
        model.train()
        return out

    wl = word_lengths(mul, n_elem) if (args.gen_ball and args.task == "group") else None
    snapdir = os.path.join(args.out_root, "out", "statetrack_ckpts", "snaps")
    hist, trail = [], []
    model.train()
    for step in range(args.steps):
        lr = args.lr if args.const_lr else H.cosine(step, args.steps, args.lr)
        if wl is not None:
            rad = max(1, int(round(min(1.0, step / max(1, args.steps // 2)) * int(wl.max()))))
            args._op_pool = np.where(wl <= rad)[0]
        n_ops_t, D_t = train_size(args, step)
        args._K_t = None
        if args.task == "keyed" and args.K_curriculum:
            fr = min(1.0, step / max(1, args.curriculum_end or args.steps // 2))
            args._K_t = max(args.K_curriculum, min(args.K, int(round(args.K_curriculum + (args.K - args.K_curriculum) * fr))))
        if args.task == "cvp" and args.cvp_leak:              # leak doubling: stage s leaks every 2^s-th gate
            end = args.curriculum_end or args.steps // 2
            stage = min(args.cvp_leak, int(step * (args.cvp_leak + 1) / max(1, end)))
            args.cvp_leak_every = 0 if stage >= args.cvp_leak else 2 ** stage
        x, tg, m, _ = H.make_batch(args, mul, n_elem, step_rng(tid, args.seed, 1, step), args.bsz, n_ops_t,
                                   D_override=D_t)
        x, m = x.to(dev), m.to(dev)
        tg = None if tg is None else tg.to(dev)
        if engine is not None:
            loss_v = engine.step(x, tg, m, lr, freeze=step < args.freeze_body_steps)
        else:
            for g in opt.param_groups:
                g["lr"] = lr
            loop_k[0] = sample_loop_k(args, kind, n_ops_t)
            with amp():
                logits = H.logits_of(kind, model, x, K=loop_k[0])
            loss = H.masked_loss(logits, x, tg, m)
            loss.backward()
            if step < args.freeze_body_steps:
                freeze_body(model)
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            loss_v = loss.item()
            skip = False
            if args.loss_guard:
                trail = (trail + [loss_v])[-200:]
                med = sorted(trail)[len(trail) // 2]
                skip = len(trail) >= 50 and loss_v > 4 * max(med, 1e-3)
                if skip:
                    print(f"LOSS-GUARD skip step {step}: {loss_v:.3f} vs median {med:.3f}", flush=True)
            if not skip:
                opt.step()
            opt.zero_grad(set_to_none=True)
        if args.snap_interval and (step % args.snap_interval == 0 or step == args.steps - 1):
            os.makedirs(snapdir, exist_ok=True)
            torch.save({"model": model.state_dict(), "step": step, "loss": round(loss_v, 4)},
                       os.path.join(snapdir, f"{tag}_{args.arch}_snap{step:06d}.pt"))
        if step % args.eval_every == 0 or step == args.steps - 1:
            acc = acc_eval()
            hist.append((step, round(loss_v, 4), acc))
            print(f"step {step}: loss {loss_v:.4f} acc {acc}", flush=True)
            main_acc = acc.get(1, 0.0)
            if main_acc > 0.998 and acc.get(max(factors), 0) > 0.998:
                print("early stop: solved incl. max length", flush=True)
                break
            if args.early_stop and step >= 1000 and main_acc >= args.early_stop:
                print(f"EARLY-STOP at step {step}: in-dist acc {main_acc:.4f}", flush=True)
                break
    final = acc_eval()
    os.makedirs(os.path.join(args.out_root, "analysis"), exist_ok=True)
    if args.eval_dump:
        ckdir = os.path.join(args.out_root, "out", "statetrack_ckpts")
        os.makedirs(ckdir, exist_ok=True)
        plain = {k: v for k, v in vars(args).items() if not k.startswith("_")}
        torch.save({"model": model.state_dict(), "args": plain}, os.path.join(ckdir, f"{tag}_{args.arch}.pt"))
    out = os.path.join(args.out_root, "analysis", f"statetrack_{tag}_{args.arch}.json")
    with open(out, "w") as fh:
        json.dump({"task": tag, "arch": args.arch, "params": n_par, "n_ops": args.n_ops, "factors": factors,
                   "layers": args.n_layers, "seed": args.seed,
                   "final": {str(k): v for k, v in final.items()},
                   "hist": [(s, l, {str(k): v for k, v in a.items()}) for s, l, a in hist]}, fh, indent=1)
    print(f"FINAL {tag} {args.arch}: {final} -> {out}", flush=True)
    return final


if __name__ == "__main__":
    main()
