"""Command-line driver of the evaluation harness on a checkpoint.

  python -m dual_mod_public_b200.eval.run_lm_eval --ckpt out/run/ckpt_latest.pt \\
      --tasks piqa,hellaswag,winogrande,arc_easy,arc_challenge,lambada_openai,wikitext
  ... --engine_K 24 --T_eval 2048            # score and generate through the wavefront engine at K = 24
  ... --tasks jrt_fda --local_data data/fda.jsonl --num_shards 4 --shard_id 1     # local recall task, sharded
  ... --tasks niah_single_1 --ruler_root data/ruler --ruler_lengths 1024,2048

Harness tasks need the `lm_eval` package; the recall (`jrt_*`) and needle (`niah_*`) tasks of
`recall_tasks.py` also run without it from local jsonl files.  Under torchrun every rank builds the model
and the harness shards the requests by rank.  Writes `lmeval_<run>_<step>_<hash>[_<tag>].json` (results,
task list, engine K) into `--out_dir`, and one `*_TEXT.jsonl` per local task with the generations.

`--backend hf` evaluates a HuggingFace causal LM through the harness's own model class with the same task
glue (the control arm).

Reference parity: lm/eval/run_lm_eval.py:1-202, lm/eval/run_hf_eval.py:1-78.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import os


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    a = ap.add_argument
    a("--ckpt", default="")
    a("--tasks", required=True)
    a("--backend", default="dualmod", choices=["dualmod", "hf"])
    a("--model_path", default="", help="--backend hf: the model folder")
    a("--batch_rows", type=int, default=16)
    a("--limit", type=int, default=None)
    a("--device", default="")
    a("--tokenizer", default="bytes", help="tokenizer folder, or 'bytes'")
    a("--num_fewshot", type=int, default=None)
    a("--ctx_len", type=int, default=None, help="evaluate at a longer context than trained (RoPE tables rebuilt)")
    a("--engine_K", type=int, default=0, help="> 0: likelihood and generation through the training engine at this K")
    a("--engine", default="wave3d", choices=["wave3d", "wavescan"])
    a("--T_eval", type=int, default=2048)
    a("--engine_kwargs", default="{}")
    a("--gen_rows", type=int, default=4)
    a("--ruler_root", default="")
    a("--ruler_lengths", default="1024,2048,4096,8192")
    a("--local_data", default="", help="jsonl of a local recall task (one task per call)")
    a("--num_shards", type=int, default=1)
    a("--shard_id", type=int, default=0)
    a("--tag", default="")
    a("--out_dir", default="analysis")
    return ap.parse_args(argv)


def build_lm(args):
    from .lm_eval_adapter import DualModEval, WavefrontEval
    common = dict(tokenizer=args.tokenizer, batch_rows=args.batch_rows, device=args.device or None,
                  ctx_len=args.ctx_len)
    if args.engine_K:
        return WavefrontEval(args.ckpt, args.engine_K, T_eval=args.T_eval, engine=args.engine, gen_rows=args.gen_rows,
                             engine_kwargs=json.loads(args.engine_kwargs), **common)
    return DualModEval(args.ckpt, max_length=args.ctx_len or args.T_eval, **common)


def out_name(args, step):
    run = os.path.basename(os.path.dirname(os.path.abspath(args.ckpt or args.model_path))) or "run"
    h = hashlib.md5(f"{args.tasks}:{args.num_fewshot}:{args.ruler_lengths}:{args.ctx_len}:{args.engine_K}".encode()
                    ).hexdigest()[:6]
    tag = f"_{args.tag}" if args.tag else ""
    sh = f"_s{args.shard_id}of{args.num_shards}" if args.num_shards > 1 else ""
    return f"lmeval_{run}_{step}_{h}{tag}{sh}"


def main(argv=None):
    args = parse_args(argv)
    from . import recall_tasks as R
    tasks = [t for t in args.tasks.split(",") if t]
    os.makedirs(args.out_dir, exist_ok=True)
    spec = f"{args.shard_id}/{args.num_shards}" if args.num_shards > 1 else ""
    results, step = {}, 0
    if args.backend == "hf":
        import lm_eval
        from lm_eval.models.huggingface import HFLM
        lm = HFLM(pretrained=args.model_path, device=args.device or "cuda:0", batch_size="auto",
                  max_length=args.ctx_len or 8448)
        results = lm_eval.simple_evaluate(model=lm, tasks=tasks, num_fewshot=args.num_fewshot, limit=args.limit)["results"]
    else:
        lm = build_lm(args)
        from ..utils.checkpoint import load_checkpoint
        step = int(load_checkpoint(args.ckpt).get("step", 0))
        base = os.path.join(args.out_dir, out_name(args, step))
        local = [t for t in tasks if (t.startswith("jrt_") and args.local_data) or (t.startswith("niah_") and args.ruler_root)]
        for t in local:
            if t.startswith("jrt_"):
                docs = R.load_jsonl(args.local_data)[:args.limit]
                results[t] = R.run_recall(lm, t[4:], docs, lm.tok, shard_spec=spec, dump=f"{base}_{t}_TEXT.jsonl")
            else:
                docs = R.load_needles(args.ruler_root, t, [int(x) for x in args.ruler_lengths.split(",")])
                results[t] = R.run_needles(lm, docs[:args.limit], shard_spec=spec)
        rest = [t for t in tasks if t not in local]
        if rest:
            import lm_eval
            results.update(lm_eval.simple_evaluate(model=lm, tasks=rest, num_fewshot=args.num_fewshot,
                                                   limit=args.limit)["results"])
    rank = int(os.environ.get("RANK", 0))
    if rank == 0:
        path = os.path.join(args.out_dir, out_name(args, step) + ".json")
        with open(path, "w") as f:
            json.dump({"ckpt": args.ckpt or args.model_path, "tasks": args.tasks, "num_fewshot": args.num_fewshot,
                       "engine_K": args.engine_K or None, "ctx_len": args.ctx_len, "results": results}, f, indent=1,
                      default=str)
        print(json.dumps(results, indent=1, default=str))
        print("wrote", path)
    return results


if __name__ == "__main__":
    main()
