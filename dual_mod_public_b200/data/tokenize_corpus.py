"""Tokenise text files into the flat token files the language-model trainers read.

  python -m dual_mod_public_b200.data.tokenize_corpus --inputs 'raw/*.jsonl' --tokenizer data/llama2_tok \\
      --out data/train.bin --val_out data/val.bin --val_docs 2000 --budget_tokens 15.5e9 --workers 32

Inputs: `.jsonl` (one JSON object per line, text under `--text_key`), `.txt` (one document per blank-line
separated paragraph block, or per line with `--line_docs`), optionally gzip-compressed.  Every document is
encoded without special tokens and followed by the tokenizer's end-of-sequence id; ids are written as uint16
(vocabularies below 65 536) or uint32.  The first `--val_docs` documents go to `--val_out`, the rest to `--out`,
stopping at `--budget_tokens`.  Files are processed by `--workers` processes in input order, so the output is a
pure function of the inputs.  A `<out>.meta.json` beside each file records the counts and the dtype.

`memmap_stream(path, T, batch, rank, world, ...)` then cuts the file into rows of T + 1 tokens.
"""

from __future__ import annotations

import argparse
import glob
import gzip
import json
import os
from concurrent.futures import ProcessPoolExecutor

import numpy as np


def documents(path, text_key="text", line_docs=False):
    """Documents (strings) of one input file."""
    opener = gzip.open if path.endswith(".gz") else open
    base = path[:-3] if path.endswith(".gz") else path
    with opener(path, "rt", encoding="utf-8") as f:
        if base.endswith(".jsonl"):
            for line in f:
                if line.strip():
                    text = json.loads(line).get(text_key, "")
                    if text:
                        yield text
        elif line_docs:
            for line in f:
                if line.strip():
                    yield line.rstrip("\n")
        else:
            block = []
            for line in f:
                if line.strip():
                    block.append(line.rstrip("\n"))
                elif block:
                    yield "\n".join(block)
                    block = []
            if block:
                yield "\n".join(block)


def _load_tokenizer(spec):
    from ..eval.lm_eval_adapter import load_tokenizer
    return load_tokenizer(spec)


def encode_file(job):
    """(path, tokenizer spec, text key, line_docs) -> list of int arrays, one per document (EOS appended)."""
    path, spec, text_key, line_docs = job
    tok = _load_tokenizer(spec)
    eos = tok.eos_token_id if tok.eos_token_id is not None else 2
    return [np.asarray(list(tok.encode(doc, add_special_tokens=False)) + [eos], dtype=np.int64)
            for doc in documents(path, text_key, line_docs)]


def run(inputs, tokenizer, out, val_out="", val_docs=0, budget_tokens=0, workers=1, text_key="text", line_docs=False,
        vocab_size=0):
    files = sorted(f for pat in inputs for f in glob.glob(pat))
    if not files:
        raise FileNotFoundError(f"no input matches {inputs}")
    tok = _load_tokenizer(tokenizer)
    vocab = vocab_size or getattr(tok, "vocab_size", None) or 65536
    dtype = np.uint16 if vocab <= 65536 else np.uint32
    jobs = [(f, tokenizer, text_key, line_docs) for f in files]
    sinks = {"train": open(out, "wb")}
    if val_out and val_docs:
        sinks["val"] = open(val_out, "wb")
    counts = {"train": [0, 0], "val": [0, 0]}                      # documents, tokens
    seen, done = 0, False

    def consume(docs):
        nonlocal seen, done
        for ids in docs:
            split = "val" if "val" in sinks and seen < val_docs else "train"
            seen += 1
            if split == "train" and budget_tokens and counts["train"][1] + len(ids) > budget_tokens:
                done = True
                return
            if ids.max(initial=0) >= np.iinfo(dtype).max + 1:
                raise ValueError(f"token id {int(ids.max())} does not fit {dtype.__name__}")
            sinks[split].write(ids.astype(dtype).tobytes())
            counts[split][0] += 1
            counts[split][1] += len(ids)

    if workers > 1:
        import multiprocessing
        with ProcessPoolExecutor(max_workers=workers, mp_context=multiprocessing.get_context("spawn")) as ex:
            for docs in ex.map(encode_file, jobs):                  # results come back in input order
                consume(docs)
                if done:
                    break
    else:
        for job in jobs:
            consume(encode_file(job))
            if done:
                break
    for name, fh in sinks.items():
        fh.close()
        path = out if name == "train" else val_out
        with open(path + ".meta.json", "w") as mf:
            json.dump({"documents": counts[name][0], "tokens": counts[name][1], "dtype": np.dtype(dtype).name,
                       "tokenizer": tokenizer if isinstance(tokenizer, str) else type(tokenizer).__name__,
                       "files": len(files)}, mf, indent=1)
    return {k: tuple(v) for k, v in counts.items()}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--inputs", nargs="+", required=True, help="files or glob patterns")
    ap.add_argument("--tokenizer", default="bytes", help="tokenizer folder / hub name, or 'bytes'")
    ap.add_argument("--out", required=True)
    ap.add_argument("--val_out", default="")
    ap.add_argument("--val_docs", type=int, default=0)
    ap.add_argument("--budget_tokens", type=float, default=0)
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--text_key", default="text")
    ap.add_argument("--line_docs", action="store_true")
    ap.add_argument("--vocab_size", type=int, default=0, help="override the tokenizer's (decides uint16 / uint32)")
    a = ap.parse_args(argv)
    res = run(a.inputs, a.tokenizer, a.out, a.val_out, a.val_docs, int(a.budget_tokens), a.workers, a.text_key,
              a.line_docs, a.vocab_size)
    print(json.dumps(res))
    return res


if __name__ == "__main__":
    main()
