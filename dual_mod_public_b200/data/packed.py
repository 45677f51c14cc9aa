"""Deterministic packed-token loaders.

A corpus is a flat array of token ids on disk.  It is cut into non-overlapping
chunks and visited epoch by epoch in a permutation seeded by `seed + epoch`, so
any step's batch is a pure function of (seed, step): resume fast-forwards exactly
and the union of the ranks' slices equals the single-process batch.

Reference parity: `PackedLoader` (models/dualmod/data.py:78-131: chunks of T with a
one-token overlap for the targets, `train_batch(step)` / `val_batch(i)`),
`memmap_stream` (lm/train_340m/train_flagship.py:110-130: chunks of T+1, rank
slice `perm[(s*world + rank)*B : ...]`) and `prepare` (data.py:21-75).
Batches are returned as one pinned host block [B, T+1]; the trainer copies it to
the device and splits inputs / targets there.
"""

from __future__ import annotations

import os
import pickle

import numpy as np
import torch


def _pin(t: torch.Tensor) -> torch.Tensor:
    return t.pin_memory() if torch.cuda.is_available() else t


class _Corpus:
    def __init__(self, path, dtype=np.uint16):
        self.arr = np.memmap(path, dtype=dtype, mode="r")

    def rows(self, starts, width):
        return torch.from_numpy(np.stack([self.arr[s:s + width] for s in starts]).astype(np.int64))


class _EpochPerm:
    """Per-epoch chunk permutation, cached for the current epoch."""

    def __init__(self, n, seed):
        self.n, self.seed, self._epoch, self._perm = n, seed, -1, None

    def at(self, epoch, pos):
        if epoch != self._epoch:
            g = torch.Generator().manual_seed(self.seed + epoch)
            self._perm, self._epoch = torch.randperm(self.n, generator=g), epoch
        return int(self._perm[pos])


class PackedLoader:
    """Chunks of T tokens (+1 lookahead) from `<data_dir>/<split>.bin`; `batch_size`
    is the GLOBAL batch, each rank returns its contiguous slice."""

    def __init__(self, data_dir, split, seq_len, batch_size, data_seed=42, device="cpu",
                 rank=0, world_size=1, dtype=np.uint16):
        assert batch_size % world_size == 0, "global batch must divide over the ranks"
        self.corpus = _Corpus(os.path.join(data_dir, f"{split}.bin"), dtype)
        self.T, self.B, self.Bl = seq_len, batch_size, batch_size // world_size
        self.rank, self.world_size, self.device = rank, world_size, device
        self.n_chunks = (len(self.corpus.arr) - 1) // seq_len
        self._perm = _EpochPerm(self.n_chunks, data_seed)

    def _block(self, chunk_ids):
        return _pin(self.corpus.rows([c * self.T for c in chunk_ids], self.T + 1))

    def _xy(self, blk):
        blk = blk.to(self.device, non_blocking=True)
        return blk[:, :-1], blk[:, 1:]

    def train_block(self, step):
        """This rank's [Bl, T+1] host block for `step`."""
        ids = []
        for i in range(self.rank * self.Bl, (self.rank + 1) * self.Bl):
            epoch, pos = divmod(step * self.B + i, self.n_chunks)
            ids.append(self._perm.at(epoch, pos))
        return self._block(ids)

    def train_batch(self, step):
        return self._xy(self.train_block(step))

    def val_block(self, i):
        base = (i * self.B) % max(self.n_chunks - self.B, 1) + self.rank * self.Bl
        return self._block(range(base, base + self.Bl))

    def val_batch(self, i):
        return self._xy(self.val_block(i))


def memmap_stream(path, seq_len, batch_size, rank, world, start_step=0, seed=42, dtype=np.uint16):
    """Endless generator of this rank's [batch_size, T+1] blocks from a flat token
    file cut into chunks of T+1.  `batch_size` is per rank."""
    corpus = _Corpus(path, dtype)
    width = seq_len + 1
    n_chunks = len(corpus.arr) // width
    per_epoch = n_chunks // (batch_size * world)
    assert per_epoch > 0, "corpus smaller than one global batch"
    perm = _EpochPerm(n_chunks, seed)
    step = start_step
    while True:
        epoch, s = divmod(step, per_epoch)
        lo = (s * world + rank) * batch_size
        ids = [perm.at(epoch, lo + j) for j in range(batch_size)]
        yield _pin(corpus.rows([c * width for c in ids], width))
        step += 1


class SyntheticStream:
    """Uniform random token ids of a given shape, a pure function of (seed, rank, step):
    the stand-in corpus of the benchmarks."""

    def __init__(self, vocab_size, seq_len, batch_size, rank=0, seed=1234):
        self.V, self.T, self.B, self.rank, self.seed = vocab_size, seq_len, batch_size, rank, seed

    def block(self, step):
        g = torch.Generator().manual_seed(self.seed + 1000003 * self.rank + step)
        return _pin(torch.randint(0, self.V, (self.B, self.T + 1), generator=g))


def write_corpus(path, tokens, dtype=np.uint16):
    """Write a flat token array (tests, small experiments)."""
    np.asarray(tokens, dtype=dtype).tofile(path)


def prepare(data_dir, num_proc=32, dataset="roneneldan/TinyStories"):
    """Tokenise a text dataset with the GPT-2 BPE into `<split>.bin` (uint16, documents
    separated by the end-of-text token) and write `meta.pkl` with token counts and the
    function-token mask (100 most frequent ids plus ids that decode to no alphanumeric
    character) used by the gate telemetry.  Needs `datasets` and `tiktoken`."""
    from datasets import load_dataset
    import tiktoken

    os.makedirs(data_dir, exist_ok=True)
    enc = tiktoken.get_encoding("gpt2")
    ds = load_dataset(dataset, num_proc=num_proc)

    def tok(example):
        ids = enc.encode_ordinary(example["text"]) + [enc.eot_token]
        return {"ids": ids, "len": len(ids)}

    tokd = ds.map(tok, remove_columns=["text"], num_proc=num_proc)
    counts = np.zeros(enc.n_vocab, dtype=np.int64)
    for split, dset in tokd.items():
        name = "val" if split == "validation" else split
        total = int(np.sum(dset["len"], dtype=np.uint64))
        out = np.memmap(os.path.join(data_dir, f"{name}.bin"), dtype=np.uint16, mode="w+", shape=(total,))
        at, shards = 0, (1024 if split == "train" else 32)
        for i in range(shards):
            part = dset.shard(num_shards=shards, index=i, contiguous=True).with_format("numpy")
            buf = np.concatenate(part["ids"])
            out[at:at + len(buf)] = buf
            at += len(buf)
            if split == "train":
                counts += np.bincount(buf, minlength=enc.n_vocab)
        out.flush()
    function = np.zeros(enc.n_vocab, dtype=bool)
    for tid in range(enc.n_vocab):
        try:
            s = enc.decode([tid])
        except Exception:
            continue
        function[tid] = len(s) > 0 and not any(ch.isalnum() for ch in s)
    top100 = np.argsort(counts)[::-1][:100]
    function[top100] = True
    with open(os.path.join(data_dir, "meta.pkl"), "wb") as f:
        pickle.dump({"vocab_size": enc.n_vocab, "counts": counts, "top100": top100,
                     "function_mask": function}, f)


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser()
    ap.add_argument("--data_dir", default="data")
    ap.add_argument("--num_proc", type=int, default=32)
    a = ap.parse_args()
    prepare(a.data_dir, a.num_proc)
