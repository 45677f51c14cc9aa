"""Evaluation-harness adapter: a checkpoint behind the `lm_eval` model interface.

  from dual_mod_public_b200.eval.lm_eval_adapter import DualModEval
  lm = DualModEval("out/run/ckpt_latest.pt", tokenizer="data/llama2_tok")
  lm.loglikelihood([("The capital of France is", " Paris")])        # [(logprob, is_greedy)]
  lm.generate_until([("Q: 2+2=\nA:", {"until": ["\n"], "max_gen_toks": 8})])

`DualModEval` subclasses `lm_eval.api.model.LM` when that package is importable (then
`lm_eval.simple_evaluate(model=lm, tasks=[...])` works, see `run_lm_eval`), and is a plain class with
the same three request methods otherwise.  Requests are `(context, continuation)` / `(context, gen_kwargs)`
tuples or objects with `.args`.

  likelihood   exact operator on whole sequences, batched in length buckets (lengths rounded up to
               `EVAL_LEN_QUANT`, default 64, so batches share shapes); `engine_K` scores through the cell
               engine at K sweeps instead of the eager scan (K = chunk is exact and much faster on a GPU)
  generation   greedy through the static-tape `GraphDecoder` (one graph launch per token) on a GPU,
               through `decode_step` otherwise; prompts longer than the context keep head + tail
               (`GEN_TRUNC=head`) or the tail
  cache        `EVAL_GEN_CACHE=<jsonl>`: finished generations are appended and served on restart;
               `EVAL_CACHE_ONLY=1` answers uncached requests with "<UNCACHED>"
  ranks        under torchrun the harness shards requests by `rank / world_size` (exposed as properties)

Reference parity: lm/eval/lm_eval_adapter.py:69-781 (`DualModEval`: likelihood :244-273, generation
:361-602, cache :117-140, distributed hooks :185-210; `Wave3DEval`: scoring through the engine at K
:605-781), lm/eval/run_lm_eval.py (driver).
"""

from __future__ import annotations

import hashlib
import json
import os

import torch
import torch.nn.functional as F

from ..utils.checkpoint import load_checkpoint, model_from_checkpoint

try:                                                     # optional dependency
    from lm_eval.api.model import LM as _Base
except Exception:                                        # the harness is not installed: same methods, no base
    _Base = object


class ByteTokenizer:
    """Fallback tokenizer: UTF-8 bytes shifted by 3 (0 pad, 1 bos, 2 eos).  Needs vocab >= 259."""
    bos_token_id, eos_token_id = 1, 2

    def encode(self, text, add_special_tokens=False):
        return [b + 3 for b in text.encode("utf-8")]

    def decode(self, ids, skip_special_tokens=True):
        return bytes(i - 3 for i in ids if i >= 3).decode("utf-8", errors="replace")


def load_tokenizer(spec):
    if spec is None or spec == "bytes":
        return ByteTokenizer()
    if hasattr(spec, "encode"):
        return spec
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(spec)


def _args(req):
    return req.args if hasattr(req, "args") else req


def trunc_keep_head(toks, cap):
    """Keep the head and a short tail when a prompt exceeds the context (answers of recall documents
    sit near the start); plain tail truncation unless GEN_TRUNC=head."""
    if len(toks) <= cap:
        return toks
    if os.environ.get("GEN_TRUNC", "tail") != "head":
        return toks[-cap:]
    keep_tail = min(128, cap // 4)
    return toks[:cap - keep_tail] + toks[-keep_tail:]


class DualModEval(_Base):
    def __init__(self, ckpt, tokenizer=None, batch_rows=16, device=None, max_length=2048, ctx_len=None,
                 engine_K=0, engine_chunk=64, model=None, gen_rows=8):
        if _Base is not object:
            super().__init__()
        self.dev = device or ("cuda" if torch.cuda.is_available() else "cpu")
        if model is None:
            ck = load_checkpoint(ckpt)
            self.arch = os.environ.get("EVAL_ARCH") or ck.get("arch", "dualmod")
            self.ckpt_engine_kwargs = ck.get("engine_kwargs")
            model = model_from_checkpoint(ck, device=self.dev, ctx_len=ctx_len)
        else:
            self.arch, self.ckpt_engine_kwargs = "dualmod", None
            model = model.to(self.dev)
        self.model = model.eval()
        cfg = self.model.cfg
        if cfg.attn_mode not in ("vanilla", "static"):
            cfg.attn_mode = "sequential"
        self.max_length = min(ctx_len or max_length, cfg.max_seq_len)
        self.tok = load_tokenizer(tokenizer)
        self.bos = self.tok.bos_token_id if self.tok.bos_token_id is not None else 1
        self.batch_rows, self.engine_K, self.engine_chunk = batch_rows, engine_K, engine_chunk
        self.gen_rows = gen_rows
        self.len_quant = int(os.environ.get("EVAL_LEN_QUANT", "64"))
        self._engines = {}
        self._rank, self._world_size = 0, 1
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            self._rank, self._world_size = dist.get_rank(), dist.get_world_size()
        self._gcache_path = os.environ.get("EVAL_GEN_CACHE", "")
        self._gcache_only = os.environ.get("EVAL_CACHE_ONLY", "0") == "1"
        self._gcache = {}
        if self._gcache_path and os.path.exists(self._gcache_path):
            for line in open(self._gcache_path):
                try:
                    d = json.loads(line)
                    self._gcache[d["k"]] = d["g"]
                except ValueError:
                    pass

    # ---- harness hooks ----------------------------------------------------------------------------
    @property
    def rank(self):
        return self._rank

    @property
    def world_size(self):
        return self._world_size

    @property
    def eot_token_id(self):
        return self.tok.eos_token_id

    def tok_encode(self, s):
        return list(self.tok.encode(s, add_special_tokens=False))

    # what the harness calls between ranks when world_size > 1 (each a no-op on one rank)
    def all_gather(self, tensor):
        import torch.distributed as dist
        if self._world_size == 1:
            return tensor.unsqueeze(0)
        out = [torch.zeros_like(tensor) for _ in range(self._world_size)]
        dist.all_gather(out, tensor)
        return torch.stack(out)

    def gather_object(self, obj, dst=0):
        import torch.distributed as dist
        if self._world_size == 1:
            return [obj]
        out = [None] * self._world_size
        dist.all_gather_object(out, obj)
        return out if self._rank == dst else None

    def barrier(self):
        import torch.distributed as dist
        if self._world_size > 1:
            dist.barrier()

    # ---- scoring -----------------------------------------------------------------------------------
    def _amp(self):
        t = torch.device(self.dev).type
        return torch.autocast(t, dtype=torch.bfloat16, enabled=t == "cuda")

    @torch.no_grad()
    def _logits(self, x):
        """x [B, L] -> logits [B, L, V] by the exact operator (or the engine at `engine_K`)."""
        B, L = x.shape
        cfg = self.model.cfg
        use_engine = self.engine_K > 0 and cfg.attn_mode != "vanilla" and L % self.engine_chunk == 0
        if not use_engine:
            with self._amp():
                return self.model(x)[0].float()
        from ..engines.schedule import uniform_chunks
        from ..engines.wavescan import WaveScanEngine
        key = (B, L)
        if key not in self._engines:
            c = self.engine_chunk
            self._engines[key] = WaveScanEngine(self.model, [uniform_chunks(L, c, min(c, self.engine_K))], B, L,
                                                device=self.dev, keep_logits=True,
                                                autocast_bf16=torch.device(self.dev).type == "cuda")
            self._engines[key].pack()
        eng = self._engines[key]
        eng.forward(x)
        return eng.logits.float()

    def _score_rows(self, rows):
        """rows: list of (tokens, n_continuation).  Returns [(sum logprob of the continuation, greedy?)] in
        the given order; batches are formed inside length buckets."""
        order = sorted(range(len(rows)), key=lambda i: len(rows[i][0]))
        out = [None] * len(rows)
        q = self.len_quant
        for b0 in range(0, len(order), self.batch_rows):
            ids = order[b0:b0 + self.batch_rows]
            L = max(len(rows[i][0]) for i in ids)
            L = min(self.max_length, -(-L // q) * q)
            x = torch.zeros(len(ids), L, dtype=torch.long)
            for r, i in enumerate(ids):
                t = rows[i][0][-L:]
                x[r, :len(t)] = torch.tensor(t)
            logp = F.log_softmax(self._logits(x.to(self.dev)), dim=-1).cpu()
            for r, i in enumerate(ids):
                toks, n_c = rows[i]
                toks = toks[-L:]
                n_c = min(n_c, len(toks) - 1)
                pos = torch.arange(len(toks) - n_c - 1, len(toks) - 1)
                tgt = torch.tensor(toks[len(toks) - n_c:])
                lp = logp[r, pos]
                out[i] = (lp.gather(1, tgt[:, None]).sum().item(), bool((lp.argmax(-1) == tgt).all()))
        return out

    def loglikelihood(self, requests):
        rows = []
        for req in requests:
            ctx, cont = _args(req)[:2]
            c, k = ([self.bos] + self.tok_encode(ctx)) if ctx else [self.bos], self.tok_encode(cont)
            rows.append((c + k, len(k)))
        return self._score_rows(rows)

    def loglikelihood_rolling(self, requests):
        """Whole-document log-likelihood in windows of the context length (disjoint windows, each
        conditioned on BOS only)."""
        out = []
        for req in requests:
            toks = self.tok_encode(_args(req)[0])
            tot, W = 0.0, self.max_length - 1
            rows = [([self.bos] + toks[s:s + W], len(toks[s:s + W])) for s in range(0, max(1, len(toks)), W)]
            tot = sum(lp for lp, _ in self._score_rows(rows))
            out.append(tot)
        return out

    # ---- generation ---------------------------------------------------------------------------------
    def _gen_key(self, prompt, until, max_new):
        return hashlib.md5(json.dumps([prompt, until, max_new]).encode()).hexdigest()

    def _cut(self, ids, stop_strs):
        """Token ids of one row -> text, cut at the end-of-sequence id and at the first stop string."""
        eos = self.tok.eos_token_id
        if eos in ids:
            ids = ids[:ids.index(eos)]
        text = self.tok.decode(ids)
        for s in stop_strs:
            if s in text:
                text = text[:text.index(s)]
        return text

    @torch.no_grad()
    def _greedy_batch(self, prompts, max_new, stop_strs):
        """Greedy continuations of prompts of ONE length (so a single position serves the whole batch) ->
        texts.  On a GPU: the static-tape `GraphDecoder` at a fixed batch of `gen_rows` rows (short batches are
        filled with copies of the last row, so one recorded graph serves every batch); on CPU: `decode_step`.
        The budget is capped at half the context, so a short context still keeps a prompt."""
        n, eos = len(prompts), self.tok.eos_token_id
        x = torch.tensor(prompts, dtype=torch.long, device=self.dev)
        plen = x.shape[1]

        def finished(rows_cpu):
            return torch.tensor([eos in r or any(s in self.tok.decode(r) for s in stop_strs)
                                 for r in rows_cpu.tolist()])

        if torch.device(self.dev).type == "cuda":
            from .graph_decode import GraphDecoder
            rows = max(self.gen_rows, n)
            P = min(-(-(plen + max_new) // 256) * 256, self.model.cfg.max_seq_len)
            key = ("dec", rows, P)
            if key not in self._engines:
                self._engines[key] = GraphDecoder(self.model, rows, P).capture()
            if rows > n:
                x = torch.cat((x, x[-1:].expand(rows - n, plen)), dim=0)
            gen, k = self._engines[key].generate(x, max_new, eos_id=eos, stop_fn=finished)
            toks = gen[:n, :k].tolist()
        else:
            caches, logits = self.model.decode_init(), None
            for t in range(plen):
                logits = self.model.decode_step(x[:, t:t + 1], t, caches)
            toks = [[] for _ in range(n)]
            for j in range(max_new):
                nxt = logits[:, -1].argmax(-1)
                for r in range(n):
                    toks[r].append(int(nxt[r]))
                if bool(finished(torch.tensor(toks)).all()) or j == max_new - 1:
                    break
                logits = self.model.decode_step(nxt[:, None], plen + j, caches)
        return [self._cut(t, stop_strs) for t in toks]

    def _greedy(self, prompt_ids, max_new, stop_strs):
        max_new = min(max_new, max(1, self.max_length // 2))
        ids = trunc_keep_head(prompt_ids, max(1, self.max_length - max_new))
        return self._greedy_batch([ids], max_new, stop_strs)[0]

    def generate_until(self, requests):
        """Greedy generation.  Requests are grouped by (prompt length in tokens, stop strings, budget): rows of
        one group share their position counter, so they decode as one batch of up to `gen_rows` rows."""
        from collections import defaultdict
        out, groups = [None] * len(requests), defaultdict(list)
        for i, req in enumerate(requests):
            prompt, kw = _args(req)[:2]
            kw = dict(kw or {})
            until = kw.get("until") or []
            until = (until,) if isinstance(until, str) else tuple(until)
            max_new = int(kw.get("max_gen_toks", kw.get("max_new_tokens", 64)))
            key = self._gen_key(prompt, list(until), max_new)
            if key in self._gcache:
                out[i] = self._gcache[key]
            elif self._gcache_only:
                out[i] = "<UNCACHED>"
            else:
                max_new = min(max_new, max(1, self.max_length // 2))
                ids = trunc_keep_head([self.bos] + self.tok_encode(prompt), max(1, self.max_length - max_new))
                groups[(len(ids), until, max_new)].append((i, key, ids))
        for (_, until, max_new), items in sorted(groups.items(), key=lambda kv: kv[0][0]):
            for b0 in range(0, len(items), self.gen_rows):
                part = items[b0:b0 + self.gen_rows]
                texts = self._greedy_batch([ids for _, _, ids in part], max_new, list(until))
                for (i, key, _), text in zip(part, texts):
                    out[i] = self._gcache[key] = text
                    if self._gcache_path:
                        with open(self._gcache_path, "a") as f:
                            f.write(json.dumps({"k": key, "g": text}) + "\n")
        return out


class WavefrontEval(DualModEval):
    """Scoring AND generation through a training engine at K sweeps: the operator the model was trained
    with (the wavefront engine at the last rung of its ladder), not the exact scan.

      likelihood   rows are right-padded to `T_eval` (a whole number of chunks) and scored in batches of
                   `batch_rows`; the engine's masks are causal, so padding never reaches a real position
      generation   greedy, one engine forward over [prompt + generated so far, padding] per token; every
                   row keeps its exact tokens at positions [0, len) and is read at its own last position;
                   rows are bucketed by (padded length, stop strings, budget), `gen_rows` per forward
      operator     `local_window` / other operator-defining engine arguments travel with the checkpoint
                   (`engine_kwargs` saved by the trainer) and are applied unless overridden
      cache        `GEN_CACHE_DIR`: the finished generations of one call are pickled per (tag, rank, world,
                   request hash), so a rank that finished is not recomputed after a failed collective

    Reference parity: lm/eval/lm_eval_adapter.py:605-781 (`Wave3DEval`)."""

    OPERATOR_KEYS = ("local_window", "raw_diag")

    def __init__(self, ckpt, K, T_eval=2048, C=64, engine="wave3d", gen_rows=4, engine_kwargs=None, **kw):
        T_eval = -(-T_eval // C) * C
        kw.setdefault("max_length", T_eval)
        super().__init__(ckpt, **kw)
        assert self.model.cfg.attn_mode != "vanilla", "engine scoring needs the Dual-Mod operator"
        self.K, self.C, self.T_eval, self.engine_name, self.gen_rows = int(K), C, T_eval, engine, gen_rows
        ekw = {k: v for k, v in (self.ckpt_engine_kwargs or {}).items() if k in self.OPERATOR_KEYS and v}
        ekw.update(engine_kwargs or {})
        ekw.pop("C", None)
        self.engine_kwargs = ekw
        self.max_length = min(self.max_length, T_eval)

    def _engine(self, B, T):
        key = (self.engine_name, B, T)
        if key not in self._engines:
            for k in [k for k in self._engines if k[0] == self.engine_name and k != key]:
                del self._engines[k]                     # one engine of this kind resident at a time
            common = dict(device=self.dev, keep_logits=True, autocast_bf16=torch.device(self.dev).type == "cuda",
                          **self.engine_kwargs)
            if self.engine_name == "wave3d":
                from ..engines.wave3d import Wave3DEngine
                eng = Wave3DEngine(self.model, [self.K], B, T, C=self.C, **common)
            else:
                from ..engines.schedule import uniform_chunks
                from ..engines.wavescan import WaveScanEngine
                eng = WaveScanEngine(self.model, [uniform_chunks(T, self.C, min(self.C, self.K))], B, T, **common)
            eng.pack()
            self._engines[key] = eng
        return self._engines[key]

    @torch.no_grad()
    def _logits(self, x):
        B, L = x.shape
        T = -(-L // self.C) * self.C
        rows = self.batch_rows
        eng = self._engine(rows, T)
        xp = torch.zeros(rows, T, dtype=torch.long, device=self.dev)
        out = []
        for b0 in range(0, B, rows):
            n = min(rows, B - b0)
            xp.zero_()
            xp[:n, :L] = x[b0:b0 + n]
            eng.forward(xp)
            out.append(eng.logits[:n, :L].float().clone())
        return torch.cat(out)

    # ---- generation through the engine --------------------------------------------------------------
    def generate_until(self, requests):
        import pickle
        cdir, cpath = os.environ.get("GEN_CACHE_DIR"), None
        if cdir:
            salt = f"{os.environ.get('GEN_TRUNC', 'tail')}:K{self.K}:"
            h = hashlib.sha1((salt + repr([(_args(r)[0], sorted(dict(_args(r)[1] or {}).items(), key=str))
                                           for r in requests])).encode()).hexdigest()[:12]
            cpath = os.path.join(cdir, f"{os.environ.get('GEN_TAG', 'gen')}_w{self._world_size}_r{self._rank}_{h}.pkl")
            if os.path.exists(cpath):
                res = pickle.load(open(cpath, "rb"))
                if len(res) == len(requests):
                    return res
        res = self._generate_engine(requests)
        if cpath:
            os.makedirs(cdir, exist_ok=True)
            with open(cpath + ".tmp", "wb") as f:
                pickle.dump(res, f)
            os.replace(cpath + ".tmp", cpath)
        return res

    @torch.no_grad()
    def _generate_engine(self, requests):
        from collections import defaultdict
        buckets = defaultdict(list)
        for i, req in enumerate(requests):
            prompt, kw = _args(req)[:2]
            kw = dict(kw or {})
            until = kw.get("until") or []
            until = (until,) if isinstance(until, str) else tuple(until)
            max_new = min(int(kw.get("max_gen_toks", kw.get("max_new_tokens", 128))), max(1, self.max_length // 2))
            toks = trunc_keep_head([self.bos] + self.tok_encode(prompt), max(1, self.max_length - max_new))
            T = min(self.max_length, -(-(len(toks) + max_new) // self.C) * self.C)
            buckets[(T, until, max_new)].append((toks, i))
        res, eos, R = [None] * len(requests), self.tok.eos_token_id, self.gen_rows
        for (T, until, max_new), group in sorted(buckets.items(), key=lambda kv: kv[0][0]):
            eng = self._engine(R, T)
            group.sort(key=lambda it: len(it[0]))
            for g0 in range(0, len(group), R):
                sub = group[g0:g0 + R]
                n = len(sub)
                x = torch.zeros(R, T, dtype=torch.long, device=self.dev)
                for b, (toks, _) in enumerate(sub):
                    x[b, :len(toks)] = torch.tensor(toks, device=self.dev)
                pos = torch.tensor([len(t) for t, _ in sub] + [1] * (R - n), device=self.dev)    # next slot per row
                ar = torch.arange(R, device=self.dev)
                outs, alive = [[] for _ in range(n)], [True] * n
                for _ in range(max_new):
                    eng.forward(x)
                    nxt = eng.logits[ar, pos - 1].float().argmax(-1)
                    for b in range(n):
                        if not alive[b]:
                            continue
                        t = int(nxt[b])
                        if t == eos:
                            alive[b] = False
                            continue
                        outs[b].append(t)
                        if until and any(u in self.tok.decode(outs[b][-16:]) for u in until):
                            alive[b] = False
                    if not any(alive) or int(pos[:n].max()) >= T:
                        break
                    wr = pos < T
                    x[ar[wr], pos[wr]] = nxt[wr]
                    pos = torch.clamp(pos + 1, max=T)
                for b, (_, i) in enumerate(sub):
                    text = self.tok.decode(outs[b])
                    for u in until:
                        if u in text:
                            text = text[:text.index(u)]
                    res[i] = text
        return res


def run_lm_eval(ckpt, tasks, tokenizer, num_fewshot=0, limit=None, out_path=None, wavefront_K=0, **kw):
    """Drive `lm_eval.simple_evaluate` with a checkpoint (needs the `lm_eval` package).  wavefront_K > 0
    scores and generates through the training engine at that K (`WavefrontEval`)."""
    import lm_eval
    lm = (WavefrontEval(ckpt, wavefront_K, tokenizer=tokenizer, **kw) if wavefront_K
          else DualModEval(ckpt, tokenizer=tokenizer, **kw))
    res = lm_eval.simple_evaluate(model=lm, tasks=list(tasks), num_fewshot=num_fewshot, limit=limit)
    if out_path and lm.rank == 0:
        json.dump(res["results"], open(out_path, "w"), indent=1)
    return res
