"""Dual-Mod on the chunked engine for the formal-language tasks.

Sequences of a few hundred tokens and more are 5-10x faster through the engine than
through the eager per-position scan.  The engine runs an exact schedule (chunks of
`ws_chunk` positions with as many sweeps), keeps the logits, and takes the gradient
of the masked cross-entropy as an explicit d_logits.  Engines are built per sequence
length on demand (curricula change the length).  Reference parity:
formal_language/harness/train_statetrack_ws.py (WaveScanEngine(keep_logits=True,
use_graphs=False) with uniform_chunks(T, 16, 16) and hand-computed d_logits, 300-312).
"""

from __future__ import annotations

import torch

from ..engines.schedule import uniform_chunks
from ..engines.wavescan import WaveScanEngine
from ..parallel.fused_optim import FusedDPAdamW, decay_groups, default_buckets
from . import harness as H


class EngineTrainer:
    def __init__(self, model, args, device):
        self.model, self.args, self.device = model.to(device), args, device
        self.opt = FusedDPAdamW(decay_groups(self.model, args.wd), default_buckets(self.model), lr=args.lr,
                                max_norm=1.0, device=device)
        self.grads = self.opt.grad_buffers()
        self._engines = {}

    def _engine(self, B, T):
        key = (B, T)
        if key not in self._engines:
            c = self.args.ws_chunk
            self._engines[key] = WaveScanEngine(
                self.model, [uniform_chunks(T, c)], B, T, device=self.device, keep_logits=True,
                autocast_bf16=self.device.type == "cuda", use_graphs=False, grads=self.grads,
                backend="generic" if getattr(self.args, "no_fused", False) else "auto")
        eng = self._engines[key]
        return eng

    def logits(self, x):
        eng = self._engine(*x.shape)
        eng.pack()
        eng.forward(x)
        return eng.logits

    def step(self, x, tgt, msk, lr, freeze=False):
        """freeze: only the embedding / head move this step (every other gradient is zeroed)."""
        eng = self._engine(*x.shape)
        self.opt.zero_grad()
        eng.pack()
        eng.forward(x)
        loss, d = H.masked_dlogits(eng.logits, x, tgt, msk)
        eng.backward(d_logits=d)
        if freeze:
            for n, p in self.model.named_parameters():
                if not (n.startswith("tok_emb") or n.startswith("lm_head")):
                    self.grads.get(p).zero_()
        self.opt.step(lr=lr)
        return float(loss)
