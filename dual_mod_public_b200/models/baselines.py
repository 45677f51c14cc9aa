"""Baseline architectures of the formal-language comparisons, all on the same trunk blocks.

  FBTLM             full-bandwidth Transformer: the previous position's top-layer state is fused
                    with the current token embedding and fed back as the layer-0 input; exact
                    sequential training or the P-pass parallel approximation
                    (reference: models/fbt/fbt_lm.py:23-79)
  LoopedLM          weight-tied blocks applied K times with input injection and a step embedding;
                    `recurrent_depth=True` switches to the recurrent-depth recipe (noise initial
                    state, adapter on [s; e], sandwich norms, coda, truncated backprop)
                    (models/looped/looped_lm.py:13-100)
  RecurrentDepthLM  LoopedLM pinned to that recipe (models/recurrent_depth/recurrent_depth_lm.py:20-26)
  LSTMLM            tied-embedding LSTM (models/baselines/lstm_lm.py:5-15)
  GatedDeltaNetLM   gated delta-rule linear recurrence.  The reference builds this arm from the
                    `fla` package (models/baselines/gdn.py:8-12); that package is not a dependency
                    here, so the layer is implemented natively (sequential state update in torch).
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import DualModConfig
from .layers import RMSNorm, SwiGLU
from .lm import Block, DualModLM
from .rope import build_rope_cache


def _uniform_jitter(x, amp):
    return x + (torch.rand_like(x) * 2 - 1) * amp


class FBTLM(nn.Module):
    def __init__(self, cfg: DualModConfig, jitter: float = 0.02):
        super().__init__()
        assert cfg.attn_mode == "vanilla", "the FBT stack is plain Transformer++ blocks"
        d = cfg.d_model
        self.core = DualModLM(cfg)
        self.w_u = nn.Linear(d, d, bias=False)       # carries the previous top-layer state
        self.w_g = nn.Linear(d, d, bias=False)       # token gate
        self.e_norm, self.in_norm = RMSNorm(d), RMSNorm(d)
        self.jitter = jitter
        for w in (self.w_u, self.w_g):
            nn.init.normal_(w.weight, std=0.02)

    def _fuse(self, h_prev, e_t):
        return self.w_u(h_prev) * torch.sigmoid(self.w_g(self.e_norm(e_t)))

    def _forward_passes(self, e, n_pass):
        """Parallel approximation: pass 1 is the plain stack on e; pass k feeds every position
        the previous pass's state of its predecessor."""
        core, T = self.core, e.shape[1]
        cos, sin = core.rope_cos[:T], core.rope_sin[:T]
        h = None
        for _ in range(int(n_pass)):
            if h is None:
                u = e
            else:
                hp = h[:, :-1]
                if self.training and self.jitter > 0:
                    hp = _uniform_jitter(hp, self.jitter)
                u = torch.cat((e[:, :1], self.in_norm(self._fuse(hp, e[:, 1:]))), dim=1)
            x = u
            for blk in core.blocks:
                x = blk(x, cos, sin)
            h = core.norm_f(x)
        return core.lm_head(h)

    def forward(self, idx, K=None):
        """K falsy: exact recurrence, one teacher-forced sequential pass over a KV cache with
        backprop through every position.  K = P >= 1: P parallel passes.  Returns (logits,)."""
        core = self.core
        B, T = idx.shape
        assert T <= core.cfg.max_seq_len
        e = core.tok_emb(idx)
        if K:
            return (self._forward_passes(e, K),)
        caches = [{"K": None, "V": None} for _ in core.blocks]
        h_prev, outs = None, []
        for t in range(T):
            u = e[:, t:t + 1]
            if h_prev is not None:
                u = self._fuse(h_prev, u)
                if self.training and self.jitter > 0:
                    u = _uniform_jitter(u, self.jitter)
                u = self.in_norm(u)
            x = u
            for blk, cache in zip(core.blocks, caches):
                x = blk.decode_step(x, t, cache, core.rope_cos, core.rope_sin)
            h_prev = core.norm_f(x)
            outs.append(core.lm_head(h_prev))
        return (torch.cat(outs, dim=1),)


class LoopedLM(nn.Module):
    def __init__(self, cfg: DualModConfig, n_unique: int = 2, k_max: int = 64, inject: bool = True,
                 huginn: bool = False, bp_iters: int = 0, emb_scale: bool = False):
        super().__init__()
        assert cfg.attn_mode == "vanilla"
        d = cfg.d_model
        self.cfg, self.n_unique, self.k_max, self.inject = cfg, n_unique, k_max, inject
        self.huginn, self.bp_iters = huginn, bp_iters
        self.emb_scale = math.sqrt(d) if (huginn and emb_scale) else 1.0
        self.tok_emb = nn.Embedding(cfg.vocab_size, d)
        self.pre = Block(cfg)
        self.loop = nn.ModuleList(Block(cfg) for _ in range(n_unique))
        self.step_emb = nn.Embedding(k_max + 1, d)
        if huginn:
            self.adapter = nn.Linear(2 * d, d, bias=False)
            self.post_norms = nn.ModuleList(nn.ModuleList([RMSNorm(d), RMSNorm(d)]) for _ in range(n_unique))
            self.coda = Block(cfg)
        self.norm_f = RMSNorm(d)
        self.lm_head = nn.Linear(d, cfg.vocab_size, bias=False)
        if cfg.tie_embeddings:
            self.lm_head.weight = self.tok_emb.weight
        cos, sin = build_rope_cache(cfg.max_seq_len, cfg.head_dim, cfg.rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)
        self._init_weights()

    def _init_weights(self):
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0.0, 0.02)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)
            elif isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, 0.0, 0.02)
        # residual outputs scale with the number of UNIQUE blocks: iterations share weights
        resid = 0.02 / math.sqrt(2 * (1 + self.n_unique))
        for blk in [self.pre, *self.loop]:
            nn.init.normal_(blk.attn.wo.weight, 0.0, resid)
            nn.init.normal_(blk.mlp.w2.weight, 0.0, resid)
        nn.init.zeros_(self.step_emb.weight)

    def _iterate(self, x, e, k, K, cos, sin):
        if self.huginn:
            if self.bp_iters and self.training and k < K - self.bp_iters:
                x = x.detach()
            x = self.adapter(torch.cat((x, e), dim=-1))
            for blk, (n_attn, n_mlp) in zip(self.loop, self.post_norms):
                x = n_attn(x + blk.attn(blk.attn_norm(x), cos, sin))
                x = n_mlp(x + blk.mlp(blk.mlp_norm(x)))
            return x
        if self.inject:
            x = x + e
        x = x + self.step_emb.weight[min(k, self.k_max)]
        for blk in self.loop:
            x = blk(x, cos, sin)
        return x

    def forward(self, idx, targets=None, K=None, return_all=False):
        K = self.k_max if K is None else K
        T = idx.shape[1]
        cos, sin = self.rope_cos[:T], self.rope_sin[:T]
        e = self.tok_emb(idx)
        if self.huginn:
            e = self.pre(e * self.emb_scale, cos, sin)
            sd = math.sqrt(0.4)
            x = nn.init.trunc_normal_(torch.empty_like(e), std=sd, a=-2 * sd, b=2 * sd)
        else:
            x = self.pre(e, cos, sin)
        states = []
        for k in range(K):
            x = self._iterate(x, e, k, K, cos, sin)
            if return_all:
                states.append(x)
        if self.huginn:
            x = self.coda(x, cos, sin)
        logits = self.lm_head(self.norm_f(x))
        loss = None
        if targets is not None:
            loss = F.cross_entropy(logits.float().view(-1, logits.shape[-1]), targets.reshape(-1))
        return (logits, loss, states) if return_all else (logits, loss)


class RecurrentDepthLM(LoopedLM):
    def __init__(self, cfg: DualModConfig, n_unique: int = 2, k_max: int = 128, bp_iters: int = 8,
                 emb_scale: bool = True):
        super().__init__(cfg, n_unique=n_unique, k_max=k_max, inject=True, huginn=True,
                         bp_iters=bp_iters, emb_scale=emb_scale)


class LSTMLM(nn.Module):
    def __init__(self, vocab, d, L):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.lstm = nn.LSTM(d, d, num_layers=L, batch_first=True)
        self.head = nn.Linear(d, vocab, bias=False)
        self.head.weight = self.emb.weight

    def forward(self, x):
        return (self.head(self.lstm(self.emb(x))[0]),)


# ---- Gated DeltaNet, native ---------------------------------------------------------------------

class GatedDeltaLayer(nn.Module):
    """S_t = a_t S_{t-1} (I - b_t k_t k_t^T) + b_t v_t k_t^T ;  o_t = S_t q_t, per head, with
    L2-normalised q/k, a short causal depthwise conv on q/k/v, a decay gate a_t in (0,1), a write
    strength b_t in (0,1) and an output gate."""

    def __init__(self, d, n_heads, head_dim=64, conv=4):
        super().__init__()
        self.h, self.dk = n_heads, head_dim
        inner = n_heads * head_dim
        self.q, self.k, self.v = (nn.Linear(d, inner, bias=False) for _ in range(3))
        self.a, self.b = nn.Linear(d, n_heads, bias=True), nn.Linear(d, n_heads, bias=True)
        self.g = nn.Linear(d, inner, bias=False)
        self.o = nn.Linear(inner, d, bias=False)
        self.conv = nn.Conv1d(3 * inner, 3 * inner, conv, groups=3 * inner, padding=conv - 1)
        self.out_norm = RMSNorm(head_dim)
        nn.init.constant_(self.a.bias, 3.0)

    def forward(self, x):
        B, T, _ = x.shape
        h, dk = self.h, self.dk
        qkv = torch.cat((self.q(x), self.k(x), self.v(x)), dim=-1).transpose(1, 2)
        qkv = F.silu(self.conv(qkv)[..., :T]).transpose(1, 2)
        q, k, v = (t.view(B, T, h, dk) for t in qkv.chunk(3, dim=-1))
        q, k = F.normalize(q.float(), dim=-1), F.normalize(k.float(), dim=-1)
        v = v.float()
        a = torch.sigmoid(self.a(x).float())                   # decay
        b = torch.sigmoid(self.b(x).float())                   # write strength
        S = x.new_zeros(B, h, dk, dk, dtype=torch.float32)     # [.., value dim, key dim]
        outs = []
        for t in range(T):
            kt, vt, bt = k[:, t], v[:, t], b[:, t, :, None]
            S = S * a[:, t, :, None, None]
            pred = torch.einsum("bhvk,bhk->bhv", S, kt)
            S = S + torch.einsum("bhv,bhk->bhvk", bt * (vt - pred), kt)
            outs.append(torch.einsum("bhvk,bhk->bhv", S, q[:, t]))
        o = self.out_norm(torch.stack(outs, dim=1)).to(x.dtype)
        o = o.reshape(B, T, h * dk) * F.silu(self.g(x))
        return self.o(o)


class GatedDeltaNetLM(nn.Module):
    def __init__(self, vocab, d, L, h, head_dim=64, hidden_ratio=4):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.layers = nn.ModuleList()
        for _ in range(L):
            self.layers.append(nn.ModuleDict({
                "n1": RMSNorm(d), "mix": GatedDeltaLayer(d, max(1, h // 2), head_dim),
                "n2": RMSNorm(d), "mlp": SwiGLU(d, int(round(hidden_ratio * d * 2 / 3 / 64) * 64) or 64)}))
        self.norm_f = RMSNorm(d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.head.weight = self.emb.weight
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, 0.0, 0.02)
            elif isinstance(m, nn.Embedding):
                nn.init.normal_(m.weight, 0.0, 0.02)

    def forward(self, x):
        z = self.emb(x)
        for lay in self.layers:
            z = z + lay["mix"](lay["n1"](z))
            z = z + lay["mlp"](lay["n2"](z))
        return (self.head(self.norm_f(z)),)


def build_gdn(vocab, d, L, h, impl="native"):
    """Gated DeltaNet of the same width / depth as the other arms of a scale.  `impl="fla"`
    builds the `fla` package's model instead (when that package works in the environment)."""
    if impl == "fla":
        from fla.models import GatedDeltaNetConfig, GatedDeltaNetForCausalLM
        cfg = GatedDeltaNetConfig(hidden_size=d, num_hidden_layers=L, num_heads=h // 2, head_dim=64, expand_v=1,
                                  hidden_ratio=4, vocab_size=vocab, tie_word_embeddings=True)
        return GatedDeltaNetForCausalLM(cfg)
    return GatedDeltaNetLM(vocab, d, L, h)
