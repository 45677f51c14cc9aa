"""Dual-Mod attention layer.

A position t reads the tape of refined entries written before it plus its own
RAW key/value (`attend_one`), then refines its key and value from what it read
(`refine_kv`) and appends the result to the tape, the key rotated at write.
Those two methods are the per-position contract shared by the exact scan, the
chunked engines and incremental decode.  Parity with the reference layer
(models/dualmod/attention.py:86-588): same parameters and state-dict keys, same
knobs, same numerics contract (fp32 softmax, fp32 gate sigmoid, fp32 norms).

Modes (`cfg.attn_mode`):
  vanilla     plain causal attention (the Transformer++ control)
  sequential  exact per-position scan (`scan.sequential_scan`)
  deq         K parallel Jacobi sweeps over the whole sequence
  static      control whose write branch reads x̂ instead of the attention output
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import DualModConfig
from .layers import LoRAGate, LoRALinear, RMSNorm, head_rms
from .rope import apply_rope

# ctx_mod -> which extra modules exist: name -> (in_mult, out_mult, bias, may_factor)
_CTX_EXTRAS = {
    "linear": {},
    "vmlp": {"v_pre": (1, 1, False, False)},
    "fusion": {"v_pre": (2, 1, False, False)},
    "puremlp": {"v_pre": (2, 1, False, False)},
    "puremlp_hw": {"v_pre": (2, 1, False, False)},
    "kmlp": {"k_pre": (1, 1, False, False)},
    "mult": {"v_gate": (1, 1, True, True), "v_map": (1, 1, False, True)},
    "mult_res": {"v_gate": (1, 1, True, True), "v_map": (1, 1, False, True)},
    "linpoint": {"v_pre": (1, 2, False, False), "v_comb": (2, 1, False, False)},
    "glu": {"v_gate": (2, 1, False, False), "v_map": (2, 1, False, False)},
}


class DualModAttention(nn.Module):
    def __init__(self, cfg: DualModConfig):
        super().__init__()
        self.cfg = cfg
        d = cfg.d_model
        self.n_heads = cfg.n_heads
        self.n_kv_heads = cfg.n_kv_heads_eff
        self.head_dim = cfg.head_dim
        self.d_attn = cfg.d_attn
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        d_kv = self.n_kv_heads * self.head_dim

        self.wq = nn.Linear(d, self.d_attn, bias=False)
        self.wk = nn.Linear(d, d_kv, bias=False)
        self.wv = nn.Linear(d, d_kv, bias=False)
        self.wo = nn.Linear(self.d_attn, d, bias=False)
        if cfg.v_norm == "rms":
            self.v_gain = nn.Parameter(torch.ones(self.n_kv_heads))
        if cfg.attn_mode == "vanilla":
            return

        def ctx_op(d_in, d_out, bias=False, may_factor=True):
            if cfg.ctx_rank > 0 and may_factor:
                return LoRALinear(d_in, cfg.ctx_rank, d_out, bias=bias)
            return nn.Linear(d_in, d_out, bias=bias)

        def gate(width):
            if cfg.gate_rank > 0:
                return LoRAGate(cfg.gate_in_dim, cfg.gate_rank, width)
            return nn.Linear(cfg.gate_in_dim, width, bias=True)

        if cfg.enable_key_mod:
            self.w_kctx = ctx_op(d, d)
            self.w_gk = gate(2 * d if cfg.gate_type == "independent" else d)
            if cfg.k_ctx_norm == "rms":
                self.k_gain = nn.Parameter(torch.full((self.n_heads,), float(cfg.k_gain_init)))
        if cfg.enable_value_mod:
            self.w_vctx = ctx_op(d, d)
            self.w_gv = gate(2 * d if cfg.gate_type_v == "independent" else d)
            if cfg.v_ctx_norm == "rms":
                self.ctx_gain = nn.Parameter(torch.ones(self.n_heads))
        for name, (im, om, bias, fac) in _CTX_EXTRAS[cfg.ctx_mod].items():
            setattr(self, name, ctx_op(im * d, om * d, bias=bias, may_factor=fac))
        for pre in ("v_pre", "k_pre"):           # residual pre-layers start as exact identity
            if hasattr(self, pre):
                nn.init.zeros_(getattr(self, pre).weight)
        if cfg.rmsnorm_on_o and (cfg.enable_key_mod or cfg.enable_value_mod):
            self.norm_ctx = RMSNorm(d)

    # ---- head layout ---------------------------------------------------------------
    def _split(self, x: torch.Tensor) -> torch.Tensor:
        """[B, T, h*dh] -> [B, h, T, dh]"""
        B, T, _ = x.shape
        return x.view(B, T, self.n_heads, self.head_dim).transpose(1, 2)

    def _merge(self, x: torch.Tensor) -> torch.Tensor:
        """[B, h, T, dh] -> [B, T, h*dh]"""
        B, h, T, dh = x.shape
        return x.transpose(1, 2).reshape(B, T, h * dh)

    # ---- the single sites of the three per-head norms --------------------------------
    def project_v(self, xhat):
        """Raw value projection (flat [.., d_kv]); `v_norm=rms` norms it per head."""
        v = self.wv(xhat)
        if self.cfg.v_norm != "rms":
            return v
        return head_rms(v, self.n_kv_heads, self.v_gain)

    def norm_vctx(self, v_ctx):
        """Per-head RMS + gain on the ctx value candidate (`v_ctx_norm=rms`)."""
        if self.cfg.v_ctx_norm != "rms":
            return v_ctx
        return head_rms(v_ctx, self.n_heads, self.ctx_gain)

    def norm_kctx(self, k_ctx):
        """Per-head RMS + gain on the ctx key candidate (`k_ctx_norm=rms`)."""
        if self.cfg.k_ctx_norm != "rms":
            return k_ctx
        return head_rms(k_ctx, self.n_heads, self.k_gain)

    def clamp_vpp(self, vpp):
        """Project each (position, head) value vector onto the L2 ball of radius tau."""
        tau = self.cfg.v_clamp_tau
        if not tau or tau <= 0:
            return vpp
        lead = vpp.shape[:-1]
        vh = vpp.reshape(*lead, self.n_kv_heads, self.head_dim).float()
        shrink = (tau / vh.norm(dim=-1, keepdim=True).clamp_min(1e-20)).clamp(max=1.0)
        return (vh * shrink).to(vpp.dtype).reshape(*lead, -1)

    # ---- read ---------------------------------------------------------------------------
    def _logn_factor(self, n_keys: int) -> float:
        ref = self.cfg.attn_logn_ref or 0
        if ref > 1 and n_keys > 1:
            return math.log(n_keys) / math.log(ref)
        return 1.0

    def _logn_rows(self, s):
        """Row i of a causal [.., T, T] score matrix has i+1 keys; scale finite entries."""
        ref = self.cfg.attn_logn_ref or 0
        if ref <= 1:
            return s
        T = s.shape[-2]
        n = torch.arange(1, T + 1, device=s.device, dtype=torch.float32)
        f = (n.log() / math.log(ref)).clamp_min(0.0).view(*([1] * (s.dim() - 2)), T, 1)
        return torch.where(torch.isinf(s), s, s * f.to(s.dtype))

    def attend_one(self, q_r, k_self_r, v_self, K_past, V_past, need_probs=False, collect=None):
        """One position's read.  q_r / k_self_r / v_self are [B,h,1,dh] (rotated
        query, rotated RAW self key, RAW self value); K_past / V_past the refined
        tape [B,h,P,dh] or None.  Returns (o [B,h,1,dh], probs or None)."""
        W = self.cfg.local_window or 0
        if K_past is not None and W and K_past.shape[2] > W - 1:
            K_past, V_past = K_past[:, :, -(W - 1):], V_past[:, :, -(W - 1):]
        if K_past is None or K_past.shape[2] == 0:
            keys, vals = k_self_r, v_self
        else:
            keys = torch.cat((K_past, k_self_r), dim=2)
            vals = torch.cat((V_past, v_self), dim=2)
        s = (q_r @ keys.transpose(-1, -2)) * self.scale
        f = self._logn_factor(keys.shape[2])
        if f != 1.0:
            s = s * f
        if collect is not None:
            collect.setdefault("attn_logit_max", []).append(
                s.detach().abs().amax(dim=-1).reshape(-1).float())
        p = torch.softmax(s.float(), dim=-1)
        return p.to(vals.dtype) @ vals, (p if need_probs else None)

    # ---- write ----------------------------------------------------------------------------
    def _gate_source(self, xhat, u):
        gi = self.cfg.gate_input
        if gi == "xu":
            return torch.cat((xhat, u), dim=-1)
        return u if gi == "u" else xhat

    def _value_transition(self, xhat, u):
        """v_in(x̂, u): what the value ctx projection reads, per ctx_mod."""
        mod = self.cfg.ctx_mod
        if mod == "vmlp":
            return u + F.silu(self.v_pre(u))
        if mod == "fusion":
            return u + F.silu(self.v_pre(torch.cat((xhat, u), dim=-1)))
        if mod in ("puremlp", "puremlp_hw"):
            return F.silu(self.v_pre(torch.cat((xhat, u), dim=-1)))
        if mod in ("mult", "mult_res"):
            branch = torch.sigmoid(self.v_gate(xhat).float()).to(u.dtype) * torch.tanh(self.v_map(u))
            return branch if mod == "mult" else self.cfg.mult_res_lambda * u + branch
        if mod == "linpoint":
            return self.v_comb(F.silu(self.v_pre(u)))
        if mod == "glu":
            xu = torch.cat((xhat, u), dim=-1)
            return F.silu(self.v_gate(xu)) * self.v_map(xu)
        return u

    def _blend(self, gate_logits, raw, ctx, collect, tag):
        """g*raw + (1-g)*ctx (convex), g1*raw + g2*ctx (independent) or the
        unbounded linear gate; sigmoid always in fp32."""
        kind = self.cfg.gate_type
        if tag == "v":
            kind = "independent" if self.cfg.gate_type_v == "independent" else "convex_sigmoid"
        g_ctx = None
        if kind == "independent":
            g, g_ctx = torch.sigmoid(gate_logits.float()).to(raw.dtype).chunk(2, dim=-1)
            out = g * raw + g_ctx * ctx
        else:
            g = (torch.sigmoid(gate_logits.float()) if kind == "convex_sigmoid"
                 else gate_logits).to(raw.dtype)
            out = g * raw + (1.0 - g) * ctx
        if collect is not None:
            collect.setdefault(f"g_{tag}", []).append(g.detach().float())
            if g_ctx is not None:
                collect.setdefault(f"g_{tag}_ctx", []).append(g_ctx.detach().float())
            ratio = ctx.detach().float().norm(dim=-1) / (raw.detach().float().norm(dim=-1) + 1e-8)
            collect.setdefault(f"ratio_{tag}", []).append(ratio)
        return out

    def refine_kv(self, xhat, o_cat, k_raw, v_raw, collect=None):
        """(k'', v'') from the read o_cat; all tensors [B, t, d].  The key comes
        back UNROTATED: the caller rotates it when writing to the tape."""
        cfg = self.cfg
        if not cfg.dual_mod_active:
            return k_raw, v_raw
        u = self.norm_ctx(o_cat) if cfg.rmsnorm_on_o else o_cat
        g_in = self._gate_source(xhat, u)
        kpp, vpp = k_raw, v_raw
        if cfg.enable_key_mod:
            k_in = u + F.silu(self.k_pre(u)) if cfg.ctx_mod == "kmlp" else u
            k_ctx = self.norm_kctx(self.w_kctx(k_in))
            kpp = self._blend(self.w_gk(g_in), k_raw, k_ctx, collect, "k")
        if cfg.enable_value_mod:
            v_ctx = self.norm_vctx(self.w_vctx(self._value_transition(xhat, u)))
            n_raw = cfg.kmod_vraw_heads
            cut = n_raw * self.head_dim
            if n_raw > 0 and cfg.kmod_mode == "gated_norm":
                # the first heads have no ctx term: the blend is a pure write gate
                v_ctx = torch.cat((torch.zeros_like(v_ctx[..., :cut]), v_ctx[..., cut:]), dim=-1)
            vpp = self._blend(self.w_gv(g_in), v_raw, v_ctx, collect, "v")
            if n_raw > 0 and cfg.kmod_mode == "raw":
                keep = v_raw[..., :cut]
                if cfg.kmod_vraw_bound == "tanh":
                    keep = torch.tanh(keep.float()).to(keep.dtype)
                vpp = torch.cat((keep, vpp[..., cut:]), dim=-1)
            vpp = self.clamp_vpp(vpp)
        if collect is not None:
            collect.setdefault("vpp", []).append(vpp.detach().float())
        return kpp, vpp

    # ---- full-sequence paths ----------------------------------------------------------------
    def forward(self, xhat, cos, sin, collect=None):
        """x̂ [B,T,d] (already normed) -> W_O o, the residual contribution."""
        mode = self.cfg.attn_mode
        if mode == "vanilla":
            return self._forward_vanilla(xhat, cos, sin)
        if mode == "sequential":
            from .scan import sequential_scan
            return self.wo(sequential_scan(self, xhat, cos, sin, collect=collect))
        if mode == "static":
            return self._forward_static(xhat, cos, sin, collect=collect)
        return self._forward_deq(xhat, cos, sin)

    def _kv_heads(self, x):
        B, T, _ = x.shape
        return x.view(B, T, self.n_kv_heads, self.head_dim).transpose(1, 2)

    def _causal_mask(self, T, device, strict=False):
        i = torch.arange(T, device=device)
        m = (i[None, :] < i[:, None]) if strict else (i[None, :] <= i[:, None])
        W = self.cfg.local_window or 0
        if W:
            m = m & (i[None, :] > i[:, None] - W)
        return m

    def _forward_vanilla(self, xhat, cos, sin):
        B, T, _ = xhat.shape
        q = apply_rope(self._split(self.wq(xhat)), cos, sin)
        k = apply_rope(self._kv_heads(self.wk(xhat)), cos, sin)
        v = self._kv_heads(self.project_v(xhat))
        gqa = self.n_heads != self.n_kv_heads
        W = self.cfg.local_window or 0
        if (self.cfg.attn_logn_ref or 0) > 1:
            if gqa:
                rep = self.n_heads // self.n_kv_heads
                k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
            s = (q @ k.transpose(-1, -2)) * self.scale
            s = s.masked_fill(~self._causal_mask(T, q.device), float("-inf"))
            o = torch.softmax(self._logn_rows(s).float(), dim=-1).to(v.dtype) @ v
        elif W:
            o = F.scaled_dot_product_attention(q, k, v, attn_mask=self._causal_mask(T, q.device),
                                               enable_gqa=gqa)
        else:
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=gqa)
        return self.wo(o.transpose(1, 2).reshape(B, T, self.d_attn))

    def _read_with_raw_diagonal(self, q_r, k_self_r, v_raw, K, V):
        """Causal read over a full-sequence tape (K, V) where every position's own
        entry is its RAW key/value: strict-lower scores from the tape, the diagonal
        from (k_self_r, v_raw)."""
        T = q_r.shape[2]
        below = self._causal_mask(T, q_r.device, strict=True)
        s = (q_r @ K.transpose(-1, -2)) * self.scale
        s = s.masked_fill(~below, float("-inf"))
        s = torch.diagonal_scatter(s, (q_r * k_self_r).sum(-1) * self.scale, dim1=-2, dim2=-1)
        p = torch.softmax(self._logn_rows(s).float(), dim=-1).to(V.dtype)
        p_self = p.diagonal(dim1=-2, dim2=-1).unsqueeze(-1)
        return (p * below) @ V + p_self * v_raw

    def _forward_deq(self, xhat, cos, sin):
        """`deq_sweeps` Jacobi passes over the whole sequence; sweep 0 reads the raw
        tape, each later sweep reads the tape refined from the previous read.
        deq_sweeps == T equals the sequential scan."""
        k_flat, v_flat = self.wk(xhat), self.project_v(xhat)
        q_r = apply_rope(self._split(self.wq(xhat)), cos, sin)
        k_self_r = apply_rope(self._split(k_flat), cos, sin)
        v_raw = self._split(v_flat)
        K, V, o = k_self_r, v_raw, None
        n = self.cfg.deq_sweeps
        for sweep in range(n):
            o = self._read_with_raw_diagonal(q_r, k_self_r, v_raw, K, V)
            if sweep + 1 < n:
                kpp, vpp = self.refine_kv(xhat, self._merge(o), k_flat, v_flat)
                K, V = apply_rope(self._split(kpp), cos, sin), self._split(vpp)
        return self.wo(self._merge(o))

    def _forward_static(self, xhat, cos, sin, collect=None):
        """Control: the write branch reads x̂ in place of the attention output, so
        (k'', v'') are functions of the token alone and one parallel pass is exact."""
        k_flat, v_flat = self.wk(xhat), self.project_v(xhat)
        q_r = apply_rope(self._split(self.wq(xhat)), cos, sin)
        k_self_r = apply_rope(self._split(k_flat), cos, sin)
        kpp, vpp = self.refine_kv(xhat, xhat, k_flat, v_flat, collect=collect)
        K, V = apply_rope(self._split(kpp), cos, sin), self._split(vpp)
        o = self._read_with_raw_diagonal(q_r, k_self_r, self._split(v_flat), K, V)
        return self.wo(self._merge(o))

    # ---- incremental decode -------------------------------------------------------------------
    def decode_step(self, xhat_j, pos, cache, cos, sin):
        """One token at absolute position `pos`; `cache` = {"K","V"} refined tape
        ([B,h,P,dh] or None), extended in place by one entry."""
        q, k, v = (self._split(t) for t in (self.wq(xhat_j), self.wk(xhat_j), self.project_v(xhat_j)))
        cj, sj = cos[pos:pos + 1], sin[pos:pos + 1]
        q_r, k_self_r = apply_rope(q, cj, sj), apply_rope(k, cj, sj)
        o, _ = self.attend_one(q_r, k_self_r, v, cache["K"], cache["V"])
        o_cat = self._merge(o)
        kpp, vpp = self.refine_kv(xhat_j, o_cat, self._merge(k), self._merge(v))
        k_new, v_new = apply_rope(self._split(kpp), cj, sj), self._split(vpp)
        if cache["K"] is None:
            cache["K"], cache["V"] = k_new, v_new
        else:
            cache["K"] = torch.cat((cache["K"], k_new), dim=2)
            cache["V"] = torch.cat((cache["V"], v_new), dim=2)
        return self.wo(o_cat)
