"""Incremental decode over a static recurrent KV tape, one CUDA graph per token.

The tape is [B, P, h, dh] per layer (token-major), the position lives on the device,
and one captured graph is one full decode step of all layers, so the host issues a
single graph launch per token.  Per layer the step is exactly `DualModAttention.decode_step`:
project, rotate at `pos`, read the live tape rows plus the position's own RAW key/value,
refine (key, value) from the read, rotate the blended key and write row `pos`.

Unlike a masked softmax over all P slots, the read touches only the `pos` live rows
(sm_100a kernel `dmb_decode_attend`, with the position read from device memory; the
plain-torch path masks instead and is what runs on CPU).  With the modulation off
(`attn_mode="vanilla"`) the same class is a plain KV-cache Transformer decoder: the
Transformer++ control.

On a B200 the rest of the step runs on the training engines' kernels and weight packs as well
(`fused=True`, the default there for the write laws with fused refine kernels): RMSNorm as one kernel, one
input GEMM for q, k, v and the gates' x-logits, RoPE at the device-side position, the read (which also returns
the per-head sum of squares the write law's norm needs), the packed context GEMM with the norm gain folded into
its columns, one refine kernel for gates, blend and rotation, SwiGLU as one kernel: about twenty launches per
layer instead of about seventy-five small framework kernels.

Reference parity: `GraphDecoder` (lm/eval/graph_decode.py:15-125): static buffers,
device-side `pos`, `capture / reset / step / generate(prompt, max_new, eos_id, stop_fn)`.
"""

from __future__ import annotations

import ctypes

import torch

from ..models.rope import apply_rope


class _Bag:
    def __init__(self, **kw):
        self.__dict__.update(kw)


class _DecodeRefine:
    """The training engine's fused write law (`WaveScanEngine._refine_fwd`: packed context GEMM, dense or factored,
    and the refine kernels of the packed and mult_res families) applied to the one row per sequence of a decode step."""

    def __init__(self, ops, cfg, family, B):
        self.ops, self.cfg, self.family, self.B = ops, cfg, family, B

    from ..engines.wavescan import WaveScanEngine as _E
    _refine_fwd, _vctx_linear, _engine_pack_linear = _E._refine_fwd, _E._vctx_linear, _E._pack_linear
    del _E

    def _pack_linear(self, P, o2, t_out=None):
        if not P.factored and self.B <= 64:          # one row per sequence: see `GraphDecoder._fused_layer`
            return self.ops.linear(o2, P.W_pack, narrow=True)
        return self._engine_pack_linear(P, o2, t_out)


class GraphDecoder:
    def __init__(self, model, B, P_max, dtype=torch.bfloat16, use_kernel=None, cast_weights=True, fused=None):
        self.dev = next(model.parameters()).device
        if (cast_weights and dtype == torch.bfloat16 and self.dev.type == "cuda"
                and next(model.parameters()).dtype == torch.float32):
            # decode from a bf16 copy of the weights: under autocast every step would otherwise re-cast
            # all fp32 master weights (hundreds of copy kernels and 3x the weight traffic per token)
            import copy
            src, model = model, copy.deepcopy(model).to(dtype)
            for name, buf in src.named_buffers():           # tables (RoPE) stay in their own precision
                mod, _, leaf = name.rpartition(".")
                setattr(model.get_submodule(mod) if mod else model, leaf, buf.clone())
        self.m = model
        assert P_max <= model.cfg.max_seq_len, (P_max, model.cfg.max_seq_len)
        a0 = model.blocks[0].attn
        L, h, dh = len(model.blocks), a0.n_heads, a0.head_dim
        self.B, self.P, self.dt, self.h, self.dh = B, P_max, dtype, h, dh
        z = lambda: torch.zeros(B, P_max, h, dh, device=self.dev, dtype=dtype)
        self.K, self.V = [z() for _ in range(L)], [z() for _ in range(L)]
        self.tok = torch.zeros(B, 1, dtype=torch.long, device=self.dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=self.dev)
        self.pos32 = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.ar = torch.arange(P_max, device=self.dev)
        self.logits = torch.zeros(B, 1, model.cfg.vocab_size, device=self.dev)
        self.next = torch.zeros(B, 1, dtype=torch.long, device=self.dev)
        self.graph = None
        self.window = model.cfg.local_window or 0
        ok = (self.dev.type == "cuda" and dtype == torch.bfloat16 and dh in (64, 128)
              and a0.n_kv_heads == a0.n_heads and not model.cfg.attn_logn_ref)
        self.use_kernel = ok if use_kernel is None else (use_kernel and ok)
        self.kernel_launches = 0
        if self.use_kernel:
            from ..ops.cuda_ops import load_library
            self.lib = load_library()
            p, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
            self.lib.dmb_decode_attend.restype = i
            self.lib.dmb_decode_attend.argtypes = [p, p, p, p, p, p, p, p, i, i, i, i, f, i, p]
        # the whole step on the engines' kernels and weight packs (see the module docstring)
        self.fused = False
        if self.use_kernel and fused is not False:
            from ..engines.wavescan import _LayerPack, fused_supported, refine_family
            cfg = model.cfg
            fam = refine_family(cfg) if cfg.attn_mode != "vanilla" and fused_supported(cfg) else None
            plain = cfg.attn_mode == "vanilla" and cfg.v_norm == "none"
            if fam in ("packed", "mrk") or plain:
                from ..ops import default_ops
                self.ops, self.family = default_ops(self.dev), fam
                self.packs = []
                for blk in self.m.blocks:
                    if fam:
                        P = _LayerPack(blk, cfg, dtype, self.dev, family=fam)
                        P.pack(blk, cfg)
                    else:                                   # plain KV cache: q, k, v as one input GEMM
                        a, c_ = blk.attn, (lambda w: w.detach().to(dtype).contiguous())
                        P = _Bag(w_an=c_(blk.attn_norm.weight), w_mn=c_(blk.mlp_norm.weight), b_in=None,
                                 W_in=torch.cat([c_(a.wq.weight), c_(a.wk.weight), c_(a.wv.weight)], 0),
                                 wo=c_(a.wo.weight), w1=c_(blk.mlp.w1.weight), w3=c_(blk.mlp.w3.weight),
                                 w2=c_(blk.mlp.w2.weight))
                    self.packs.append(P)
                self.refine = _DecodeRefine(self.ops, cfg, fam, B) if fam else None
                # the kernels read fp32 rotation tables (a model converted with .bfloat16() carries bf16 ones)
                self.cos32, self.sin32 = self.m.rope_cos.float().contiguous(), self.m.rope_sin.float().contiguous()
                self.fused = True
        if fused and not self.fused:
            raise ValueError("fused decode needs the kernel read and a write law with fused refine kernels")

    # ---- the read ---------------------------------------------------------------------------
    def _read(self, attn, q_r, k_r, v, l, ssq=None):
        """q_r, k_r, v: [B, h, dh] (rotated query, rotated RAW self key, RAW self value); `ssq` (kernel path):
        [B, h] fp32 that receives the sum of squares of every head's read."""
        Kb, Vb = self.K[l], self.V[l]
        if self.use_kernel:
            assert q_r.is_contiguous() and k_r.is_contiguous() and v.is_contiguous()
            out = torch.empty_like(q_r)
            st = ctypes.c_void_p(torch.cuda.current_stream(self.dev).cuda_stream)
            rc = self.lib.dmb_decode_attend(q_r.data_ptr(), k_r.data_ptr(), v.data_ptr(), Kb.data_ptr(), Vb.data_ptr(),
                                            self.pos32.data_ptr(), out.data_ptr(), ssq.data_ptr() if ssq is not None else None,
                                            self.B, self.P, self.h, self.dh, attn.scale, self.window, st)
            if rc != 0:
                raise RuntimeError(f"decode read failed ({rc})")
            self.kernel_launches += 1
            return out
        # plain torch: scores over every slot, live ones kept by a mask; self as an extra column
        s = torch.einsum("bhd,bphd->bhp", q_r.float(), Kb.float()) * attn.scale
        live = self.ar < self.pos
        if self.window:
            live = live & (self.ar > self.pos - self.window)
        s = s.masked_fill(~live, float("-inf"))
        s_self = (q_r.float() * k_r.float()).sum(-1, keepdim=True) * attn.scale
        p = torch.softmax(torch.cat((s, s_self), dim=-1), dim=-1)
        o = torch.einsum("bhp,bphd->bhd", p[..., :-1], Vb.float()) + p[..., -1:] * v.float()
        return o.to(v.dtype)

    def _attn(self, attn, xhat, l, cos_p, sin_p):
        B, h, dh = self.B, self.h, self.dh
        q, k, v = attn.wq(xhat), attn.wk(xhat), attn.project_v(xhat)            # [B,1,d]
        rot = lambda t: apply_rope(t.view(B, 1, h, dh).transpose(1, 2), cos_p, sin_p).transpose(1, 2).reshape(B, h, dh)
        q_r, k_r = rot(q).to(self.dt), rot(k).to(self.dt)
        o = self._read(attn, q_r.contiguous(), k_r.contiguous(), v.view(B, h, dh).to(self.dt).contiguous(), l)
        o_cat = o.reshape(B, 1, h * dh).to(xhat.dtype)
        kpp, vpp = attn.refine_kv(xhat, o_cat, k, v)
        self.K[l].index_copy_(1, self.pos, rot(kpp).to(self.dt).unsqueeze(1))
        self.V[l].index_copy_(1, self.pos, vpp.view(B, 1, h, dh).to(self.dt))
        return attn.wo(o_cat)

    def _fused_layer(self, blk, l, x, cos_p, sin_p):
        """One layer of the step on the engines' kernels: x [B, 1, d] in the decode dtype -> the layer's output."""
        ops, P, cfg = self.ops, self.packs[l], self.m.cfg
        B, h, dh, d = self.B, self.h, self.dh, self.h * self.dh
        # one row per sequence: the products stream their weights once over a sliver of rows (half an MMA tile
        # at batch 64), which is library-GEMM territory (`narrow`; 17.5 us per product on the own kernel)
        lin = lambda x_, w_, b_=None: ops.linear(x_, w_, bias=b_, narrow=B <= 64)
        xhat, _ = ops.rms_fwd(x, P.w_an)
        qkvg = lin(xhat, P.W_in, P.b_in)
        k, v = qkvg[..., d:2 * d], qkvg[..., 2 * d:3 * d]
        q_r = ops.rope(qkvg[..., :d].unflatten(-1, (h, dh)), cos_p, sin_p)            # [B, 1, h, dh]
        kself_r = ops.rope(k.unflatten(-1, (h, dh)), cos_p, sin_p)
        ssq = torch.empty(B, 1, h, dtype=torch.float32, device=self.dev) if self.refine else None
        o = self._read(blk.attn, q_r.view(B, h, dh), kself_r.view(B, h, dh), v.reshape(B, h, dh).contiguous(), l, ssq)
        if self.refine is not None:
            S = _Bag(P=P, k=k, v=v, glx=qkvg[..., 3 * d:5 * d], vgx=qkvg[..., 5 * d:] if self.family == "mrk" else None,
                     cos=cos_p, sin=sin_p, pin=cfg.kmod_vraw_heads * dh)
            K_new, V_new, _ = self.refine._refine_fwd(S, slice(0, 1), o.view(B, 1, h, dh), ssq)
        else:                                                                        # plain KV cache
            K_new, V_new = kself_r, v.unflatten(-1, (h, dh))
        self.K[l].index_copy_(1, self.pos, K_new)
        self.V[l].index_copy_(1, self.pos, V_new)
        x_mid = x + lin(o.view(B, 1, d), P.wo)
        xn, _ = ops.rms_fwd(x_mid, P.w_mn)
        g = ops.swiglu_fwd(lin(xn, P.w1), lin(xn, P.w3))
        return x_mid + lin(g, P.w2)

    def _decode_token(self):
        """One token through every layer at the device-side position; leaves the fp32 logits and the
        arg-max in the static outputs and advances the position counters."""
        model, at = self.m, self.pos
        cos_p, sin_p = model.rope_cos.index_select(0, at), model.rope_sin.index_select(0, at)
        stream = model.tok_emb(self.tok)
        if self.fused:
            cos_f, sin_f = self.cos32.index_select(0, at), self.sin32.index_select(0, at)
        for l, blk in enumerate(model.blocks):
            if self.fused:
                stream = self._fused_layer(blk, l, stream.to(self.dt), cos_f, sin_f)
                continue
            stream = stream + self._attn(blk.attn, blk.attn_norm(stream), l, cos_p, sin_p)
            stream = stream + blk.mlp(blk.mlp_norm(stream))
        scores = model.lm_head(model.norm_f(stream)).float()
        self.logits.copy_(scores)
        torch.argmax(scores, dim=-1, out=self.next)
        for counter in (self.pos, self.pos32):
            counter.add_(1)

    def _eager_token(self):
        on_gpu = self.dev.type == "cuda" and self.dt == torch.bfloat16
        with torch.no_grad(), torch.autocast(self.dev.type, dtype=torch.bfloat16, enabled=on_gpu, cache_enabled=False):
            self._decode_token()

    def capture(self, warm_tokens=3):
        """Record one decode step as a CUDA graph (a no-op on CPU).  A few eager tokens on a side stream
        first, so lazy initialisation (library handles, autotuned plans) stays out of the recording."""
        if self.dev.type == "cuda":
            main, side = torch.cuda.current_stream(self.dev), torch.cuda.Stream(device=self.dev)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                for _ in range(warm_tokens):
                    self._eager_token()
            main.wait_stream(side)
            self.reset()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._eager_token()
            self.reset()
        return self

    def reset(self):
        """Empty tape, position 0."""
        for t in [self.pos, self.pos32, *self.K, *self.V]:
            t.zero_()

    def step(self):
        """Consume `self.tok` at the current position (graph replay when recorded)."""
        (self._eager_token if self.graph is None else self.graph.replay)()

    @torch.no_grad()
    def prefill(self, prompt):
        """Token-by-token prefill (the tape is recurrent: row t depends on the read at t)."""
        for column in prompt.split(1, dim=1):
            self.tok.copy_(column)
            self.step()

    @torch.no_grad()
    def generate(self, prompt, max_new, eos_id=None, stop_fn=None, check_every=16):
        """Greedy continuation.  prompt [B, L] on the device, all rows the same length.
        Returns (gen [B, k] on CPU, k = steps run).  `stop_fn(gen_cpu) -> bool [B]` marks
        finished rows; generation ends when every row is finished.  The host looks at the
        generated tokens only every `check_every` steps, so the launches in between queue freely."""
        rows, plen = prompt.shape
        if rows != self.B or plen + max_new > self.P:
            raise ValueError(f"prompt {tuple(prompt.shape)} + {max_new} new tokens does not fit [{self.B}, {self.P}]")
        self.reset()
        self.prefill(prompt)
        out = torch.zeros(rows, max_new, dtype=torch.long, device=self.dev)
        finished = torch.zeros(rows, dtype=torch.bool)
        for n in range(1, max_new + 1):
            out[:, n - 1] = self.next[:, 0]                    # the prediction made by the previous step
            if n % check_every == 0 or n == max_new:
                seen = out[:, :n].cpu()
                if eos_id is not None:
                    finished |= (seen == eos_id).any(dim=1)
                if stop_fn is not None:
                    finished |= stop_fn(seen)
                if finished.all():
                    return seen, n
            if n < max_new:
                self.tok.copy_(self.next)
                self.step()
        return out.cpu(), max_new
