"""Layer-major chunked training engine ("wavescan" class).

One layer at a time over the whole sequence: raw projections for all T
positions as large GEMMs, then the chunk cells in order (committed-prefix pass
once per cell, K Jacobi sweeps each = tail read -> RMSNorm -> packed ctx/gate
GEMM -> refine/rotate/write), then W_O and the SwiGLU block over all T.  The
backward is a reverse scan with exact per-cell recompute; gradients accumulate
in fp32 in one flat buffer shaped for the fused data-parallel update.

Two backends share the API:
  fused    hand-derived backward over the op table (`ops.TorchOps` on CPU,
           `ops.CudaOps` = sm_100a kernels on GPU).  Config family: linear ctx_mod,
           convex gates on [x̂;u], key and value modulation on, optional raw-value
           heads and sliding window, optional factored gates / ctx operators.
  generic  every knob, by re-running `cell.chunk_cell_forward` under autograd.

Reference parity: `WaveScanEngine` (engines/wavescan/engine/graphs.py:36-792) —
`forward / backward / train_step / finish_grads / debug_scan`, static buffers,
per-schedule CUDA graphs — and the reverse-scan backward of
engines/wavescan/engine/backward.py:87-206.
"""

from __future__ import annotations

import os
import time
from types import SimpleNamespace

import torch
import torch.nn.functional as F

from ..models.layers import LoRAGate, LoRALinear
from . import cell as gcell
from . import fused_math as fm
from .gradbuf import GradBuffers
from .schedule import check_schedule

FUSED_CTX_MODS = ("linear",)


def packed_refine_supported(cfg) -> bool:
    """The write law family with a fully hand-written refine step: one packed GEMM of the read, then the
    fused gate / blend / RoPE kernels and their explicit backward."""
    return (cfg.attn_mode != "vanilla" and cfg.enable_key_mod and cfg.enable_value_mod
            and cfg.ctx_mod in FUSED_CTX_MODS and cfg.gate_type == "convex_sigmoid"
            and cfg.gate_type_v == "convex" and cfg.gate_input == "xu" and cfg.rmsnorm_on_o
            and cfg.v_norm == "none" and cfg.v_ctx_norm == "none" and cfg.k_ctx_norm == "none"
            and not cfg.v_clamp_tau and not cfg.attn_logn_ref
            and (cfg.kmod_vraw_heads == 0 or (cfg.kmod_mode == "raw" and cfg.kmod_vraw_bound == "none")))


def mrk_refine_supported(cfg) -> bool:
    """The mult_res family of the reference's 1.3B recipe (wave3d_ops.check_cfg, engines/wave3d/wave3d_ops.py:31-43):
    multiplicative-residual value branch, per-head rms on the ctx key, optional value clamp and raw-pinned
    heads, convex sigmoid gates on [x;u]; any LoRA rank.  Explicit forward / backward (fused_math.mrk_*)."""
    return (cfg.attn_mode != "vanilla" and cfg.enable_key_mod and cfg.enable_value_mod
            and cfg.ctx_mod == "mult_res" and cfg.gate_type == "convex_sigmoid" and cfg.gate_type_v == "convex"
            and cfg.gate_input == "xu" and cfg.rmsnorm_on_o and cfg.k_ctx_norm == "rms"
            and cfg.v_norm == "none" and cfg.v_ctx_norm == "none" and not cfg.attn_logn_ref
            and (cfg.kmod_vraw_heads == 0 or (cfg.kmod_mode == "raw" and cfg.kmod_vraw_bound == "none")))


def refine_family(cfg) -> str:
    return "packed" if packed_refine_supported(cfg) else "mrk" if mrk_refine_supported(cfg) else "module"


def fused_supported(cfg) -> bool:
    """Configurations the kernel backend runs.  Outside the packed family the attention, projections,
    MLP and head still run on the kernels; only the per-sweep write law `refine_kv` (any ctx_mod, gate
    type, ctx norms, clamp, ...) runs as the module's own torch code on a compute-dtype copy of the layer,
    differentiated per sweep by autograd."""
    return (cfg.attn_mode != "vanilla" and cfg.dual_mod_active and cfg.v_norm == "none"
            and not cfg.attn_logn_ref and cfg.n_kv_heads_eff == cfg.n_heads)


def _dense(mod):
    """Dense [out, in] weight of a Linear / LoRALinear / LoRAGate."""
    if isinstance(mod, LoRAGate):
        return mod.dense_weight()
    return mod.weight


class _LayerPack:
    """Compute-dtype copies of one layer's weights in the layouts the ops want.
    Refreshed from the fp32 master parameters by `pack()` once per optimizer step."""

    def __init__(self, blk, cfg, dtype, device, family="packed"):
        d, hid = cfg.d_model, cfg.mlp_hidden
        mk = lambda *s: torch.empty(*s, dtype=dtype, device=device)
        self.family = family
        self.packed = packed = family != "module"
        self.factored = False
        n_in = 6 * d if family == "mrk" else 5 * d          # mrk: + the x-logits of the multiplicative branch's gate
        self.w_an, self.w_mn, self.w_ctx = mk(d), mk(d), mk(d)
        self.wo = mk(d, d)
        self.w1, self.w3, self.w2 = mk(hid, d), mk(hid, d), mk(d, hid)
        if not packed:
            # the write law runs as module code on `shadow`, a compute-dtype copy of the attention block
            import copy
            self.W_in, self.b_in = mk(3 * d, d), None
            self.wq, self.wk, self.wv = self.W_in[:d], self.W_in[d:2 * d], self.W_in[2 * d:]
            self.shadow = copy.deepcopy(blk.attn).to(device=device, dtype=dtype)
            skip = {"wq.weight", "wk.weight", "wv.weight", "wo.weight"}
            self.shadow_names = [n for n, _ in self.shadow.named_parameters() if n not in skip]
            self.shadow_set = set(self.shadow_names)
            for p_ in self.shadow.parameters():
                p_.requires_grad_(False)
            # fp32 gradient accumulators of the write law's weights, in the order of shadow_names
            src = dict(self.shadow.named_parameters())
            self.shadow_gacc = [torch.zeros_like(src[n], dtype=torch.float32) for n in self.shadow_names]
            return
        # one input projection for q, k, v and the x-half of both gates: [wq ; wk ; wv ; W_gx], bias
        # [0 ; 0 ; 0 ; b_g] -- a single GEMM forward, a single dX and a single dW GEMM backward
        self.W_in, self.b_in = mk(n_in, d), torch.zeros(n_in, dtype=dtype, device=device)
        self.wq, self.wk, self.wv = self.W_in[:d], self.W_in[d:2 * d], self.W_in[2 * d:3 * d]
        # When every operator of the write law is factored (LoRA), the sweeps apply the factors instead of the
        # composed d x d matrices: one GEMM onto the stacked down factors [sum of ranks, d], then one narrow
        # GEMM per operator from its rank columns to its d output columns.  2 (r_k + r_v + 2 r_g) / 4d of the
        # dense FLOPs, in the forward, the input gradient and the deferred weight gradients alike.
        a = blk.attn
        second = a.v_map if family == "mrk" else a.w_vctx
        ops4 = (a.w_kctx, second, a.w_gk, a.w_gv)
        self.factored = (all(isinstance(m, LoRALinear) for m in ops4[:2]) and all(isinstance(m, LoRAGate) for m in ops4[2:])
                         and (family != "mrk" or isinstance(a.w_vctx, LoRALinear))
                         and os.environ.get("DMB_DENSE_WRITE_LAW", "0") != "1")
        if self.factored:
            self.ranks = [a.w_kctx.down.weight.shape[0], second.down.weight.shape[0],
                          a.w_gk.a.weight.shape[0], a.w_gv.a.weight.shape[0]]
            self.factored = all(r % 8 == 0 for r in self.ranks) and (
                family != "mrk" or a.w_vctx.down.weight.shape[0] % 8 == 0)
        if self.factored:
            self.roff = [0]
            for r_ in self.ranks:
                self.roff.append(self.roff[-1] + r_)
            self.D_all = mk(self.roff[-1], d)                 # stacked down factors, context-norm gain folded in
            self.U = [mk(d, r_) for r_ in self.ranks]         # up factors
            self.W_pack = None
        else:
            self.W_pack = mk(4 * d, d)    # [W_kctx ; W_vctx (mrk: V_map) ; W_gk[:, d:] ; W_gv[:, d:]]
        self.W_gx = self.W_in[3 * d:5 * d]    # [W_gk[:, :d] ; W_gv[:, :d]]
        self.b_g = self.b_in[3 * d:5 * d]
        if family == "mrk":
            self.W_vgate, self.b_vgate = self.W_in[5 * d:], self.b_in[5 * d:]
            if self.factored:
                rv = a.w_vctx.down.weight.shape[0]
                self.Dv, self.Uv, self.W_vctx = mk(rv, d), mk(d, rv), None
            else:
                self.W_vctx = mk(d, d)
            self.k_gain = torch.ones(cfg.n_heads, dtype=torch.float32, device=device)

    @torch.no_grad()
    def pack(self, blk, cfg):
        a, d = blk.attn, cfg.d_model
        self.w_an.copy_(blk.attn_norm.weight)
        self.w_mn.copy_(blk.mlp_norm.weight)
        if self.packed:
            self.w_ctx.copy_(a.norm_ctx.weight)
        for dst, src in ((self.wq, a.wq), (self.wk, a.wk), (self.wv, a.wv), (self.wo, a.wo),
                         (self.w1, blk.mlp.w1), (self.w3, blk.mlp.w3), (self.w2, blk.mlp.w2)):
            dst.copy_(src.weight)
        if not self.packed:
            src = dict(a.named_parameters())
            for n, p_ in self.shadow.named_parameters():
                p_.copy_(src[n])
            return
        gk, gv = _dense(a.w_gk), _dense(a.w_gv)
        # the context-norm gain is folded into the packed weight's columns: the sweeps feed the
        # GEMM with the un-normalised read and apply 1/rms afterwards, row by row
        wc = a.norm_ctx.weight.float()[None, :]
        second = a.v_map if self.family == "mrk" else a.w_vctx
        if self.factored:
            downs = (a.w_kctx.down.weight, second.down.weight, a.w_gk.a.weight[:, d:], a.w_gv.a.weight[:, d:])
            ups = (a.w_kctx.up.weight, second.up.weight, a.w_gk.b.weight, a.w_gv.b.weight)
            for i, (dn, up) in enumerate(zip(downs, ups)):
                self.D_all[self.roff[i]:self.roff[i + 1]].copy_(dn.float() * wc)
                self.U[i].copy_(up)
        else:
            self.W_pack[:d].copy_(a.w_kctx.weight.float() * wc)
            self.W_pack[d:2 * d].copy_(second.weight.float() * wc)
            self.W_pack[2 * d:3 * d].copy_(gk[:, d:].float() * wc)
            self.W_pack[3 * d:].copy_(gv[:, d:].float() * wc)
        if self.family == "mrk":
            if self.factored:
                self.Dv.copy_(a.w_vctx.down.weight)
                self.Uv.copy_(a.w_vctx.up.weight)
            else:
                self.W_vctx.copy_(a.w_vctx.weight)
            self.W_vgate.copy_(a.v_gate.weight)
            self.b_vgate.copy_(a.v_gate.bias)
            self.k_gain.copy_(a.k_gain)
        self.W_gx[:d].copy_(gk[:, :d])
        self.W_gx[d:].copy_(gv[:, :d])
        self.b_g[:d].copy_(a.w_gk.bias)
        self.b_g[d:].copy_(a.w_gv.bias)


class WaveScanEngine:
    MAX_SWEEPS = None            # per cell: sweeps <= chunk length (K = c is already exact)

    def __init__(self, model, schedules, B, T, device=None, autocast_bf16=False,
                 keep_logits=False, loss_rows=4096, use_graphs=False, backend="auto",
                 ops=None, grad_bf16_ids=None, grad_alloc=None, grad_pad_to=1, sat_tau=0.0,
                 grads=None, on_layer_grads_final=None, keep_sweeps="auto"):
        cfg = model.cfg
        self.model, self.cfg = model, cfg
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.schedules = [list(s) for s in schedules]
        for s in self.schedules:
            check_schedule(s, T, self.MAX_SWEEPS)
        self.B, self.T, self.L = B, T, cfg.n_layers
        self.autocast_bf16 = autocast_bf16
        self.act = torch.bfloat16 if autocast_bf16 else torch.float32
        self.keep_logits = keep_logits
        self.loss_rows = loss_rows
        self.window = cfg.local_window or 0
        self.sat_tau = float(sat_tau)
        self.track_rho = False                       # set True to fill `chain_rho_max` without saturating
        self.chain_rho_max = torch.zeros((), dtype=torch.float32, device=self.device)
        assert not cfg.attn_logn_ref, "the engines do not implement the log-n logit scale"
        if backend == "auto":
            backend = "fused" if fused_supported(cfg) else "generic"
        if backend == "fused":
            assert fused_supported(cfg), "config outside the fused family; use backend='generic'"
        self.backend = backend
        if ops is None:
            from ..ops import default_ops
            ops = default_ops(self.device)
        from ..ops.checked import maybe_checked
        self.ops = maybe_checked(ops)                    # DMB_CHECK_ARGS=1: every launch's arguments are validated

        dev, act = self.device, self.act
        L, h, dh, d = self.L, cfg.n_heads, cfg.head_dim, cfg.d_model
        z = lambda *s, dt=act: torch.zeros(*s, dtype=dt, device=dev)
        self.idx = torch.zeros(B, T, dtype=torch.long, device=dev)
        self.targets = torch.zeros(B, T, dtype=torch.long, device=dev)
        self.xl = [z(B, T, d) for _ in range(L + 1)]          # layer inputs, xl[L] feeds norm_f
        self.loss = torch.zeros((), dtype=torch.float32, device=dev)
        self.grads = grads if grads is not None else GradBuffers(
            list(model.parameters()), bf16_ids=grad_bf16_ids, alloc=grad_alloc, pad_total_to=grad_pad_to)
        # called as fn(layer_index) right after a layer's parameter gradients are complete
        # (layer_index == -1: the head / final norm), so a data-parallel reducer can start
        # that layer's bucket while the reverse scan continues
        self.on_layer_grads_final = on_layer_grads_final
        self.dx_top = z(B, T, d)                               # d loss / d xl[L]
        self.dx_cur = z(B, T, d)                               # gradient flowing down the layers
        if keep_logits:
            self.logits = z(B, T, cfg.vocab_size)
            self.d_logits = z(B, T, cfg.vocab_size)
        if backend == "fused":
            # token-major tapes [B, T, h, dh]
            self.K_caches = [z(B, T, h, dh) for _ in range(L)]
            self.V_caches = [z(B, T, h, dh) for _ in range(L)]
            self.o_saved = [z(B, T, d) for _ in range(L)]      # last-sweep reads per layer
            # prefix-backward inputs of one layer, indexed by absolute position (reused per layer):
            # d o_c of every row, corr = d o_c . o_c - d lse_c, and lse_c
            self.doc_all = z(B, T, h, dh)
            self.corr_all = z(B, T, h, dt=torch.float32)
            self.lsec_all = z(B, T, h, dt=torch.float32)
            self.dK = self.dV = None
            self.family = refine_family(cfg)
            self.packed_refine = self.family != "module"      # packed GEMM + explicit backward (both kernel families)
            self.packs = [_LayerPack(b, cfg, act, dev, self.family) for b in model.blocks]
            self.emb_c = z(cfg.vocab_size, d)
            self.w_f = z(d)
            self.head_w = None if cfg.tie_embeddings else z(cfg.vocab_size, d)
            P0 = self.packs[0]
            self.factored = self.packed_refine and P0.factored
            self.dW_in = z(6 * d, d, dt=torch.float32)
            self.dW_gx = self.dW_in[3 * d:5 * d]
            if self.factored:
                # gradients of the factors: the up factors and the (folded) stacked down factors
                self.dU = [z(d, r_, dt=torch.float32) for r_ in P0.ranks]
                self.dD_all = z(P0.roff[-1], d, dt=torch.float32)
                self.dW_pack = None
            elif self.packed_refine:
                self.dW_pack = z(4 * d, d, dt=torch.float32)
            if refine_family(cfg) == "mrk":
                if self.factored:
                    rv = P0.Dv.shape[0]
                    self.dUv, self.dDv, self.dW_vctx = z(d, rv, dt=torch.float32), z(rv, d, dt=torch.float32), None
                else:
                    self.dW_vctx = z(d, d, dt=torch.float32)
                self.dkgain_acc = z(cfg.n_heads, dt=torch.float32)
                self.dwctx_acc = z(d, dt=torch.float32)
                self._stash2 = {}
            self._stash_fac = {}
            # committed-prefix partials of every cell, kept from the forward so the backward
            # does not redo the prefix pass: per schedule, [L][n_cells] dense slots
            self._prefix_saved = {}
            # per-layer stash of (d ctx/gate logits, u) of every sweep: the packed weight
            # gradient is ONE GEMM over all of a layer's sweep rows instead of one per sweep
            self._dw_stash = {}
            # per (schedule, layer): every sweep's (K_in, V_in, read, lse, ssq, ctx logits) kept from
            # a training forward, so the reverse scan starts each cell's backward at once instead
            # of re-running its sweeps.  `keep_sweeps`: number of layers (from layer 0) that keep
            # them, "auto" = as many as fit in about half of the device memory, 0 = recompute.
            self._sweep_saved = {}
            self._sweeps_valid = False
            self.keep_layers = self._keep_layers(keep_sweeps)
            self._packed = False
        else:
            self.K_caches = [z(B, h, T, dh) for _ in range(L)]
            self.V_caches = [z(B, h, T, dh) for _ in range(L)]
            self.dK = z(B, h, T, dh, dt=torch.float32)
            self.dV = z(B, h, T, dh, dt=torch.float32)
        self._sid = 0
        self._side, self._side_keep, self._side_used = None, [], False
        self.side_stream_ok = os.environ.get("DMB_SIDE_STREAM", "1") == "1"
        self._have_dx_top = False
        self.stats = {"fwd_cells": 0, "bwd_cells": 0}
        self.use_graphs = bool(use_graphs) and self.device.type == "cuda"
        self._graphs = {}
        self._graph_launches = {}
        self.capture_seconds = {}
        self.nvtx = os.environ.get("DMB_NVTX", "0") == "1" and self.device.type == "cuda"

    # =============================================================================
    # public API
    # =============================================================================
    def _keep_layers(self, keep_sweeps):
        if keep_sweeps != "auto":
            return max(0, min(self.L, int(keep_sweeps)))
        if self.device.type != "cuda":
            return self.L
        per_row = 7 * self.cfg.d_model * (2 if self.autocast_bf16 else 4)
        rows = max(self.B * sum(c * k for _, c, k in sch) for sch in self.schedules)
        room = 0.5 * torch.cuda.get_device_properties(self.device).total_memory
        return max(0, min(self.L, int(room // max(1, rows * per_row * len(self.schedules)))))

    def pack(self):
        """Refresh the compute-dtype weight copies from the master parameters."""
        if self.backend != "fused":
            return
        for p, blk in zip(self.packs, self.model.blocks):
            p.pack(blk, self.cfg)
        with torch.no_grad():
            self.emb_c.copy_(self.model.tok_emb.weight)
            self.w_f.copy_(self.model.norm_f.weight)
            if self.head_w is not None:
                self.head_w.copy_(self.model.lm_head.weight)
        self._packed = True

    def zero_grads(self):
        self.grads.zero_()
        self.chain_rho_max.zero_()

    @torch.no_grad()
    def forward(self, idx, targets=None, sid=0, train=False):
        """Chunked forward at schedule `sid`.  Returns the mean CE loss (fp32 scalar
        tensor) when targets are given, else None; with keep_logits the logits are
        in `self.logits`.  `train=True` also produces d loss / d x_L during the head
        pass so `backward()` needs no second head GEMM."""
        self.idx.copy_(idx)
        if targets is not None:
            self.targets.copy_(targets)
        self._sid = sid
        if self.backend == "fused":
            if not self._packed:
                self.pack()
            self._run("emb", 0, self._fused_embed)
            for li in range(self.L):
                keep = bool(train) and li < self.keep_layers
                self._run(("fwd", li, keep), sid, lambda li=li, keep=keep: self._fused_layer_fwd(li, sid, keep),
                          replay_after_capture=True)
            self._sweeps_valid = bool(train)
            if targets is not None or self.keep_logits:
                self._run(("head", bool(train), targets is not None), 0,
                          lambda: self._fused_head(train, targets is not None))
            self._have_dx_top = bool(train) and targets is not None
        else:
            self._generic_forward(sid, targets is not None)
            self._have_dx_top = False
        return self.loss if targets is not None else None

    @torch.no_grad()
    def backward(self, d_logits=None):
        """Reverse scan.  Default: gradient of the mean CE computed by `forward`.
        With `d_logits` [B,T,V] (needs keep_logits): gradient of an external loss."""
        if d_logits is not None:
            assert self.keep_logits, "explicit d_logits needs keep_logits=True"
            self.d_logits.copy_(d_logits)
        if self.backend == "fused":
            if d_logits is not None:
                self._fused_head_bwd_from_dlogits()
            elif not self._have_dx_top:
                self._fused_head(True, True)
            sid = self._sid
            self.dx_cur.copy_(self.dx_top)
            if self.on_layer_grads_final is not None:
                self.on_layer_grads_final(-1)
            for li in range(self.L - 1, -1, -1):
                kept = self._sweeps_valid and li < self.keep_layers
                self._run(("bwd", li, kept), sid, lambda li=li, kept=kept: self._fused_layer_bwd(li, sid, kept))
                if self.on_layer_grads_final is not None:
                    self.on_layer_grads_final(li)
            self._run("embb", 0, self._fused_embed_bwd)
        else:
            self._generic_backward(self._sid, d_logits is not None)
        self._have_dx_top = False

    def train_step(self, idx, targets, sid=0):
        """forward + backward of one micro-batch; gradients ACCUMULATE in the flat
        buffer (call `zero_grads()` at the start of an optimizer step)."""
        loss = self.forward(idx, targets, sid=sid, train=True)
        self.backward()
        return loss

    def finish_grads(self, world_size=1, process_group=None, bitwise_sync=True):
        """Average the flat gradient buffers over data-parallel ranks with library
        collectives (the baseline path; the fused reduce+AdamW kernels in
        `parallel.fused_optim` replace it) and expose them as `p.grad`.
        bitwise_sync: reduce to rank 0, divide, broadcast, so every rank holds
        identical bytes."""
        if world_size > 1:
            import torch.distributed as dist
            for flat in self.grads.flats:
                if bitwise_sync:
                    dist.reduce(flat, dst=0, group=process_group)
                    flat.div_(world_size)
                    dist.broadcast(flat, src=0, group=process_group)
                else:
                    dist.all_reduce(flat, group=process_group)
                    flat.div_(world_size)
        self.grads.to_param_grads()

    def debug_scan(self):
        """Names of persistent buffers holding non-finite values."""
        bad = []
        named = {"loss": self.loss, "dx_top": self.dx_top}
        if self.dK is not None:
            named["dK"], named["dV"] = self.dK, self.dV
        for i, t in enumerate(self.xl):
            named[f"xl[{i}]"] = t
        for i, (k, v) in enumerate(zip(self.K_caches, self.V_caches)):
            named[f"K[{i}]"], named[f"V[{i}]"] = k, v
        for i, f in enumerate(self.grads.flats):
            named[f"grads.flat[{i}]"] = f
        for name, t in named.items():
            if not torch.isfinite(t.float()).all():
                bad.append(name)
        return bad

    # =============================================================================
    # CUDA graphs
    # =============================================================================
    def _run(self, key, sid, body, replay_after_capture=False):
        """Run one phase of the step (embedding, a layer's forward, the head, a layer's backward, ...):
        eagerly, or as a CUDA graph recorded on first use.  With DMB_NVTX=1 every phase is an NVTX
        range named after its key, so a timeline shows the engine's phases."""
        if self.nvtx:
            torch.cuda.nvtx.range_push(f"dmb:{key}:sid{sid}")
        try:
            self._run_phase(key, sid, body, replay_after_capture)
        finally:
            if self.nvtx:
                torch.cuda.nvtx.range_pop()

    def _run_phase(self, key, sid, body, replay_after_capture):
        if not self.use_graphs:
            return body()
        gkey = (key, sid)
        g = self._graphs.get(gkey)
        if g is not None:
            g.replay()
            return
        # first use: run eagerly (this IS the step's result), then record the same
        # body for later replays; recording executes nothing, so accumulating bodies
        # (the backward) are not applied twice
        n0 = self.ops.launches
        body()
        self._graph_launches[gkey] = self.ops.launches - n0
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, pool=self._graphs.get("pool")):
            body()
        self._graphs.setdefault("pool", g.pool())
        self._graphs[gkey] = g
        # seconds spent recording, per schedule id (a trainer logs it once per rung)
        self.capture_seconds[sid] = self.capture_seconds.get(sid, 0.0) + time.perf_counter() - t0
        if replay_after_capture:
            # tensors the body left for later bodies now live in the graph's pool and were not
            # written by the recording: run the (idempotent) body once more through the graph
            g.replay()

    def graph_kernel_count(self):
        """Hand-written kernel launches recorded in the captured graphs of one
        forward + backward (replays do not pass through the op table's counter)."""
        return sum(self._graph_launches.values())

    def capture(self, sids=None):
        """Capture forward / head / backward graphs for the given schedule ids using
        the current buffer contents as dummy inputs, then zero the gradients."""
        if not self.use_graphs:
            return
        for sid in (range(len(self.schedules)) if sids is None else sids):
            self.train_step(self.idx.clone(), self.targets.clone(), sid=sid)
        self.zero_grads()

    # =============================================================================
    # fused backend
    # =============================================================================
    def _rows(self):
        return self.B * self.T

    def _fused_embed(self):
        self.xl[0].copy_(F.embedding(self.idx, self.emb_c))

    def _fused_embed_bwd(self):
        self.ops.embed_bwd(self.grads.get(self.model.tok_emb.weight), self.idx,
                           self.dx_cur.reshape(-1, self.cfg.d_model))

    def _fused_layer_fwd(self, li, sid, keep=False):
        ops, cfg = self.ops, self.cfg
        B, T, h, dh, d = self.B, self.T, cfg.n_heads, cfg.head_dim, cfg.d_model
        scale = 1.0 / dh ** 0.5
        cos, sin = self.model.rope_cos[:T], self.model.rope_sin[:T]
        pin = cfg.kmod_vraw_heads * dh
        if True:
            P = self.packs[li]
            x = self.xl[li]
            xhat, _ = ops.rms_fwd(x, P.w_an)
            qkvg = ops.linear(xhat, P.W_in, bias=P.b_in)
            k, v = qkvg[..., d:2 * d], qkvg[..., 2 * d:3 * d]
            glx = qkvg[..., 3 * d:5 * d] if self.packed_refine else None
            vgx = qkvg[..., 5 * d:] if self.family == "mrk" else None
            q_r = ops.rope(qkvg[..., :d].unflatten(-1, (h, dh)), cos, sin)
            kself_r = ops.rope(k.unflatten(-1, (h, dh)), cos, sin)
            Kc, Vc, o_all = self.K_caches[li], self.V_caches[li], self.o_saved[li]
            v4 = v.unflatten(-1, (h, dh))
            S = SimpleNamespace(P=P, q_r=q_r, kself_r=kself_r, v4=v4, k=k, v=v, glx=glx, Kc=Kc, Vc=Vc,
                                o_all=o_all, cos=cos, sin=sin, scale=scale, pin=pin, xhat=xhat, vgx=vgx)
            self._cells_fwd(li, sid, S, keep)
            x_mid = x + ops.linear(o_all, P.wo)
            xn, _ = ops.rms_fwd(x_mid, P.w_mn)
            g = ops.swiglu_fwd(ops.linear(xn, P.w1), ops.linear(xn, P.w3))
            self.xl[li + 1].copy_(x_mid + ops.linear(g, P.w2))

    def _cells_fwd(self, li, sid, S, keep):
        """The cells of one layer in order: committed-prefix read once per cell, K Jacobi sweeps, commit."""
        ops, cfg = self.ops, self.cfg
        B, h, dh, d = self.B, cfg.n_heads, cfg.head_dim, cfg.d_model
        P, q_r, kself_r, v4, k, v, glx = S.P, S.q_r, S.kself_r, S.v4, S.k, S.v, S.glx
        Kc, Vc, o_all, cos, sin, scale, pin = S.Kc, S.Vc, S.o_all, S.cos, S.sin, S.scale, S.pin
        saved = self._prefix_slots(sid, li)
        kept = [] if keep else None
        for ci, (pos0, c, n_sweeps) in enumerate(self.schedules[sid]):
            r = slice(pos0, pos0 + c)
            o_c, lse_c = ops.prefix_fwd(q_r[:, r], Kc, Vc, pos0, scale, self.window, out=saved[ci])
            K_in, V_in = kself_r[:, r], v4[:, r]
            o, st = None, []
            for s in range(n_sweeps):
                o, lse, ssq = ops.tail_fwd(q_r[:, r], kself_r[:, r], v4[:, r], K_in, V_in,
                                           o_c, lse_c, scale, self.window)
                # the last sweep's refinement is the commit: written straight into the tape rows
                last = s == n_sweeps - 1
                K_prev, V_prev = K_in, V_in
                K_in, V_in, raw = self._refine_fwd(S, r, o, ssq, out=(Kc[:, r], Vc[:, r]) if last else None)
                if keep:
                    # sweep 0 reads the raw rows, which the backward re-projects anyway
                    st.append((K_prev if s else None, V_prev if s else None, o, lse, ssq, raw))
            if keep:
                kept.append(st)
            o_all[:, r] = o.reshape(B, c, d)
            self.stats["fwd_cells"] += 1
        if keep:
            self._sweep_saved[(sid, li)] = kept

    # ---- the write law of one sweep -------------------------------------------------------------------
    # ---- the write law's two linear maps, dense or factored -----------------------------------------
    def _pack_linear(self, P, o2, t_out=None):
        """[k_ctx | v_ctx (mrk: v_map) | gate-k u-logits | gate-v u-logits] of the un-normalised read o2
        [B, c, d] -> [B, c, 4d].  Factored: the down outputs [rows, sum of ranks] are left in `t_out` when given."""
        ops = self.ops
        if not P.factored:
            return ops.linear(o2, P.W_pack)
        B, c, d = o2.shape
        t = ops.linear(o2.view(B * c, d), P.D_all, out=t_out, narrow=True).view(B * c, -1)
        raw = torch.empty(B, c, 4 * d, dtype=o2.dtype, device=o2.device)
        raw2 = raw.view(B * c, 4 * d)
        for i, U in enumerate(P.U):
            ops.linear(t[:, P.roff[i]:P.roff[i + 1]], U, out=raw2[:, i * d:(i + 1) * d], narrow=True)
        return raw

    def _pack_linear_dx(self, P, dcg, dt_out=None):
        """d (normalised read) [B, c, d] from d (packed logits) [B, c, 4d]; factored: also leaves
        d (down outputs) [rows, sum of ranks] in `dt_out` for the deferred gradient of the down factors."""
        ops = self.ops
        if not P.factored:
            return ops.linear_dx(dcg, P.W_pack)
        B, c, d4 = dcg.shape
        d = d4 // 4
        dcg2 = dcg.view(B * c, d4)
        dt = dt_out if dt_out is not None else torch.empty(B * c, P.roff[-1], dtype=dcg.dtype, device=dcg.device)
        for i, U in enumerate(P.U):
            ops.linear_dx(dcg2[:, i * d:(i + 1) * d], U, out=dt[:, P.roff[i]:P.roff[i + 1]], narrow=True)
        return ops.linear_dx(dt, P.D_all, narrow=True).view(B, c, d)

    def _vctx_linear(self, P, vin, tv_out=None):
        if not P.factored:
            return self.ops.linear(vin, P.W_vctx)
        B, c, d = vin.shape
        tv = self.ops.linear(vin.view(B * c, d), P.Dv, out=tv_out, narrow=True)
        return self.ops.linear(tv, P.Uv, narrow=True).view(B, c, d)

    def _refine_fwd(self, S, r, o, ssq, out=None, stash_row=None):
        """(k'', v'') rows [B, c, h, dh] from the read `o` of the rows `r` (key rotated), written into `out`
        when given.  Also returns what the backward wants besides (o, ssq): the packed ctx / gate logits
        in the packed family, nothing when the write law runs as module code.  `stash_row` (a forward re-run inside
        the backward): the deferred weight gradients' inputs that this forward computes anyway (the down outputs of the
        factors and, in the mult_res family, v_in) go straight into their stash rows starting there, so the backward
        of the same sweep does not compute them again (S.fwd_stashed)."""
        ops, cfg = self.ops, self.cfg
        B, h, dh, d = self.B, cfg.n_heads, cfg.head_dim, cfg.d_model
        c = o.shape[1]
        rows = slice(stash_row, stash_row + B * c) if stash_row is not None else None
        fac = rows is not None and S.P.factored
        if self.family == "packed":
            raw = self._pack_linear(S.P, o.reshape(B, c, d), S.t_stash[rows] if fac else None)
            K_new, V_new = ops.refine_fwd(raw, ssq, S.glx[:, r], S.k[:, r], S.v[:, r], S.cos[r], S.sin[r], h, S.pin,
                                          out=out)
            return K_new, V_new, raw
        if self.family == "mrk":
            o2 = o.reshape(B, c, d)
            raw = self._pack_linear(S.P, o2, S.t_stash[rows] if fac else None)
            vin = ops.mrk_vin_fwd(raw, ssq, o2, S.P.w_ctx, S.vgx[:, r], cfg.mult_res_lambda,
                                  out=S.vin_stash[rows].view(B, c, d) if rows is not None else None)
            vc = self._vctx_linear(S.P, vin, S.tv_stash[rows] if fac else None)
            K_new, V_new = ops.mrk_refine_fwd(raw, vc, ssq, S.glx[:, r], S.k[:, r], S.v[:, r], S.cos[r], S.sin[r], h,
                                              S.pin, S.P.k_gain, cfg.v_clamp_tau, out=out)
            return K_new, V_new, (raw, vc)
        with torch.no_grad(), self._amp():
            kpp, vpp = S.P.shadow.refine_kv(S.xhat[:, r], o.reshape(B, c, d), S.k[:, r], S.v[:, r])
        K_new = ops.rope(kpp.unflatten(-1, (h, dh)), S.cos[r], S.sin[r])
        V_new = vpp.unflatten(-1, (h, dh))
        if out is not None:
            out[0].copy_(K_new)
            out[1].copy_(V_new)
            return out[0], out[1], None
        return K_new, V_new, None

    def _down_outputs_of_uhat(self, S, rows, ssq, stashed):
        """t = D' uhat of one sweep's rows into the stash (input of the up factors' deferred weight gradient).  The
        forward's down outputs are D' o of the un-normalised read; when the forward re-run left them in the stash they
        only need the rows' 1 / rms, else the product is formed from the stashed uhat."""
        if not stashed:
            self.ops.linear(S.u_stash[rows], S.P.D_all, out=S.t_stash[rows], narrow=True)
            return
        rstd = fm.row_rstd(ssq.reshape(-1, ssq.shape[-1]), self.cfg.d_model)          # [rows, 1] fp32
        S.t_stash[rows].mul_(rstd)                                                    # fp32 product, one rounding

    def _refine_bwd(self, S, r, o, ssq, raw, dK_out, dV_out, stash_row, residual):
        """Backward of `_refine_fwd` for one sweep: returns d loss / d o [B, c, d] fp32 (plus `residual`)
        and accumulates the gradients of the layer-level inputs (S.dk, S.dv and, per family, the gate
        x-logits S.dglx or the normed input S.dxhat_acc) and of the write law's weights (packed family:
        stashed for one deferred GEMM per layer; module code: into the pack's fp32 accumulators)."""
        ops, cfg = self.ops, self.cfg
        B, h, dh, d = self.B, cfg.n_heads, cfg.head_dim, cfg.d_model
        c = o.shape[1]
        if self.family == "mrk":
            n, o2, P = B * c, o.reshape(B, c, d), S.P
            raw, vc = raw
            lam, rows = cfg.mult_res_lambda, slice(stash_row, stash_row + n)
            dcg = S.dcg_stash[rows].view(B, c, 4 * d)
            dvc = S.dvc_stash[rows].view(B, c, d)
            ops.mrk_refine_bwd(dK_out, dV_out, raw, vc, ssq, o2, S.glx[:, r], S.k[:, r], S.v[:, r], S.cos[r], S.sin[r],
                               S.pin, P.k_gain, cfg.v_clamp_tau, S.dk[:, r], S.dv[:, r], (S.dglx[:, r] if S.dglx is not None else None), dcg,
                               S.u_stash[rows].view(B, c, d), dvc, S.dkg_stash[rows].view(B, c, h))
            dvin = S.dvin_stash[rows].view(B, c, d)
            # v_in for the deferred W_vctx gradient (one GEMM per layer over all sweeps' rows): the forward re-run left
            # it in the stash, else it is formed again (cheap)
            stashed = getattr(S, "fwd_stashed", False)
            vin = S.vin_stash[rows]
            if not stashed:
                ops.mrk_vin_fwd(raw, ssq, o2, P.w_ctx, S.vgx[:, r], lam, out=vin.view(B, c, d))
            if P.factored:
                # stashes of the factored deferred gradients: down outputs and their gradients
                if not stashed:
                    ops.linear(vin, P.Dv, out=S.tv_stash[rows], narrow=True)
                ops.linear_dx(dvc.view(n, d), P.Uv, out=S.dtv_stash[rows], narrow=True)
                ops.linear_dx(S.dtv_stash[rows], P.Dv, out=dvin.view(n, d), narrow=True)
            else:
                dvin.copy_(ops.linear_dx(dvc, P.W_vctx))
            du_hat = ops.mrk_vin_bwd(dvin, raw, ssq, o2, P.w_ctx, S.vgx[:, r], lam, dcg, S.dvgx[:, r])
            du = self._pack_linear_dx(P, dcg, S.dt_stash[rows] if P.factored else None)
            if P.factored:
                self._down_outputs_of_uhat(S, rows, ssq, stashed)
            return ops.rmsn_bwd(du, o2, ssq, residual=residual, extra=du_hat)
        if self.family == "packed":
            n = B * c
            dcg = S.dcg_stash[stash_row:stash_row + n].view(B, c, 4 * d)
            ops.refine_bwd(dK_out, dV_out, raw, ssq, o.reshape(B, c, d), S.glx[:, r], S.k[:, r], S.v[:, r],
                           S.cos[r], S.sin[r], S.pin, S.dk[:, r], S.dv[:, r], (S.dglx[:, r] if S.dglx is not None else None), dcg,
                           S.u_stash[stash_row:stash_row + n].view(B, c, d))
            rows = slice(stash_row, stash_row + n)
            du = self._pack_linear_dx(S.P, dcg, S.dt_stash[rows] if S.P.factored else None)
            if S.P.factored:
                self._down_outputs_of_uhat(S, rows, ssq, getattr(S, "fwd_stashed", False))
            return ops.rmsn_bwd(du, o.reshape(B, c, d), ssq, residual=residual)
        from ..models.rope import apply_rope
        sh = S.P.shadow
        params = [p_ for n_, p_ in sh.named_parameters() if n_ in S.P.shadow_set]
        with torch.enable_grad(), self._amp():
            ins = [t.detach().requires_grad_(True) for t in (o.reshape(B, c, d), S.xhat[:, r], S.k[:, r], S.v[:, r])]
            for p_ in params:
                p_.requires_grad_(True)
            kpp, vpp = sh.refine_kv(ins[1], ins[0], ins[2], ins[3])
            K_new = apply_rope(kpp.view(B, c, h, dh).transpose(1, 2), S.cos[r], S.sin[r])
            V_new = vpp.view(B, c, h, dh)
        gs = torch.autograd.grad([K_new, V_new], ins + params,
                                 [dK_out.transpose(1, 2).to(K_new.dtype), dV_out.to(V_new.dtype)], allow_unused=True)
        for p_ in params:
            p_.requires_grad_(False)
        zero = lambda t: torch.zeros_like(t, dtype=torch.float32)
        d_o = gs[0].float() if gs[0] is not None else zero(ins[0])
        if gs[1] is not None:
            S.dxhat_acc[:, r] += gs[1]
        if gs[2] is not None:
            S.dk[:, r] += gs[2]
        if gs[3] is not None:
            S.dv[:, r] += gs[3]
        for acc, g_ in zip(S.P.shadow_gacc, gs[4:]):
            if g_ is not None:
                acc += g_
        return d_o if residual is None else d_o + residual

    def _prefix_slots(self, sid, li):
        """[(o_c [B,c,h,dh] fp32, lse_c [B,c,h] fp32)] per cell of layer li at schedule sid."""
        key = (sid, li)
        if key not in self._prefix_saved:
            cfg, f32 = self.cfg, torch.float32
            self._prefix_saved[key] = [
                (torch.zeros(self.B, c, cfg.n_heads, cfg.head_dim, dtype=f32, device=self.device),
                 torch.zeros(self.B, c, cfg.n_heads, dtype=f32, device=self.device))
                for _, c, _ in self.schedules[sid]]
        return self._prefix_saved[key]

    def _stash_for(self, sid):
        """(dcg stash [rows, 4d], u stash [rows, d], row offset of every (cell, sweep)) shared by all
        layers of a schedule; rows = B * sum_cells c * sweeps."""
        if sid not in self._dw_stash:
            d, offs, n = self.cfg.d_model, {}, 0
            for ci, (_, c, k) in enumerate(self.schedules[sid]):
                for s_ in range(k):
                    offs[(ci, s_)] = n
                    n += self.B * c
            self._dw_stash[sid] = (torch.zeros(n, 4 * d, dtype=self.act, device=self.device),
                                   torch.zeros(n, d, dtype=self.act, device=self.device), offs)
        return self._dw_stash[sid]

    def _stash2_for(self, sid):
        """(d v_c, v_in, d v_in) [rows, d] and the per-row k_gain gradient [rows, h] of every sweep of a layer:
        the mult_res family's W_vctx gradient is one deferred GEMM per layer like the packed weight's, and its
        two small reductions over rows (context-norm gain, k_gain) are done once per layer too."""
        if sid not in self._stash2:
            n = self._stash_for(sid)[0].shape[0]
            d, z = self.cfg.d_model, lambda w, dt: torch.zeros(n, w, dtype=dt, device=self.device)
            self._stash2[sid] = (z(d, self.act), z(d, self.act), z(d, self.act), z(self.cfg.n_heads, torch.float32))
        return self._stash2[sid]

    def _stash_fac_for(self, sid):
        """Factored write law: (down outputs of the normalised read, their gradients) [rows, sum of ranks] and,
        in the mult_res family, the same pair for the W_vctx factors [rows, rank] of every sweep of a layer."""
        if sid not in self._stash_fac:
            n, P = self._stash_for(sid)[0].shape[0], self.packs[0]
            z = lambda w: torch.zeros(n, w, dtype=self.act, device=self.device)
            rv = P.Dv.shape[0] if self.family == "mrk" else 0
            self._stash_fac[sid] = (z(P.roff[-1]), z(P.roff[-1]), z(rv) if rv else None, z(rv) if rv else None)
        return self._stash_fac[sid]

    def _head_weight(self):
        return self.emb_c if self.head_w is None else self.head_w

    def _head_grad_view(self):
        return self.grads.get(self.model.lm_head.weight)

    def _fused_head(self, train, have_targets):
        """norm_f + unembedding + fp32 CE over row slabs (no [B,T,V] tensor unless
        keep_logits); with train=True also d x_L and the head weight gradients."""
        ops, d = self.ops, self.cfg.d_model
        N = self._rows()
        x = self.xl[self.L].view(N, d)
        tg = self.targets.view(N)
        W = self._head_weight()
        inv_n = 1.0 / max(1, N) if not have_targets else None
        if have_targets:
            inv_n = 1.0 / (tg >= 0).sum().clamp_min(1).float()
        self.loss.zero_()
        dxt = self.dx_top.view(N, d)
        for r0 in range(0, N, self.loss_rows):
            r = slice(r0, min(N, r0 + self.loss_rows))
            xf, rstd = ops.rms_fwd(x[r], self.w_f)
            logits = ops.linear(xf, W)
            if self.keep_logits:
                self.logits.view(N, -1)[r] = logits
            if not have_targets:
                continue
            loss, dlog = ops.ce_chunk(logits, tg[r], inv_n)
            self.loss += loss
            if train:
                ops.linear_dw_acc(self._head_grad_view(), dlog, xf)
                dxf = ops.linear_dx(dlog, W)
                dxt[r] = ops.rms_bwd(dxf, x[r], self.w_f, rstd, self.grads.get(self.model.norm_f.weight),
                                     out_dtype=self.act)

    def _fused_head_bwd_from_dlogits(self):
        ops, d = self.ops, self.cfg.d_model
        N = self._rows()
        x, W = self.xl[self.L].view(N, d), self._head_weight()
        dl = self.d_logits.view(N, -1)
        dxt = self.dx_top.view(N, d)
        for r0 in range(0, N, self.loss_rows):
            r = slice(r0, min(N, r0 + self.loss_rows))
            xf, rstd = ops.rms_fwd(x[r], self.w_f)
            ops.linear_dw_acc(self._head_grad_view(), dl[r], xf)
            dxt[r] = ops.rms_bwd(ops.linear_dx(dl[r], W), x[r], self.w_f, rstd,
                                 self.grads.get(self.model.norm_f.weight), out_dtype=self.act)

    def _fused_layer_bwd(self, li, sid, kept=False):
        ops, cfg, G = self.ops, self.cfg, self.grads
        B, T, h, dh, d = self.B, self.T, cfg.n_heads, cfg.head_dim, cfg.d_model
        act, f32 = self.act, torch.float32
        scale = 1.0 / dh ** 0.5
        cos, sin = self.model.rope_cos[:T], self.model.rope_sin[:T]
        pin = cfg.kmod_vraw_heads * dh
        dev = self.device
        dx = self.dx_cur                                           # d loss / d x_{l+1}
        if True:
            P, blk = self.packs[li], self.model.blocks[li]
            a = blk.attn
            x = self.xl[li]
            o_all = self.o_saved[li]
            # ---- W_O + SwiGLU block, all T ------------------------------------------------
            x_mid = x + ops.linear(o_all, P.wo)
            xn, rstd_m = ops.rms_fwd(x_mid, P.w_mn)
            h1, h3 = ops.linear(xn, P.w1), ops.linear(xn, P.w3)
            g = ops.swiglu_fwd(h1, h3)
            ops.linear_dw_acc(G.get(blk.mlp.w2.weight), dx, g)
            dg = ops.linear_dx(dx, P.w2)
            dh1, dh3 = ops.swiglu_bwd(dg, h1, h3)
            ops.linear_dw_acc(G.get(blk.mlp.w1.weight), dh1, xn)
            ops.linear_dw_acc(G.get(blk.mlp.w3.weight), dh3, xn)
            dxn = ops.linear_dx(dh1, P.w1) + ops.linear_dx(dh3, P.w3)
            dx_mid = ops.rms_bwd(dxn, x_mid, P.w_mn, rstd_m, G.get(blk.mlp_norm.weight),
                                 residual=dx, out_dtype=act)
            ops.linear_dw_acc(G.get(a.wo.weight), dx_mid, o_all)
            dO_all = ops.linear_dx(dx_mid, P.wo).view(B, T, h, dh)
            # ---- recompute the layer projections ----------------------------------------------
            xhat, rstd_a = ops.rms_fwd(x, P.w_an)
            qkvg = ops.linear(xhat, P.W_in, bias=P.b_in)
            q, k, v = qkvg[..., :d], qkvg[..., d:2 * d], qkvg[..., 2 * d:3 * d]
            packed, mrk = self.packed_refine, self.family == "mrk"
            glx = qkvg[..., 3 * d:5 * d] if packed else None
            vgx = qkvg[..., 5 * d:] if mrk else None
            q_r = ops.rope(q.unflatten(-1, (h, dh)), cos, sin)
            kself_r = ops.rope(k.unflatten(-1, (h, dh)), cos, sin)
            v4 = v.unflatten(-1, (h, dh))
            Kc, Vc = self.K_caches[li], self.V_caches[li]
            # every cell's first backward sweep WRITES its rows of dq_r in the cell engine; the wavefront engine
            # accumulates into it from the first step on and needs the zeros
            dq_r = (torch.empty if type(self) is WaveScanEngine else torch.zeros)(B, T, h, dh, dtype=f32, device=dev)
            dks_r = torch.zeros(B, T, h, dh, dtype=f32, device=dev)
            dk = torch.zeros(B, T, d, dtype=f32, device=dev)
            dv = torch.zeros(B, T, d, dtype=f32, device=dev)
            # gradient of the gates' x-logits: equal, sweep by sweep, to the gate columns of the stashed
            # d(ctx / gate logits).  With a uniform schedule (every cell c rows, K sweeps: the stash rows are
            # ordered cell, sweep, batch, row) it is summed from the stash once per layer; otherwise the
            # refine backward accumulates it per sweep.
            sch = self.schedules[sid]
            from_stash = (packed and type(self) is WaveScanEngine and len({(c_, k_) for _, c_, k_ in sch}) == 1
                          and [p_ for p_, _, _ in sch] == list(range(0, T, sch[0][1])))
            dglx = torch.zeros(B, T, 2 * d, dtype=f32, device=dev) if packed and not from_stash else None
            dxhat_acc = None if packed else torch.zeros(B, T, d, dtype=f32, device=dev)
            dv4 = dv.view(B, T, h, dh)
            if not packed:
                for acc in P.shadow_gacc:
                    acc.zero_()
            elif self.factored:
                for t_ in self.dU + [self.dD_all]:
                    t_.zero_()
            else:
                self.dW_pack.zero_()
            S = SimpleNamespace(P=P, q_r=q_r, kself_r=kself_r, v4=v4, k=k, v=v, glx=glx, Kc=Kc, Vc=Vc,
                                cos=cos, sin=sin, scale=scale, pin=pin, dO_all=dO_all, dq_r=dq_r, dks_r=dks_r,
                                dk=dk, dv=dv, dglx=dglx, dv4=dv4, xhat=xhat, dxhat_acc=dxhat_acc, vgx=vgx)
            if mrk:
                S.dvgx = torch.zeros(B, T, d, dtype=f32, device=dev)
                S.dvc_stash, S.vin_stash, S.dvin_stash, S.dkg_stash = self._stash2_for(sid)
                for t_ in ((self.dUv, self.dDv) if self.factored else (self.dW_vctx,)) + (self.dkgain_acc, self.dwctx_acc):
                    t_.zero_()
            if self.factored:
                S.t_stash, S.dt_stash, S.tv_stash, S.dtv_stash = self._stash_fac_for(sid)
            dcg_stash, u_stash = self._cells_bwd(li, sid, S, kept)
            if packed:
                if self.factored:
                    # d U_i = d(logits_i)^T (down output_i);  d D' = d(down outputs)^T (normalised read)
                    for i, dU in enumerate(self.dU):
                        ops.linear_dw_acc(dU, dcg_stash[:, i * d:(i + 1) * d], S.t_stash[:, P.roff[i]:P.roff[i + 1]])
                    ops.linear_dw_acc(self.dD_all, S.dt_stash, u_stash)
                else:
                    ops.linear_dw_acc(self.dW_pack, dcg_stash, u_stash)
                if mrk:
                    if self.factored:
                        ops.linear_dw_acc(self.dUv, S.dvc_stash, S.tv_stash)
                        ops.linear_dw_acc(self.dDv, S.dtv_stash, S.vin_stash)
                    else:
                        ops.linear_dw_acc(self.dW_vctx, S.dvc_stash, S.vin_stash)
                    # u enters v_in directly as well: d w_ctx += lam * sum_rows(d v_in * uhat); k_gain: sum of the rows
                    ops.col_dot_acc(self.dwctx_acc, S.dvin_stash, u_stash)
                    self.dwctx_acc.mul_(cfg.mult_res_lambda)
                    ops.col_sum_acc(self.dkgain_acc, S.dkg_stash)
                self._unfold_packed_grad(a)
            # ---- close the layer: projections, gate-x logits, attn_norm -----------------------------
            n_in = P.W_in.shape[0]
            dY = torch.empty(B, T, n_in, dtype=act, device=dev)       # [dq | dk | dv (| dglx)]
            dY[..., :d] = ops.unrope(dq_r, cos, sin).reshape(B, T, d)
            dY[..., d:2 * d] = dk + ops.unrope(dks_r, cos, sin).reshape(B, T, d)
            dY[..., 2 * d:3 * d] = dv
            if packed:
                if from_stash:
                    dglx = ops.stash_gate_sum(dcg_stash, B, T, sch[0][1], sch[0][2])
                dY[..., 3 * d:5 * d] = dglx
            if mrk:
                dY[..., 5 * d:] = S.dvgx
            dW_in = self.dW_in[:n_in]
            dW_in.zero_()
            ops.linear_dw_acc(dW_in, dY, xhat)
            G.get(a.wq.weight).add_(dW_in[:d])
            G.get(a.wk.weight).add_(dW_in[d:2 * d])
            G.get(a.wv.weight).add_(dW_in[2 * d:3 * d])
            dxhat = ops.linear_dx(dY, P.W_in)
            if packed:
                db_g = torch.zeros(2 * d, dtype=f32, device=dev)
                ops.col_sum_acc(db_g, dglx)
            else:
                dxhat = (dxhat.float() + dxhat_acc).to(act)           # the write law read the normed input too
            self.dx_cur.copy_(ops.rms_bwd(dxhat, x, P.w_an, rstd_a, G.get(blk.attn_norm.weight),
                                          residual=dx_mid, out_dtype=act))
            if packed:
                self._scatter_packed_grads(a, db_g)
                if mrk:
                    self._scatter_mrk_grads(a, S.dvgx)
            else:
                master = dict(a.named_parameters())
                for name, acc in zip(P.shadow_names, P.shadow_gacc):
                    G.get(master[name]).add_(acc)

    def _cells_bwd(self, li, sid, S, kept):
        """Reverse scan over the cells of one layer.  Accumulates into S.dq_r / dks_r / dk / dv / dglx and
        returns the (d ctx-gate logits, u) stashes of every sweep for the deferred packed-weight GEMM."""
        ops, cfg = self.ops, self.cfg
        B, h, dh, d = self.B, cfg.n_heads, cfg.head_dim, cfg.d_model
        f32, dev = torch.float32, self.device
        P, q_r, kself_r, v4, k, v, glx = S.P, S.q_r, S.kself_r, S.v4, S.k, S.v, S.glx
        Kc, Vc, cos, sin, scale, pin = S.Kc, S.Vc, S.cos, S.sin, S.scale, S.pin
        dO_all, dq_r, dks_r, dk, dv, dglx, dv4 = S.dO_all, S.dq_r, S.dks_r, S.dk, S.dv, S.dglx, S.dv4
        # ---- cells in reverse ---------------------------------------------------------------
        saved = self._prefix_slots(sid, li)
        dcg_stash, u_stash, stash_off = self._stash_for(sid)
        S.dcg_stash, S.u_stash = dcg_stash, u_stash
        n_cells = len(self.schedules[sid])
        for ci in range(n_cells - 1, -1, -1):
            pos0, c, n_sweeps = self.schedules[sid][ci]
            r = slice(pos0, pos0 + c)
            qc, ksc, vc4 = q_r[:, r], kself_r[:, r], v4[:, r]
            o_c, lse_c = saved[ci]
            if kept:
                st = [(ksc, vc4) + t[2:] if t[0] is None else t for t in self._sweep_saved[(sid, li)][ci]]
            else:
                # forward recompute, keeping each sweep's state
                st = []
                K_in, V_in = ksc, vc4
                for _ in range(n_sweeps):
                    o, lse, ssq = ops.tail_fwd(qc, ksc, vc4, K_in, V_in, o_c, lse_c, scale, self.window)
                    K_new, V_new, raw = self._refine_fwd(S, r, o, ssq)
                    st.append((K_in, V_in, o, lse, ssq, raw))
                    K_in, V_in = K_new, V_new
            # gradient of this cell's committed rows from every later cell's prefix read
            dK_out, dV_out = ops.prefix_dkv(q_r, self.doc_all, self.corr_all, self.lsec_all, Kc, Vc,
                                            pos0, c, pos0 + c, scale, self.window)
            d_o = dO_all[:, r].float()
            if self.sat_tau > 0 or self.track_rho:
                dK_out, dV_out = self._saturate_carry(dK_out, dV_out, d_o)
            # per sweep only the intra-block products run (d q accumulates straight into the cell's rows of the layer's
            # array, the first sweep processed writes it); the row-scalar x row sums over the sweeps (d v_raw, d o_c,
            # d lse_c, the self column) are formed once, at the end of the cell, from the sweeps' kept d o
            scal = torch.empty(n_sweeps, 3, B, c, h, dtype=f32, device=dev)
            d_os = [None] * n_sweeps
            for s in range(n_sweeps - 1, -1, -1):
                K_in, V_in, o, lse, ssq, raw = st[s]
                d_o = self._refine_bwd(S, r, o, ssq, raw, dK_out, dV_out, stash_off[(ci, s)],
                                       d_o.view(B, c, d) if s == n_sweeps - 1 else None).view(B, c, h, dh)
                d_os[s] = d_o
                dK_out, dV_out = ops.tail_bwd_sweep(d_o, qc, ksc, K_in, V_in, lse_c, o, lse, scale, self.window,
                                                    dq_r[:, r], s == n_sweeps - 1, scal[s])
            # sweep 0 read the raw rows; publish this cell's (d o_c, corr, lse_c) for the earlier cells' gathers
            corr = ops.cell_finish_sweeps(d_os, scal, qc, ksc, vc4, o_c, lse_c, dK_out, dV_out, self.doc_all[:, r],
                                          self.corr_all[:, r], self.lsec_all[:, r], dks_r[:, r], dv4[:, r], dq_r[:, r],
                                          scale)
            del d_os
            # d q of the cell's prefix read touches only this cell's rows of dq_r and nothing the earlier cells
            # wait for: it runs beside their backward on a second stream (a parallel branch of the layer's graph)
            with self._beside(keep=(corr, lse_c)):
                ops.prefix_dq(qc, Kc, Vc, pos0, scale, self.window, lse_c, self.doc_all[:, r], corr, dq_r[:, r])
            self.stats["bwd_cells"] += 1
        self._join_beside()
        return dcg_stash, u_stash

    # ---- a second stream for work nothing downstream waits for ------------------------------------------
    def _beside(self, keep=()):
        """Context: launches inside run on the engine's side stream, ordered after everything launched so far on
        the main stream.  `keep`: tensors the side work reads that would otherwise be freed (and their memory
        reused by main-stream work) before it ran; they are held until `_join_beside`.  On CPU: a no-op."""
        import contextlib
        if self.device.type != "cuda" or not self.side_stream_ok:
            return contextlib.nullcontext()
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        self._side.wait_stream(torch.cuda.current_stream(self.device))
        self._side_keep.extend(keep)
        self._side_used = True
        return torch.cuda.stream(self._side)

    def _join_beside(self):
        """The main stream waits for the side stream's work (before anyone reads what it wrote)."""
        if self._side_used:
            torch.cuda.current_stream(self.device).wait_stream(self._side)
            self._side_keep.clear()
            self._side_used = False

    def _saturate_carry(self, dK, dV, d_o):
        """Gradient carried into a cell's committed rows from all later cells, measured against the
        gradient entering the cell directly: rho = (largest row norm of the carry) / (mean row norm of
        d o).  `chain_rho_max` keeps the largest rho of the backward (the LR governor's signal); with
        sat_tau > 0 rows of the carry above sat_tau x that mean are scaled down to it (direction kept,
        non-finite rows zeroed).  Reference parity: engines/wavescan/engine/graphs.py:345-371."""
        ref = d_o.norm(dim=-1).mean().clamp_min(1e-12)
        out = []
        for g in (dK, dV):
            g = torch.nan_to_num(g, nan=0.0, posinf=0.0, neginf=0.0)
            n = g.flatten(2).norm(dim=-1)                                   # [B, c] row norms over all heads
            self.chain_rho_max.copy_(torch.maximum(self.chain_rho_max, n.max() / ref))
            if self.sat_tau > 0:
                g = g * (self.sat_tau * ref / n.clamp_min(1e-20)).clamp(max=1.0)[..., None, None]
            out.append(g)
        return out

    def _unfold_packed_grad(self, a):
        """dW_pack holds the gradient of the FOLDED weight W' = W * w_ctx (per column).  Recover
        d w_ctx = sum_rows dW' * W and dW = dW' * w_ctx."""
        d = self.cfg.d_model
        second = a.v_map if self.family == "mrk" else a.w_vctx
        if self.family == "mrk":
            self.grads.get(a.norm_ctx.weight).add_(self.dwctx_acc)      # u also enters v_in directly
        if self.factored:
            # the same for the folded down factors D' = D * w_ctx
            D = torch.cat((a.w_kctx.down.weight, second.down.weight, a.w_gk.a.weight[:, d:], a.w_gv.a.weight[:, d:]),
                          dim=0).float()
            self.grads.get(a.norm_ctx.weight).add_((self.dD_all * D).sum(0))
            self.dD_all.mul_(a.norm_ctx.weight.float()[None, :])
            return
        gk, gv = _dense(a.w_gk), _dense(a.w_gv)
        W = torch.cat((a.w_kctx.weight, second.weight, gk[:, d:], gv[:, d:]), dim=0).float()
        self.grads.get(a.norm_ctx.weight).add_((self.dW_pack * W).sum(0))
        self.dW_pack.mul_(a.norm_ctx.weight.float()[None, :])

    def _scatter_packed_grads(self, a, db_g):
        """Route the packed-weight gradients of one layer to the parameters."""
        G, d = self.grads, self.cfg.d_model
        dWp, dWx = self.dW_pack, self.dW_gx
        second = a.v_map if self.family == "mrk" else a.w_vctx
        if self.factored:
            ro, dD = self.packs[0].roff, self.dD_all
            for i, mod in enumerate((a.w_kctx, second)):
                G.get(mod.up.weight).add_(self.dU[i])
                G.get(mod.down.weight).add_(dD[ro[i]:ro[i + 1]])
            for i, mod, rx in ((2, a.w_gk, slice(0, d)), (3, a.w_gv, slice(d, 2 * d))):
                # gate logits = b (a_x x + a_u u) + bias: the u half went through the factors, the x half
                # through the composed matrix of the layer's input projection
                a_w, b_w = mod.a.weight.float(), mod.b.weight.float()
                G.get(mod.b.weight).add_(self.dU[i] + dWx[rx] @ a_w[:, :d].t())
                ga = G.get(mod.a.weight)
                ga[:, :d].add_(b_w.t() @ dWx[rx])
                ga[:, d:].add_(dD[ro[i]:ro[i + 1]])
                G.get(mod.b.bias).add_(db_g[rx])
            return
        for mod, rows in ((a.w_kctx, slice(0, d)), (second, slice(d, 2 * d))):
            self._add_linear_grad(mod, dWp[rows])
        for mod, ru, rx, rb in ((a.w_gk, slice(2 * d, 3 * d), slice(0, d), slice(0, d)),
                                (a.w_gv, slice(3 * d, 4 * d), slice(d, 2 * d), slice(d, 2 * d))):
            dW = torch.cat((dWx[rx], dWp[ru]), dim=1)                 # [d, 2d] = [x half | u half]
            if isinstance(mod, LoRAGate):
                G.get(mod.b.weight).add_(dW @ mod.a.weight.float().t())
                G.get(mod.a.weight).add_(mod.b.weight.float().t() @ dW)
                G.get(mod.b.bias).add_(db_g[rb])
            else:
                G.get(mod.weight).add_(dW)
                G.get(mod.bias).add_(db_g[rb])

    def _add_linear_grad(self, mod, dW, db=None):
        """Route the gradient of a dense [out, in] weight to a Linear or to the two factors of a LoRALinear."""
        G = self.grads
        if isinstance(mod, LoRALinear):
            G.get(mod.up.weight).add_(dW @ mod.down.weight.float().t())
            G.get(mod.down.weight).add_(mod.up.weight.float().t() @ dW)
            if db is not None:
                G.get(mod.up.bias).add_(db)
        else:
            G.get(mod.weight).add_(dW)
            if db is not None:
                G.get(mod.bias).add_(db)

    def _scatter_mrk_grads(self, a, dvgx):
        """Weights only the mult_res family has: W_vctx (deferred GEMM), the gate of the multiplicative branch
        (rows 5d:6d of the input projection's gradient, bias = column sums of its logits' gradient), k_gain."""
        d = self.cfg.d_model
        if self.factored:
            self.grads.get(a.w_vctx.up.weight).add_(self.dUv)
            self.grads.get(a.w_vctx.down.weight).add_(self.dDv)
        else:
            self._add_linear_grad(a.w_vctx, self.dW_vctx)
        db = torch.zeros(d, dtype=torch.float32, device=self.device)
        self.ops.col_sum_acc(db, dvgx)
        self._add_linear_grad(a.v_gate, self.dW_in[5 * d:6 * d], db)
        self.grads.get(a.k_gain).add_(self.dkgain_acc)

    # =============================================================================
    # generic backend (every config knob; autograd re-run of the reference cell)
    # =============================================================================
    def _amp(self):
        return torch.autocast(self.device.type, dtype=torch.bfloat16,
                              enabled=self.autocast_bf16, cache_enabled=False)

    def _generic_forward(self, sid, have_targets):
        m = self.model
        with self._amp():
            x = m.tok_emb(self.idx)
            cos, sin = m.rope_cos[:self.T], m.rope_sin[:self.T]
            for li, blk in enumerate(m.blocks):
                self.xl[li].copy_(x)
                o = gcell.layer_forward(blk.attn, blk.attn_norm(x), cos, sin, self.schedules[sid],
                                        self.K_caches[li], self.V_caches[li])
                x = x + blk.attn.wo(o)
                x = x + blk.mlp(blk.mlp_norm(x))
                self.stats["fwd_cells"] += len(self.schedules[sid])
            self.xl[self.L].copy_(x)
            if have_targets or self.keep_logits:
                self._generic_head(False, have_targets)

    def _generic_head(self, with_grad, have_targets, d_logits=None):
        m, d = self.model, self.cfg.d_model
        N = self._rows()
        x, tg = self.xl[self.L].view(N, d), self.targets.view(N)
        hp = [m.norm_f.weight, m.lm_head.weight]
        inv_n = 1.0 / (tg >= 0).sum().clamp_min(1).float() if have_targets else None
        if not with_grad:
            self.loss.zero_()
        for r0 in range(0, N, self.loss_rows):
            r = slice(r0, min(N, r0 + self.loss_rows))
            with torch.set_grad_enabled(with_grad), self._amp():
                xr = x[r].detach().requires_grad_(with_grad)
                logits = m.lm_head(m.norm_f(xr))
                if self.keep_logits and not with_grad:
                    self.logits.view(N, -1)[r] = logits
                if d_logits is None and have_targets:
                    ls = F.cross_entropy(logits.float(), tg[r], ignore_index=-1,
                                         reduction="sum") * inv_n
            if not with_grad:
                if have_targets:
                    self.loss += ls
                continue
            if d_logits is None:
                gs = torch.autograd.grad([ls], [xr] + hp, allow_unused=True)
            else:
                gs = torch.autograd.grad([logits], [xr] + hp, [d_logits.view(N, -1)[r].to(logits.dtype)],
                                         allow_unused=True)
            self.dx_top.view(N, d)[r] = gs[0]
            for p, g in zip(hp, gs[1:]):
                self.grads.add(p, g)

    def _generic_backward(self, sid, from_dlogits):
        m, G = self.model, self.grads
        T = self.T
        cos, sin = m.rope_cos[:T], m.rope_sin[:T]
        self._generic_head(True, not from_dlogits, self.d_logits if from_dlogits else None)
        dx = self.dx_top.clone()
        for li in range(self.L - 1, -1, -1):
            blk = m.blocks[li]
            attn = blk.attn
            params = list(blk.parameters())
            x_l, Kc, Vc = self.xl[li], self.K_caches[li], self.V_caches[li]
            self.dK.zero_()
            self.dV.zero_()
            dx_l = torch.zeros_like(x_l)
            for pos0, c, n_sweeps in reversed(self.schedules[sid]):
                r = slice(pos0, pos0 + c)
                with torch.enable_grad(), self._amp():
                    x_c = x_l[:, r].detach().requires_grad_(True)
                    K_comm = Kc[:, :, :pos0].detach().requires_grad_(True)
                    V_comm = Vc[:, :, :pos0].detach().requires_grad_(True)
                    o_cat, K_rows, V_rows = gcell.chunk_cell_forward(
                        attn, blk.attn_norm(x_c), cos[r], sin[r], K_comm, V_comm, n_sweeps)
                    x_mid = x_c + attn.wo(o_cat)
                    x_next = x_mid + blk.mlp(blk.mlp_norm(x_mid))
                gs = torch.autograd.grad(
                    [x_next, K_rows, V_rows], [x_c, K_comm, V_comm] + params,
                    [dx[:, r].to(x_next.dtype), self.dK[:, :, r].to(K_rows.dtype),
                     self.dV[:, :, r].to(V_rows.dtype)], allow_unused=True)
                gx, gK, gV = gs[0], gs[1], gs[2]
                if self.sat_tau > 0:
                    gx, gK, gV = self._saturate(gx, gK, gV, dx[:, r])
                dx_l[:, r] = gx
                if pos0 > 0 and gK is not None:
                    self.dK[:, :, :pos0] += gK.float()
                    self.dV[:, :, :pos0] += gV.float()
                for p, g in zip(params, gs[3:]):
                    G.add(p, g)
                self.stats["bwd_cells"] += 1
            dx = dx_l
        G.get(m.tok_emb.weight).index_add_(0, self.idx.view(-1),
                                           dx.reshape(-1, self.cfg.d_model).float())

    def _saturate(self, gx, gK, gV, dx_in):
        """Saturating backward: cap each row of the gradients a cell hands to earlier
        positions at sat_tau x the norm of the gradient entering that row, keeping
        the direction; rows with non-finite entries become zero."""
        ref = dx_in.float().norm(dim=-1).mean().clamp_min(1e-12) * self.sat_tau

        def cap(g):
            if g is None:
                return g
            gf = torch.nan_to_num(g.float(), nan=0.0, posinf=0.0, neginf=0.0)
            n = gf.norm(dim=-1, keepdim=True)
            return (gf * (ref / n.clamp_min(1e-20)).clamp(max=1.0)).to(g.dtype)

        return cap(gx), cap(gK), cap(gV)
