"""Diagonal-wavefront engine: K sweeps per chunk with a sliding window of K in-flight chunks.

The operator (per layer).  The sequence is cut into chunks of C positions.  At step s the window holds
chunks lo = max(0, s-K+1) .. hi = min(s, n-1); every window chunk does ONE sweep, all against the tape
as it stood after step s-1:

    read   position t of chunk i attends  tape rows < i*C (committed chunks AND the in-flight window
           chunks before i, whatever version they are at), the strictly-lower rows of its own chunk
           (raw at the chunk's first sweep, else its previous refinement) and its own RAW key/value
    write  (k'', v'') = refine_kv(read) replaces the chunk's tape rows

A chunk enters raw at step i, is swept at steps i .. i+K-1, and its K-th refinement is its commit; the
read of its K-th sweep is the layer's attention output.  Unlike the layer-major cell engine
(`wavescan.py`), a chunk starts sweeping while its K-1 predecessors are still moving.

Schedule on B200.  The reference pipelines all layers' wavefronts K steps apart so that the per-step ops
can be batched over ~L layers, because it runs micro-batches of 4 sequences
(engines/wave3d/wave3d.py:1-45, wave3d_x.py:738-1161).  The operator itself has no cross-layer coupling
beyond "layer l+1 reads layer l's output", so here a layer runs its whole wavefront before the next one
starts (identical numerics), the micro-batch supplies the parallelism, the full-sequence projections
stay large GEMMs, and the engine shares everything else (packs, CUDA graphs, flat gradients, deferred
packed-weight gradient, head) with `WaveScanEngine`.

Far / near split of the read.  For chunk i the tape rows before (i-K+1)*C are committed before the
chunk enters and never change again: their softmax partial (o_far, lse_far) is computed ONCE per chunk and
merged into all K sweeps by log-sum-exp, instead of re-reading the whole prefix every sweep as one
lower-right-causal attention call per step does (wave3d_x.py `_AttendGroup`).  Only the K-1 chunks just
before i ("near") are re-read per sweep.  Attention work per chunk drops from K full-prefix passes to one
full-prefix pass plus K passes over at most (K-1)*C + C keys.

Backward.  Reverse over steps.  The tape is rolled back one version per step (every version of the
current layer is kept from a forward re-run, so memory is one layer's worth), gradients of tape rows
wait in a pending fp32 buffer until the sweep that produced that version is reached, far reads are
back-propagated owner-computes once per chunk (`prefix_dkv` over all far readers), near reads by a
gather per (step, key chunk).  No atomics; every accumulation has one owner.

`wavefront_layer_reference` is the same operator in plain autograd torch through `refine_kv`
(any configuration); it is the oracle of the fused path and the generic backend.

Reference parity: engines/wave3d/wave3d.py:213-543 (operator, schedule `n_steps = n - 1 + L*K` per
pipeline = `n + K - 1` per layer), wave3d_x.py:738-1471 (production engine: write-once caches, (o, lse)
stash, deferred dW), lm/train_1p3b/validate_rawdiag.py (exactness protocol, raw diagonal).
"""

from __future__ import annotations

import torch

from ..models.rope import apply_rope
from .cell import PrefixRead, intra_mask, merged_read
from .wavescan import WaveScanEngine

NEG = -1e30


# =================================================================================================
# plain-torch statement of the operator (autograd; every config knob through refine_kv)
# =================================================================================================
def wavefront_layer_reference(attn, xhat, cos, sin, C, K):
    """One layer's wavefront.  xhat [B,T,d] (normed input).  Returns (o_cat [B,T,d], K_rows, V_rows
    [B,h,T,dh]): the attention output and the committed tape."""
    B, T, _ = xhat.shape
    assert T % C == 0, "sequence length must be a whole number of chunks"
    n, W = T // C, attn.cfg.local_window or 0
    assert W == 0 or W >= T, "the wavefront statement covers full attention"
    mask = intra_mask(C, xhat.device, 0)
    q_r = apply_rope(attn._split(attn.wq(xhat)), cos, sin)
    k_flat, v_flat = attn.wk(xhat), attn.project_v(xhat)
    ks_r, v_raw = apply_rope(attn._split(k_flat), cos, sin), attn._split(v_flat)
    rows = [slice(i * C, (i + 1) * C) for i in range(n)]
    Kv = [ks_r[:, :, r] for r in rows]                   # current version of every chunk (raw before entry)
    Vv = [v_raw[:, :, r] for r in rows]
    o_fin = [None] * n
    for s in range(n + K - 1):
        lo, hi = max(0, s - K + 1), min(s, n - 1)
        new = {}
        for i in range(lo, hi + 1):
            r = rows[i]
            Kp = torch.cat(Kv[:i], dim=2) if i else None
            Vp = torch.cat(Vv[:i], dim=2) if i else None
            pre = PrefixRead(q_r[:, :, r], Kp, Vp, attn.scale, 0)
            o = merged_read(q_r[:, :, r], ks_r[:, :, r], v_raw[:, :, r], Kv[i], Vv[i], pre, mask, attn.scale)
            o_cat = attn._merge(o)
            kpp, vpp = attn.refine_kv(xhat[:, r], o_cat, k_flat[:, r], v_flat[:, r])
            new[i] = (apply_rope(attn._split(kpp), cos[r], sin[r]), attn._split(vpp))
            if s == i + K - 1:
                o_fin[i] = o_cat
        for i, (a, b) in new.items():                     # Jacobi across the window: publish after the step
            Kv[i], Vv[i] = a, b
    return torch.cat(o_fin, dim=1), torch.cat(Kv, dim=2), torch.cat(Vv, dim=2)


def wavefront_model_forward(model, idx, C, K):
    """Whole model through the wavefront operator -> logits [B,T,V] (autograd)."""
    x = model.tok_emb(idx)
    T = x.shape[1]
    cos, sin = model.rope_cos[:T], model.rope_sin[:T]
    for blk in model.blocks:
        o, _, _ = wavefront_layer_reference(blk.attn, blk.attn_norm(x), cos, sin, C, K)
        x = x + blk.attn.wo(o)
        x = x + blk.mlp(blk.mlp_norm(x))
    return model.lm_head(model.norm_f(x))


def _merge_partials(o_a, lse_a, o_b, lse_b):
    """Log-sum-exp merge of two softmax partials ([B,c,h,dh] fp32, [B,c,h] fp32)."""
    lse = torch.logaddexp(lse_a, lse_b)
    wa, wb = torch.exp(lse_a - lse), torch.exp(lse_b - lse)
    return wa.unsqueeze(-1) * o_a + wb.unsqueeze(-1) * o_b, lse, wa, wb


# =================================================================================================
# engine
# =================================================================================================
class Wave3DEngine(WaveScanEngine):
    """`WaveScanEngine` API (forward / backward / train_step / finish_grads / loss / grads / CUDA graphs)
    with the wavefront operator.  `ladder`: the sweep counts K selectable by `sid` (a K-ladder);
    `C`: chunk length."""

    MAX_SWEEPS = 1 << 20         # in-flight predecessors deepen the dependency chain: K may exceed C

    def __init__(self, model, ladder, B, T, C=64, **kw):
        ladder = [int(k) for k in (ladder if isinstance(ladder, (list, tuple)) else [ladder])]
        assert T % C == 0, "sequence length must be a whole number of chunks"
        assert (model.cfg.local_window or 0) in (0,) or model.cfg.local_window >= T, \
            "sliding-window attention is not covered by the wavefront engine"
        kw.setdefault("keep_sweeps", 0)
        # sweeps may exceed the chunk length here (in-flight predecessors deepen the dependency chain)
        super().__init__(model, [[(p, C, k) for p in range(0, T, C)] for k in ladder], B, T, **kw)
        self.ladder, self.C = ladder, C
        if self.backend == "fused":
            cfg, dev = self.cfg, self.device
            z = lambda *s, dt: torch.zeros(*s, dtype=dt, device=dev)
            h, dh = cfg.n_heads, cfg.head_dim
            # near-read backward inputs of the step being processed, indexed by absolute position
            self.docn_all = z(B, T, h, dh, dt=self.act)
            self.corrn_all = z(B, T, h, dt=torch.float32)
            self.lsen_all = z(B, T, h, dt=torch.float32)
            # gradient of the tape rows' current version, waiting for the sweep that wrote it
            self.dKp = z(B, T, h, dh, dt=torch.float32)
            self.dVp = z(B, T, h, dh, dt=torch.float32)
            self._versions = {}

    def _version_store(self, K):
        """Tape rows after 1 .. K-1 refinements of the layer in flight: [K-1, B, T, h, dh] x 2."""
        if K not in self._versions:
            cfg = self.cfg
            shape = (max(1, K - 1), self.B, self.T, cfg.n_heads, cfg.head_dim)
            self._versions[K] = (torch.zeros(shape, dtype=self.act, device=self.device),
                                 torch.zeros(shape, dtype=self.act, device=self.device))
        return self._versions[K]

    # ---- generic backend: autograd through the plain-torch operator (any configuration) -------------
    def _generic_forward(self, sid, have_targets):
        m, K = self.model, self.ladder[sid]
        with self._amp():
            x = m.tok_emb(self.idx)
            cos, sin = m.rope_cos[:self.T], m.rope_sin[:self.T]
            for li, blk in enumerate(m.blocks):
                self.xl[li].copy_(x)
                o, Kr, Vr = wavefront_layer_reference(blk.attn, blk.attn_norm(x), cos, sin, self.C, K)
                self.K_caches[li].copy_(Kr)
                self.V_caches[li].copy_(Vr)
                x = x + blk.attn.wo(o)
                x = x + blk.mlp(blk.mlp_norm(x))
            self.xl[self.L].copy_(x)
            if have_targets or self.keep_logits:
                self._generic_head(False, have_targets)

    def _generic_backward(self, sid, from_dlogits):
        m, G, K = self.model, self.grads, self.ladder[sid]
        cos, sin = m.rope_cos[:self.T], m.rope_sin[:self.T]
        self._generic_head(True, not from_dlogits, self.d_logits if from_dlogits else None)
        dx = self.dx_top.clone()
        for li in range(self.L - 1, -1, -1):
            blk = m.blocks[li]
            params = list(blk.parameters())
            with torch.enable_grad(), self._amp():
                x_in = self.xl[li].detach().requires_grad_(True)
                o, _, _ = wavefront_layer_reference(blk.attn, blk.attn_norm(x_in), cos, sin, self.C, K)
                x_mid = x_in + blk.attn.wo(o)
                x_next = x_mid + blk.mlp(blk.mlp_norm(x_mid))
            gs = torch.autograd.grad([x_next], [x_in] + params, [dx.to(x_next.dtype)], allow_unused=True)
            dx = gs[0]
            for p, g in zip(params, gs[1:]):
                G.add(p, g)
        G.get(m.tok_emb.weight).index_add_(0, self.idx.view(-1), dx.reshape(-1, self.cfg.d_model).float())

    # ---- forward ----------------------------------------------------------------------------------------
    def _wave_step_chunk(self, S, i, m, K, far, verK=None, verV=None, save=None):
        """One sweep of chunk i (its m-th, 0-based) against the tape as it stands.  Writes the new rows
        in place; with `save` also records what the backward needs."""
        ops, cfg = self.ops, self.cfg
        B, h, dh, d, C = self.B, cfg.n_heads, cfg.head_dim, cfg.d_model, self.C
        r = slice(i * C, (i + 1) * C)
        qc, ksc, vc4 = S.q_r[:, r], S.kself_r[:, r], S.v4[:, r]
        fe = max(0, i - K + 1) * C                              # far rows: [0, fe), near rows: [fe, i*C)
        if m == 0:
            far[i] = ops.prefix_fwd(qc, S.Kc, S.Vc, fe, S.scale, 0)
            K_in, V_in = ksc, vc4
        else:
            K_in, V_in = S.Kc[:, r], S.Vc[:, r]
        o_f, lse_f = far[i]
        if i * C - fe > 0:
            o_n, lse_n = ops.prefix_fwd(qc, S.Kc[:, fe:], S.Vc[:, fe:], i * C - fe, S.scale, 0)
            o_c, lse_c, w_f, w_n = _merge_partials(o_f, lse_f, o_n, lse_n)
        else:
            o_n = lse_n = w_f = w_n = None
            o_c, lse_c = o_f, lse_f
        o, lse, ssq = ops.tail_fwd(qc, ksc, vc4, K_in, V_in, o_c, lse_c, S.scale, 0)
        raw = ops.linear(o.reshape(B, C, d), S.P.W_pack)
        K_new, V_new = ops.refine_fwd(raw, ssq, S.glx[:, r], S.k[:, r], S.v[:, r], S.cos[r], S.sin[r], h, S.pin)
        S.Kc[:, r] = K_new
        S.Vc[:, r] = V_new
        if verK is not None and m + 1 <= K - 1:
            verK[m][:, r] = K_new                              # version after m+1 refinements
            verV[m][:, r] = V_new
        if m == K - 1 and getattr(S, "o_all", None) is not None:
            S.o_all[:, r] = o.reshape(B, C, d)
        if save is not None:
            save[(i, m)] = (o, lse, ssq, raw, o_c, lse_c, o_n, lse_n, w_f, w_n)

    def _cells_fwd(self, li, sid, S, keep):
        K, C = self.ladder[sid], self.C
        n = self.T // C
        far = {}
        for s in range(n + K - 1):
            lo, hi = max(0, s - K + 1), min(s, n - 1)
            for i in range(hi, lo - 1, -1):                     # descending: lower chunks are still at step s-1
                self._wave_step_chunk(S, i, s - i, K, far)
            if s - K + 1 >= 0:
                far.pop(s - K + 1, None)
            self.stats["fwd_cells"] += hi - lo + 1

    # ---- backward -------------------------------------------------------------------------------------------
    def _cells_bwd(self, li, sid, S, kept):
        ops, cfg = self.ops, self.cfg
        B, h, dh, d, C = self.B, cfg.n_heads, cfg.head_dim, cfg.d_model, self.C
        K, n = self.ladder[sid], self.T // self.C
        f32, dev = torch.float32, self.device
        Kc, Vc, scale = S.Kc, S.Vc, S.scale
        dcg_stash, u_stash, stash_off = self._stash_for(sid)
        verK, verV = self._version_store(K)
        # ---- forward re-run of this layer, keeping every version and every sweep's state
        far, save = {}, {}
        for s in range(n + K - 1):
            lo, hi = max(0, s - K + 1), min(s, n - 1)
            for i in range(hi, lo - 1, -1):
                self._wave_step_chunk(S, i, s - i, K, far, verK, verV, save)
        self.dKp.zero_()
        self.dVp.zero_()
        dq_c, DOf, DLf = {}, {}, {}
        rows = lambda i: slice(i * C, (i + 1) * C)
        for s in range(n + K - 2, -1, -1):
            lo, hi = max(0, s - K + 1), min(s, n - 1)
            # the chunk whose commit is this step: gather the far reads of its final rows (still on the tape)
            far_grad = None
            j = s - K + 1
            if j >= 0 and (j + K) * C < self.T:
                far_grad = ops.prefix_dkv(S.q_r, self.doc_all, self.corr_all, self.lsec_all, Kc, Vc,
                                          j * C, C, (j + K) * C, scale, 0)
            # roll the window back to the tape of step s-1
            for i in range(lo, hi + 1):
                m, r = s - i, rows(i)
                if m >= 1:
                    Kc[:, r] = verK[m - 1][:, r]
                    Vc[:, r] = verV[m - 1][:, r]
            for i in range(lo, hi + 1):
                m, r = s - i, rows(i)
                qc, ksc, vc4 = S.q_r[:, r], S.kself_r[:, r], S.v4[:, r]
                o, lse, ssq, raw, o_c, lse_c, o_n, lse_n, w_f, w_n = save.pop((i, m))
                o_f, lse_f = far[i]
                dK_out, dV_out = self.dKp[:, r].clone(), self.dVp[:, r].clone()
                if m == K - 1:
                    if far_grad is not None:
                        dK_out += far_grad[0]
                        dV_out += far_grad[1]
                    dq_c[i] = torch.zeros(B, C, h, dh, dtype=f32, device=dev)
                    DOf[i] = torch.zeros(B, C, h, dh, dtype=f32, device=dev)
                    DLf[i] = torch.zeros(B, C, h, dtype=f32, device=dev)
                off = stash_off[(i, m)]
                dcg = dcg_stash[off:off + B * C].view(B, C, 4 * d)
                ops.refine_bwd(dK_out, dV_out, raw, ssq, o.reshape(B, C, d), S.glx[:, r], S.k[:, r], S.v[:, r],
                               S.cos[r], S.sin[r], S.pin, S.dk[:, r], S.dv[:, r], S.dglx[:, r], dcg,
                               u_stash[off:off + B * C].view(B, C, d))
                du = ops.linear_dx(dcg, S.P.W_pack)
                d_o = ops.rmsn_bwd(du, o.reshape(B, C, d), ssq,
                                   residual=S.dO_all[:, r].float().reshape(B, C, d) if m == K - 1 else None
                                   ).view(B, C, h, dh)
                do_c = torch.zeros(B, C, h, dh, dtype=f32, device=dev)
                dlse_c = torch.zeros(B, C, h, dtype=f32, device=dev)
                K_in, V_in = (ksc, vc4) if m == 0 else (Kc[:, r], Vc[:, r])
                dK_in, dV_in = ops.tail_bwd(d_o, qc, ksc, vc4, K_in, V_in, o_c, lse_c, o, lse, scale, 0,
                                            dq_c[i], S.dks_r[:, r], S.dv4[:, r], do_c, dlse_c)
                if m == 0:                                      # the first sweep read the raw rows
                    S.dks_r[:, r] += dK_in
                    S.dv4[:, r] += dV_in
                    self.dKp[:, r] = 0
                    self.dVp[:, r] = 0
                else:
                    self.dKp[:, r] = dK_in
                    self.dVp[:, r] = dV_in
                # split d(o_c, lse_c) between the far and the near partial
                if o_n is None:
                    DOf[i] += do_c
                    DLf[i] += dlse_c
                else:
                    g_f = (do_c * (o_f - o_c)).sum(-1) + dlse_c
                    g_n = (do_c * (o_n - o_c)).sum(-1) + dlse_c
                    DOf[i] += w_f.unsqueeze(-1) * do_c
                    DLf[i] += w_f * g_f
                    do_n = w_n.unsqueeze(-1) * do_c
                    corr_n = (do_n * o_n).sum(-1) - w_n * g_n
                    self.docn_all[:, r] = do_n
                    self.corrn_all[:, r] = corr_n
                    self.lsen_all[:, r] = lse_n
                    fe = max(0, i - K + 1) * C
                    ops.prefix_dq(qc, Kc[:, fe:], Vc[:, fe:], i * C - fe, scale, 0, lse_n,
                                  self.docn_all[:, r], corr_n.contiguous(), dq_c[i])
                if m == 0:                                      # every sweep of chunk i has been processed
                    corr_f = (DOf[i] * o_f).sum(-1) - DLf[i]
                    self.doc_all[:, r] = DOf[i]
                    self.corr_all[:, r] = corr_f
                    self.lsec_all[:, r] = lse_f
                    fe = max(0, i - K + 1) * C
                    ops.prefix_dq(qc, Kc, Vc, fe, scale, 0, lse_f, self.doc_all[:, r], corr_f.contiguous(),
                                  dq_c[i])
                    S.dq_r[:, r] = dq_c.pop(i)
                    del DOf[i], DLf[i], far[i]
                self.stats["bwd_cells"] += 1
            # near reads of this step, key side: chunk j was read by window chunks (j, j+K-1]
            for j in range(max(0, lo - K + 1), hi):
                q0, q1 = max(j + 1, lo) * C, min(j + K, hi + 1) * C
                if q0 < q1:
                    dK, dV = ops.prefix_dkv(S.q_r, self.docn_all, self.corrn_all, self.lsen_all, Kc, Vc,
                                            j * C, C, q0, scale, 0, q_end=q1)
                    self.dKp[:, rows(j)] += dK
                    self.dVp[:, rows(j)] += dV
        return dcg_stash, u_stash
