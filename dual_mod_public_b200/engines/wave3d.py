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

One launch per op and step.  All chunks of the window sweep at once: the window's rows are contiguous in
time, so the packed GEMM, the refine chain and the norm backward see one [B, G*C, d] block, and the
attention kernels take a group dimension (grid z = chunk of the window, each with its own key range).

Backward.  Reverse over steps.  A forward re-run of the layer keeps what every step read from the tape's
window (so rolling the tape back one step is one block copy; memory is one layer's worth) and every
step's sweep state; gradients of tape rows wait in a pending fp32 buffer until the step that wrote that
version is reached; far reads are back-propagated owner-computes once per chunk (`prefix_dkv` over all
far readers), near reads by a gather per (step, key chunk).  No atomics; every accumulation has one owner.

`wavefront_layer_reference` is the same operator in plain autograd torch through `refine_kv`
(any configuration, sliding window included); it is the oracle of the fused path and the generic backend.

Reference parity: engines/wave3d/wave3d.py:213-543 (operator, schedule `n_steps = n - 1 + L*K` per
pipeline = `n + K - 1` per layer), wave3d_x.py:738-1471 (production engine: write-once caches, (o, lse)
stash, deferred dW), lm/train_1p3b/validate_rawdiag.py (exactness protocol, raw diagonal).
"""

from __future__ import annotations

import os

import torch

from ..models.rope import apply_rope
from .cell import PrefixRead, intra_mask, merged_read
from .wavescan import WaveScanEngine


# =================================================================================================
# plain-torch statement of the operator (autograd; every config knob through refine_kv)
# =================================================================================================
def wavefront_layer_reference(attn, xhat, cos, sin, C, K):
    """One layer's wavefront.  xhat [B,T,d] (normed input).  Returns (o_cat [B,T,d], K_rows, V_rows
    [B,h,T,dh]): the attention output and the committed tape."""
    B, T, _ = xhat.shape
    assert T % C == 0, "sequence length must be a whole number of chunks"
    n, W = T // C, attn.cfg.local_window or 0
    mask = intra_mask(C, xhat.device, W)
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
            pre = PrefixRead(q_r[:, :, r], Kp, Vp, attn.scale, W)
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
        kw.setdefault("keep_sweeps", 0)
        # every layer keeps the far partials (o_far, lse_far) of its chunks from the training forward, so the
        # forward re-run inside the backward skips the far reads (fp32 [B, T, d] + [B, T, h] per layer)
        keep_far = bool(kw.pop("keep_far", os.environ.get("DMB_KEEP_FAR", "1") == "1"))
        # sweeps may exceed the chunk length here (in-flight predecessors deepen the dependency chain)
        super().__init__(model, [[(p, C, k) for p in range(0, T, C)] for k in ladder], B, T, **kw)
        self.ladder, self.C = ladder, C
        self.keep_far = keep_far and self.backend == "fused"
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
            # far partial of every chunk (computed when it enters) and the accumulators of its gradient
            self._far = [(z(B, T, h, dh, dt=torch.float32), z(B, T, h, dt=torch.float32))
                         for _ in range(self.L if self.keep_far else 1)]
            self.ofar_all, self.lsefar_all = self._far[0]
            if self.keep_far:
                self.keep_layers = self.L          # `kept` in the backward = this layer's far partials are the forward's
            self.DOf_all = z(B, T, h, dh, dt=torch.float32)
            self.DLf_all = z(B, T, h, dt=torch.float32)
            self._versions = {}

    # ---- the reference engine's calling surface (engines/wave3d/wave3d.py:203 `make_engine`,
    #      wave3d_x.py:1292 `forward_logits`, :1287-1289 `stats`, :1383-1398 `mem`) ---------------------
    def sid_of_K(self, K):
        """Schedule id of sweep count K; a K outside the ladder is added as a new rung (its graphs are
        recorded on first use, like every rung's)."""
        K = int(K)
        if K not in self.ladder:
            self.ladder.append(K)
            self.schedules.append([(p, self.C, K) for p in range(0, self.T, self.C)])
        return self.ladder.index(K)

    def forward_K(self, idx, targets, K, train=False):
        """`forward(idx, targets, K)` of the reference engine: the mean CE at sweep count K (fp32 scalar
        tensor).  With train=True, `backward()` then accumulates the gradients (the reference calls
        `.backward()` on the returned loss; here the reverse pass is explicit)."""
        return self.forward(idx, targets, sid=self.sid_of_K(K), train=train)

    def forward_logits(self, idx, K):
        """Logits [B, T, V] of a no-grad forward at sweep count K (needs keep_logits=True)."""
        assert self.keep_logits, "forward_logits needs an engine built with keep_logits=True"
        self.forward(idx, None, sid=self.sid_of_K(K), train=False)
        return self.logits

    def set_compile(self, mode="all", dynamic=False):
        """Accepted for interface parity; there is no tracing compiler on this engine's path."""
        return self

    @property
    def mem(self):
        """Capture seconds per rung and the allocator's view of the device, as the reference's `engine.mem`."""
        out = {f"capture_K{self.ladder[s]}_s": round(sec, 2) for s, sec in self.capture_seconds.items()
               if s < len(self.ladder)}
        if self.device.type == "cuda":
            out["peak_gb"] = torch.cuda.max_memory_allocated(self.device) / 2 ** 30
            out["reserved_gb"] = torch.cuda.memory_reserved(self.device) / 2 ** 30
        return out

    def wave_stats(self, K):
        """Schedule counters of one layer's wavefront at sweep count K (`engine.stats` of the reference):
        steps per layer, the largest window and the rows swept per step."""
        n = self.T // self.C
        return {"steps": n + K - 1, "max_active": min(K, n), "rows_per_step": self.B * self.C * min(K, n),
                "layers": self.L, "chunks": n}

    def _window_store(self, K):
        """What every step read from the tape's window (K_in, V_in of all window chunks, the entering chunk
        raw): [steps, B, K*C, h, dh] x 2 for the layer in flight.  Rolling the tape back one step in the
        backward is one copy of a block."""
        if K not in self._versions:
            cfg = self.cfg
            shape = (self.T // self.C + K - 1, self.B, K * self.C, cfg.n_heads, cfg.head_dim)
            self._versions[K] = (torch.zeros(shape, dtype=self.act, device=self.device),
                                 torch.zeros(shape, dtype=self.act, device=self.device))
        return self._versions[K]

    def _step_offsets(self, K):
        """Row offset of every step's block in the (d logits, u) stashes of the deferred weight gradient."""
        n, offs, tot = self.T // self.C, [], 0
        for s in range(n + K - 1):
            offs.append(tot)
            tot += self.B * self.C * (min(s, n - 1) - max(0, s - K + 1) + 1)
        return offs

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
    def _far_arrays(self, li):
        self.ofar_all, self.lsefar_all = self._far[li if self.keep_far else 0]

    def _wave_step(self, S, s, K, save=None, win=None, far_kept=False):
        """Step s of one layer: the chunk entering (if any) computes its far partial and puts its raw rows
        on the tape; then ALL window chunks do one sweep in one launch per op (window tensors are
        [B, G*C, ...], G = chunks in the window) and their new rows replace the old ones."""
        ops, cfg = self.ops, self.cfg
        B, h, dh, d, C = self.B, cfg.n_heads, cfg.head_dim, cfg.d_model, self.C
        n = self.T // C
        lo, hi = max(0, s - K + 1), min(s, n - 1)
        G, w = hi - lo + 1, slice(lo * C, (hi + 1) * C)
        if s < n and not far_kept:
            # the entering chunk's far partial: it reads rows committed before this step and is needed by the merge
            # only, so it runs on the second stream beside the window's near read
            r = slice(s * C, (s + 1) * C)
            fe = max(0, s - K + 1) * C
            with self._beside():
                o_f, lse_f = ops.prefix_fwd(S.q_r[:, r], S.Kc, S.Vc, fe, S.scale, self.window, qoff=s * C - fe)
                self.ofar_all[:, r] = o_f
                self.lsefar_all[:, r] = lse_f
                del o_f, lse_f
            # (the chunk's raw rows are on the tape already: `_raw_tape` put every chunk's there before step 0)
        K_in, V_in = S.Kc[:, w], S.Vc[:, w]
        if win is not None:
            ops.copy_pair(win[0][s][:, :G * C], K_in, win[1][s][:, :G * C], V_in)
        qw = S.q_r[:, w]
        o_n, lse_n = ops.win_near_fwd(qw, S.Kc, S.Vc, lo * C, (lo - K + 1) * C, C, S.scale, self.window)
        self._join_beside()
        # (merging in the read kernel's epilogue, `win_near_merged`, measured slower than this kernel of its own)
        o_c, lse_c, w_f, w_n = ops.merge_partials(self.ofar_all[:, w], self.lsefar_all[:, w], o_n, lse_n)
        o, lse, ssq = ops.win_tail_fwd(qw, S.kself_r[:, w], S.v4[:, w], K_in, V_in, o_c, lse_c, C, S.scale, self.window)
        # every window chunk's new rows replace the old ones (all reads of this step are done)
        # (a forward re-run inside the backward also leaves the deferred weight gradients' inputs in their stash rows)
        _, _, raw = self._refine_fwd(S, w, o, ssq, out=(S.Kc[:, w], S.Vc[:, w]),
                                     stash_row=S.step_offs[s] if save is not None else None)
        if s - K + 1 >= 0 and getattr(S, "o_all", None) is not None:
            S.o_all[:, lo * C:(lo + 1) * C] = o[:, :C].reshape(B, C, d)      # chunk lo's K-th read is final
        if save is not None:
            save[s] = (o, lse, ssq, raw, o_c, lse_c, o_n, lse_n, w_f, w_n)
        self.stats["fwd_cells"] += G

    @staticmethod
    def _raw_tape(S):
        """Every chunk enters the wavefront raw.  No step reads tape rows at or beyond its window's last
        chunk, so all raw rows go onto the tape in one copy per tape before step 0 instead of one per step."""
        S.Kc.copy_(S.kself_r)
        S.Vc.copy_(S.v4)

    def _cells_fwd(self, li, sid, S, keep):
        K = self.ladder[sid]
        self._far_arrays(li)
        self._raw_tape(S)
        for s in range(self.T // self.C + K - 1):
            self._wave_step(S, s, K)

    # ---- backward -------------------------------------------------------------------------------------------
    def _cells_bwd(self, li, sid, S, kept):
        ops, cfg = self.ops, self.cfg
        B, h, dh, d, C = self.B, cfg.n_heads, cfg.head_dim, cfg.d_model, self.C
        K, n = self.ladder[sid], self.T // self.C
        f32, dev = torch.float32, self.device
        Kc, Vc, scale = S.Kc, S.Vc, S.scale
        dcg_stash, u_stash, _ = self._stash_for(sid)
        S.dcg_stash, S.u_stash = dcg_stash, u_stash
        offs = self._step_offsets(K)
        win = self._window_store(K)
        rows = lambda i: slice(i * C, (i + 1) * C)
        # ---- forward re-run of this layer, keeping what every step read and produced
        save = {}
        S.step_offs, S.fwd_stashed = offs, True
        self._far_arrays(li)
        self._raw_tape(S)
        for s in range(n + K - 1):
            self._wave_step(S, s, K, save, win, far_kept=bool(kept) and self.keep_far)
        for t in (self.dKp, self.dVp, self.DOf_all, self.DLf_all):
            t.zero_()
        # per-step scratch of the partial's gradient: written (not accumulated) by the tail kernel
        do_c_buf = torch.empty(B, K * C, h, dh, dtype=f32, device=dev)
        dlse_c_buf = torch.empty(B, K * C, h, dtype=f32, device=dev)
        # d o and the self column's scalars (p_self, dss) of the last K steps: a chunk's raw-row gradients
        # (d v_raw = sum over its sweeps of p_self dO, d k_self = (sum dss) q) are formed once, when its last sweep
        # has been processed, instead of read-modify-written by every step
        ring = {}
        # the gates' x-logit gradient is summed once per chunk from the stashed d(ctx / gate logits) of its K sweeps
        # (chunk end) instead of being accumulated by every step's refine backward
        dglx_full, S.dglx = S.dglx, None
        for s in range(n + K - 2, -1, -1):
            lo, hi = max(0, s - K + 1), min(s, n - 1)
            G, w, j = hi - lo + 1, slice(lo * C, (hi + 1) * C), s - K + 1
            # the chunk whose commit is this step: the far reads of its final rows (still on the tape) are
            # gathered straight into the pending gradient of those rows
            if j >= 0 and (j + K) * C < self.T:
                ops.prefix_dkv(S.q_r, self.doc_all, self.corr_all, self.lsec_all, Kc, Vc, j * C, C, (j + K) * C, scale,
                               self.window, out=(self.dKp[:, rows(j)], self.dVp[:, rows(j)]), accumulate=True)
            self._join_beside()                                 # the far d q of step s+1 read rows this window rolls back
            ops.copy_pair(Kc[:, w], win[0][s][:, :G * C], Vc[:, w], win[1][s][:, :G * C])   # the tape as step s read it
            o, lse, ssq, raw, o_c, lse_c, o_n, lse_n, w_f, w_n = save.pop(s)
            # gradient of the rows this step wrote: read in place (window views of the pending arrays)
            d_o = self._refine_bwd(S, w, o, ssq, raw, self.dKp[:, w], self.dVp[:, w], offs[s], None)
            if j >= 0:                                          # chunk j's K-th read is the layer's output
                d_o[:, :C] += S.dO_all[:, rows(j)].reshape(B, C, d)
            d_o = d_o.view(B, G * C, h, dh)
            do_c = do_c_buf[:, :G * C] if G == K else torch.empty(B, G * C, h, dh, dtype=f32, device=dev)
            dlse_c = dlse_c_buf[:, :G * C] if G == K else torch.empty(B, G * C, h, dtype=f32, device=dev)
            # gradient of what step s read = rows of step s-1: replaces the pending gradient of the window's
            # rows; d q goes straight into the layer's array
            stash = torch.empty(2, B, G * C, h, dtype=f32, device=dev)
            ring[s] = (d_o, stash, lo, dcg_stash[offs[s]:offs[s] + B * G * C].view(B, G * C, 4 * d))
            ops.win_tail_bwd(d_o, S.q_r[:, w], S.kself_r[:, w], S.v4[:, w], Kc[:, w], Vc[:, w], o_c, lse_c, o, lse, C,
                             scale, S.dq_r[:, w], S.dks_r[:, w], S.dv4[:, w], do_c, dlse_c, self.window, init=2,
                             dkv_out=(self.dKp[:, w], self.dVp[:, w]), raw_stash=stash)
            # split d(o_c, lse_c) between the far and the near partial
            corr_n = torch.empty(B, G * C, h, dtype=f32, device=dev)
            ops.split_partials(do_c, dlse_c, self.ofar_all[:, w], o_c, o_n, lse_n, w_f, w_n, self.DOf_all[:, w],
                               self.DLf_all[:, w], self.docn_all[:, w], self.corrn_all[:, w], self.lsen_all[:, w],
                               corrn_dense=corr_n)
            ops.win_near_dq(S.q_r[:, w], Kc, Vc, lo * C, (lo - K + 1) * C, C, scale, lse_n.contiguous(),
                            self.docn_all[:, w], corr_n, S.dq_r[:, w], self.window)
            if s < n:
                # chunk s entered at this step and every sweep of it has now been processed: what this step read of
                # it were its raw rows (their pending gradient moves to the raw-row gradients), and its far read's
                # gradient is complete
                r, fe = rows(s), max(0, s - K + 1) * C
                sweeps = []
                for k in range(K):                              # sweep k of chunk s ran at step s + k
                    g_o, g_st, g_lo, g_dcg = ring[s + k]
                    gr = rows(s - g_lo)
                    sweeps.append((g_o[:, gr], g_st[0][:, gr], g_st[1][:, gr]) + ((g_dcg[:, gr],) if dglx_full is not None else ()))
                corr_f, lse_f = ops.chunk_finish(self.DOf_all[:, r], self.DLf_all[:, r], self.ofar_all[:, r],
                                                 self.lsefar_all[:, r], self.dKp[:, r], self.dVp[:, r], S.dks_r[:, r],
                                                 S.dv4[:, r], self.doc_all[:, r], self.corr_all[:, r], self.lsec_all[:, r],
                                                 sweeps=sweeps, q=S.q_r[:, r],
                                                 dglx=dglx_full[:, r] if dglx_full is not None else None)
                del sweeps
                # d q of the far read: it writes only chunk s's rows of dq_r, which no later step of the reverse pass
                # touches, and runs on the second stream beside the key-side gathers that follow; it is joined
                # before the next step rolls tape rows back (some of its keys lie in that window)
                with self._beside(keep=(corr_f, lse_f)):
                    ops.prefix_dq(S.q_r[:, r], Kc, Vc, fe, scale, self.window, lse_f, self.doc_all[:, r], corr_f,
                                  S.dq_r[:, r], qoff=s * C - fe)
            # near reads of this step, key side: chunk jk was read by the window chunks in (jk, jk+K-1]
            j0 = max(0, lo - K + 1)
            if hi > j0:
                wk = slice(j0 * C, hi * C)
                ops.win_near_dkv(S.q_r, self.docn_all, self.corrn_all, self.lsen_all, Kc, Vc, j0, hi - j0, C,
                                 lo * C, (hi + 1) * C, K * C, scale, self.window,
                                 out=(self.dKp[:, wk], self.dVp[:, wk]), accumulate=True)
            ring.pop(s + K - 1, None)                           # chunk s - 1 needs the steps s - 1 .. s + K - 2 only
            self.stats["bwd_cells"] += G
        self._join_beside()
        S.dglx = dglx_full
        return dcg_stash, u_stash


def make_engine(model, B, T, engine="x", C=64, ladder=(8, 16, 32), **kw):
    """Factory with the reference's signature (engines/wave3d/wave3d.py:203): returns the wavefront engine
    for micro-batches of B sequences of length T.  `engine` is accepted for compatibility ("x" and "vmap"
    name two implementations of one operator in the reference; there is one here).  Keyword arguments of
    the reference that steer its memory policy or library kernels (`seg_steps`, `use_ckpt`, `attn_impl`,
    `n_snapshots`, `sac`, `store_frac`, `compile_bodies`, `fused`, `reentrant`, `stash_attn`, `defer_dw`,
    `fused_refine`) have no counterpart and are ignored; `graphs` maps to `use_graphs`, `local_window` must
    agree with the model's config (the window is part of the operator), `raw_diag` must be true or absent
    (a position always reads its own raw key / value here, which is what makes K = C consistent with the
    sequential scan's convention)."""
    ignored = ("seg_steps", "use_ckpt", "attn_impl", "n_snapshots", "sac", "store_frac", "compile_bodies", "fused",
               "reentrant", "stash_attn", "defer_dw", "fused_refine")
    kw = {k: v for k, v in kw.items() if k not in ignored}
    if "graphs" in kw:
        kw["use_graphs"] = bool(kw.pop("graphs"))
    assert kw.pop("raw_diag", True), "the refined-diagonal variant of the reference operator is not implemented"
    lw = kw.pop("local_window", None)
    assert not lw or int(lw) == int(model.cfg.local_window or 0), "local_window is read from the model's config"
    kw.setdefault("autocast_bf16", next(model.parameters()).is_cuda)
    return Wave3DEngine(model, list(ladder), B, T, C=C, **kw)
