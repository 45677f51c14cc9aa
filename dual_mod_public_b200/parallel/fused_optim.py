"""Data-parallel gradient reduction fused with AdamW, over NVLink peer memory.

`FusedDPAdamW` owns three flat fp32 arrays laid out bucket by bucket (one bucket
per layer, in the order the reverse-scan backward finishes them):

  grads   peer-mapped; the engines' `GradBuffers` views point into it
  params  peer-mapped master weights; `p.data` of every parameter is a view into it
  m, v    AdamW moments of the slices THIS rank owns (1/world of every bucket)

`step()` launches one cooperative kernel (csrc/fused_optim.cu) that reduce-scatters
the gradients with peer loads (fixed rank order, so every rank ends with identical
bytes), scales, forms the global norm across ranks through peer-mapped slots, clips,
applies the skip predicate, updates the owned slices and stores the new parameters
into every peer's buffer.  `reduce_bucket(b)` may be called earlier, on a side
stream, as soon as bucket b's gradients are final, so the reduce-scatter overlaps
the rest of the backward.

Replaces the reference's unfused chain `finish_grads` (reduce + div + broadcast of
one flat tensor, engines/wavescan/engine/graphs.py:768-792) or `GradAllReducer`
(lm/train_1p3b/train_hero_wave3d.py:314-352), then `clip_grad_norm_`, the skip
decision and `torch.optim.AdamW.step()`.  `NcclAdamW` is that baseline chain behind
the same interface.  With `nvls=True` (or DMB_NVLS=1) the gradient and parameter arrays are bound to an NVLink
multicast object instead and the two collective phases run as `multimem.ld_reduce` / `multimem.st` (the NVSwitch
adds and replicates); flags, waits and the status word are the same.  `state_dict()` gathers the sharded moments into the plain
torch AdamW layout, so checkpoints stay interchangeable.

Without a CUDA device (CPU tests, gloo ranks) the same bucket / slice / segment
plan runs through `_step_host`, a torch statement of the kernel.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from ..engines.gradbuf import GradBuffers, unique_params

MAX_WORLD, MAX_BUCKETS = 8, 64
SLOT_OPEN, SLOT_NORM, SLOT_CLOSE, SLOT_BUCKET0 = 0, 1, 2, 3
ALIGN = 64


class _Comm(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int),
                ("grads", ctypes.c_void_p * MAX_WORLD), ("params", ctypes.c_void_p * MAX_WORLD),
                ("flags", ctypes.c_void_p * MAX_WORLD), ("norms", ctypes.c_void_p * MAX_WORLD),
                ("mc_grads", ctypes.c_void_p), ("mc_params", ctypes.c_void_p)]


class _Plan(ctypes.Structure):
    _fields_ = [("n_buckets", ctypes.c_int), ("n_segs", ctypes.c_int),
                ("bucket_off", ctypes.c_longlong * MAX_BUCKETS),
                ("bucket_len", ctypes.c_longlong * MAX_BUCKETS),
                ("moment_off", ctypes.c_longlong * MAX_BUCKETS),
                ("reduced", ctypes.c_int * MAX_BUCKETS)]


class _Hyper(ctypes.Structure):
    _fields_ = [("lr", ctypes.c_float), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float),
                ("eps", ctypes.c_float),
                ("grad_scale", ctypes.c_float), ("max_norm", ctypes.c_float),
                ("skip_norm", ctypes.c_float), ("epoch", ctypes.c_uint),
                ("wait_cycles", ctypes.c_longlong)]


class _RawCuda:
    """Exposes a raw device pointer to torch through the CUDA array interface."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2}


class PeerWaitExpired(RuntimeError):
    """A bounded cross-GPU wait of the optimizer kernels ran out (a peer is lost or far behind)."""


def _ck(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: CUDA error {rc}")


class PeerBuffer:
    """A device allocation mapped into every rank of the group (CUDA IPC, one process per
    GPU on one node).  `ptrs[r]` is rank r's buffer as seen from this process."""

    def __init__(self, lib, nbytes, device, group, rank, world):
        self.lib, self.nbytes, self.rank, self.world = lib, nbytes, rank, world
        self._opened = []
        own = ctypes.c_void_p()
        with torch.cuda.device(device):
            _ck(lib.dmb_ipc_alloc(ctypes.c_size_t(nbytes), ctypes.byref(own)), "ipc alloc")
            self.own = own.value
            self.ptrs = [None] * world
            self.ptrs[rank] = self.own
            if world > 1:
                hsz = lib.dmb_ipc_handle_size()
                buf = ctypes.create_string_buffer(hsz)
                _ck(lib.dmb_ipc_get_handle(ctypes.c_void_p(self.own), buf), "ipc handle")
                handles = [None] * world
                dist.all_gather_object(handles, bytes(buf.raw), group=group)
                for r, h in enumerate(handles):
                    if r == rank:
                        continue
                    p = ctypes.c_void_p()
                    _ck(lib.dmb_ipc_open(ctypes.create_string_buffer(h, hsz), ctypes.byref(p)),
                        f"ipc open (rank {r})")
                    self.ptrs[r] = p.value
                    self._opened.append(p.value)
        self._holder = _RawCuda(self.own, nbytes)
        try:
            self.bytes_tensor = torch.as_tensor(self._holder, device=device)
        except Exception:
            storage = torch._C._construct_storage_from_data_pointer(self.own, torch.device(device), nbytes)
            self.bytes_tensor = torch.empty(0, dtype=torch.uint8, device=device).set_(storage)
        assert self.bytes_tensor.data_ptr() == self.own and self.bytes_tensor.numel() == nbytes

    def view(self, dtype, numel=None):
        t = self.bytes_tensor.view(dtype)
        return t if numel is None else t[:numel]

    def close(self):
        for p in self._opened:
            self.lib.dmb_ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if self.own:
            self.lib.dmb_ipc_free(ctypes.c_void_p(self.own))
            self.own = None


class MulticastBuffer:
    """The same surface as `PeerBuffer`, with the memory taken from torch's symmetric-memory allocator and bound to
    an NVLink multicast object: `mc` is the multicast address (one multimem.ld_reduce reads the sum over all ranks,
    one multimem.st writes to all ranks), `ptrs[r]` rank r's copy as seen from this process.  Raises when the
    group has no multicast mapping (no NVSwitch, or NVLS not available to this process)."""

    def __init__(self, nbytes, device, group, rank, world):
        import torch.distributed._symmetric_memory as symm
        self.nbytes, self.rank, self.world = nbytes, rank, world
        self.bytes_tensor = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.bytes_tensor.zero_()
        self._hdl = symm.rendezvous(self.bytes_tensor, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in self._hdl.buffer_ptrs]
        self.own = self.ptrs[rank]
        self.mc = int(getattr(self._hdl, "multicast_ptr", 0) or 0)
        assert self.own == self.bytes_tensor.data_ptr()
        if not self.mc:
            raise RuntimeError("the process group has no NVLink multicast mapping (NVLS) for this allocation")

    def view(self, dtype, numel=None):
        t = self.bytes_tensor.view(dtype)
        return t if numel is None else t[:numel]

    def close(self):
        self._hdl = None
        self.own = None


def _pad(n, m):
    return -(-n // m) * m


class BucketLayout:
    """Flat placement of parameters, bucket after bucket.  Every parameter starts on an
    ALIGN-element boundary; every bucket's length is a multiple of world * ALIGN so the
    `world` slices are equal and 16-byte aligned."""

    def __init__(self, buckets, world):
        self.world = world
        self.buckets = [unique_params(b) for b in buckets]
        seen = set()
        self.offsets, self.bucket_off, self.bucket_len = {}, [], []
        off = 0
        for b in self.buckets:
            start = off
            for p in b:
                assert id(p) not in seen, "a parameter may sit in one bucket only"
                seen.add(id(p))
                self.offsets[id(p)] = off
                off += _pad(p.numel(), ALIGN)
            off = start + _pad(off - start, world * ALIGN)
            self.bucket_off.append(start)
            self.bucket_len.append(off - start)
        self.numel = off
        self.params = [p for b in self.buckets for p in b]
        assert len(self.buckets) <= MAX_BUCKETS

    def view(self, flat, p):
        o = self.offsets[id(p)]
        return flat[o:o + p.numel()].view_as(p)

    def slice_of(self, b, rank):
        n = self.bucket_len[b] // self.world
        lo = self.bucket_off[b] + rank * n
        return lo, lo + n

    def moment_offsets(self):
        out, o = [], 0
        for b in range(len(self.buckets)):
            out.append(o)
            o += self.bucket_len[b] // self.world
        return out, o


def default_buckets(model):
    """Buckets in the order the reverse scan completes gradients: final norm first, then
    the layers from last to first, the (tied) embedding last."""
    emb_ids = {id(model.tok_emb.weight), id(model.lm_head.weight)}
    head = [model.norm_f.weight]
    layers = [[p for p in blk.parameters()] for blk in reversed(model.blocks)]
    tail = unique_params([model.lm_head.weight, model.tok_emb.weight])
    rest = [p for p in model.parameters()
            if id(p) not in emb_ids and id(p) != id(model.norm_f.weight)
            and not any(id(p) == id(q) for lay in layers for q in lay)]
    return [head + rest] + layers + [tail]


def decay_groups(model, weight_decay, decay_all=False):
    """Matrices decay; gains, biases and other 1-D parameters do not."""
    params = unique_params(model.parameters())
    if decay_all:
        return [{"params": params, "weight_decay": weight_decay}]
    return [{"params": [p for p in params if p.dim() >= 2], "weight_decay": weight_decay},
            {"params": [p for p in params if p.dim() < 2], "weight_decay": 0.0}]


class FusedDPAdamW:
    def __init__(self, param_groups, buckets, *, lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                 max_norm=1.0, skip_norm=0.0, grad_accum=1, process_group=None, device=None,
                 wait_seconds=5.0, use_kernel=None, nvls=None):
        self.group = process_group
        if dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(process_group), dist.get_rank(process_group)
        else:
            self.world, self.rank = 1, 0
        assert self.world <= MAX_WORLD
        self.lr, self.betas, self.eps = lr, betas, eps
        self.max_norm, self.skip_norm, self.grad_accum = max_norm, skip_norm, grad_accum
        self.param_groups = [dict(g) for g in param_groups]
        for g in self.param_groups:
            g.setdefault("weight_decay", 0.0)
            g.setdefault("lr_mult", 1.0)
            g["params"] = unique_params(g["params"])
        self.layout = BucketLayout(buckets, self.world)
        grouped = {id(p) for g in self.param_groups for p in g["params"]}
        assert grouped == {id(p) for p in self.layout.params}, "groups and buckets must cover the same parameters"
        self.device = torch.device(device) if device is not None else self.layout.params[0].device
        self.use_kernel = self.device.type == "cuda" if use_kernel is None else use_kernel
        # AdamW's t counts APPLIED updates only (a step voided by the skip predicate does not advance it,
        # as torch.optim.AdamW's `step` does not when step() is not called).  On the kernel path the
        # counter lives on the device (status[3]) because the skip decision is taken there; the host
        # attribute mirrors it for the host statement and is refreshed by `applied_steps()`.
        self.step_count = 0
        self.epoch = 0
        # set for one step by a caller that excluded ranks from the average (their gradients zeroed):
        # 1 / (ranks kept * micro-batches); None = 1 / (world * micro-batches)
        self.grad_scale_override = None
        self.wait_seconds = wait_seconds
        self.nvls = False
        n = self.layout.numel
        nslots = SLOT_BUCKET0 + len(self.layout.buckets)
        if self.use_kernel:
            from ..ops.cuda_ops import load_library
            self.lib = load_library()
            self._bind()
            mk = lambda nbytes: PeerBuffer(self.lib, nbytes, self.device, self.group, self.rank, self.world)
            # NVLS variant (opt-in: `nvls=True` or DMB_NVLS=1): gradient and parameter buffers bound to an NVLink
            # multicast object, reduce-scatter by multimem.ld_reduce and all-gather by multimem.st.  Not for runs in
            # which a rank may leave while the others still hold the mapping.
            self.nvls = bool(int(os.environ.get("DMB_NVLS", "0")) if nvls is None else nvls) and self.world > 1
            if self.nvls:
                mc = lambda nbytes: MulticastBuffer(nbytes, self.device, self.group, self.rank, self.world)
                self._pb_grads, self._pb_params = mc(4 * n), mc(4 * n)
            else:
                self._pb_grads, self._pb_params = mk(4 * n), mk(4 * n)
            self._pb_flags, self._pb_norms = mk(4 * nslots * MAX_WORLD), mk(4 * 2 * MAX_WORLD)
            self.flat_grads = self._pb_grads.view(torch.float32, n)
            self.flat_params = self._pb_params.view(torch.float32, n)
        else:
            self.flat_grads = torch.zeros(n, dtype=torch.float32, device=self.device)
            self.flat_params = torch.zeros(n, dtype=torch.float32, device=self.device)
        # adopt the parameters: copy into the flat buffer, then alias
        with torch.no_grad():
            for p in self.layout.params:
                v = self.layout.view(self.flat_params, p)
                v.copy_(p.detach())
                p.data = v
        self._sync_initial_params()
        self.moment_off, n_own = self.layout.moment_offsets()
        self.m = torch.zeros(n_own, dtype=torch.float32, device=self.device)
        self.v = torch.zeros(n_own, dtype=torch.float32, device=self.device)
        self._build_segments()
        # ctrl: [grad norm, clip coefficient, skipped, spare, t, 1 - beta1^t, 1 - beta2^t, wait error code]
        self.ctrl = torch.zeros(8, dtype=torch.float32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._reduced = [0] * len(self.layout.buckets)
        self._early_partials = 0
        if self.use_kernel:
            blocks = ctypes.c_int()
            with torch.cuda.device(self.device):
                _ck(self.lib.dmb_opt_max_blocks(ctypes.byref(blocks)), "occupancy query")
            self.blocks = blocks.value
            self.bucket_blocks = 64
            self.partial = torch.zeros(self.blocks + self.bucket_blocks * len(self.layout.buckets),
                                       dtype=torch.float32, device=self.device)
            self._comm = _Comm()
            self._comm.world, self._comm.rank = self.world, self.rank
            for r in range(self.world):
                self._comm.grads[r], self._comm.params[r] = self._pb_grads.ptrs[r], self._pb_params.ptrs[r]
                self._comm.flags[r], self._comm.norms[r] = self._pb_flags.ptrs[r], self._pb_norms.ptrs[r]
            self._comm.mc_grads = self._pb_grads.mc if self.nvls else None
            self._comm.mc_params = self._pb_params.mc if self.nvls else None
            sm_hz = 1.9e9
            self._wait_cycles = int(wait_seconds * sm_hz)
        if self.world > 1:
            dist.barrier(group=self.group)

    # ---- construction helpers ---------------------------------------------------------------------
    def _bind(self):
        L, p, i, ll, f, u = self.lib, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_uint
        L.dmb_ipc_alloc.argtypes, L.dmb_ipc_alloc.restype = [ctypes.c_size_t, ctypes.POINTER(p)], i
        L.dmb_ipc_free.argtypes = [p]
        L.dmb_ipc_get_handle.argtypes = [p, p]
        L.dmb_ipc_open.argtypes = [p, ctypes.POINTER(p)]
        L.dmb_ipc_close.argtypes = [p]
        L.dmb_ipc_handle_size.restype = i
        L.dmb_opt_max_blocks.argtypes = [ctypes.POINTER(i)]
        L.dmb_opt_signal.argtypes = [ctypes.POINTER(_Comm), i, u, p]
        L.dmb_opt_reduce_bucket.argtypes = [ctypes.POINTER(_Comm), ll, ll, f, p, i, u, i, ll, p, p]
        L.dmb_opt_fused_step.argtypes = [ctypes.POINTER(_Comm), ctypes.POINTER(_Plan), ctypes.POINTER(_Hyper),
                                         p, p, p, p, p, p, i, p, p, i, p]
        sizes = [ctypes.c_int() for _ in range(3)]
        L.dmb_opt_struct_sizes(*[ctypes.byref(s) for s in sizes])
        assert [s.value for s in sizes] == [ctypes.sizeof(_Comm), ctypes.sizeof(_Plan), ctypes.sizeof(_Hyper)], \
            "host/device struct layout mismatch"

    def _sync_initial_params(self):
        if self.world > 1:
            dist.broadcast(self.flat_params, src=dist.get_global_rank(self.group, 0) if self.group else 0,
                           group=self.group)

    def _build_segments(self):
        """Per-parameter (start, weight decay, lr multiplier), sorted by start."""
        hyp = {}
        for g in self.param_groups:
            for p in g["params"]:
                hyp[id(p)] = (g["weight_decay"], g["lr_mult"])
        segs = sorted((self.layout.offsets[id(p)],) + hyp[id(p)] for p in self.layout.params)
        self.seg_start = torch.tensor([s[0] for s in segs], dtype=torch.int64, device=self.device)
        self.seg_wd = torch.tensor([s[1] for s in segs], dtype=torch.float32, device=self.device)
        self.seg_lr = torch.tensor([s[2] for s in segs], dtype=torch.float32, device=self.device)

    def grad_buffers(self) -> GradBuffers:
        """A `GradBuffers` whose views alias this optimizer's flat gradient array."""
        return GradBuffers.from_flat(self.layout.params, self.layout, self.flat_grads)

    def zero_grad(self):
        self.flat_grads.zero_()
        self._reduced = [0] * len(self.layout.buckets)
        self._early_partials = 0

    # ---- the step ------------------------------------------------------------------------------------
    def _grad_scale(self):
        return self.grad_scale_override or 1.0 / (self.world * self.grad_accum)

    def _hyper(self, lr):
        self.epoch += 1
        b1, b2 = self.betas
        return dict(lr=lr, beta1=b1, beta2=b2, eps=self.eps, grad_scale=self._grad_scale(),
                    max_norm=self.max_norm or 0.0, skip_norm=self.skip_norm or 0.0)

    def applied_steps(self):
        """Number of updates applied so far (AdamW's t).  Kernel path: a host read of the device counter."""
        if self.use_kernel:
            self.step_count = int(self.status[3].item())
        return self.step_count

    def bucket_ready(self, b, stream=None):
        """Announce that this rank's gradients of bucket b are final and start its
        reduce-scatter (on `stream`, default current)."""
        if not self.use_kernel:
            return
        epoch = self.epoch + 1
        st = ctypes.c_void_p((stream or torch.cuda.current_stream(self.device)).cuda_stream)
        _ck(self.lib.dmb_opt_signal(ctypes.byref(self._comm), SLOT_BUCKET0 + b, epoch, st), "signal")
        off, ln = self.layout.bucket_off[b], self.layout.bucket_len[b]
        part = self.partial[self._early_partials:]
        _ck(self.lib.dmb_opt_reduce_bucket(ctypes.byref(self._comm), off, ln,
                                           self._grad_scale(), part.data_ptr(),
                                           self.bucket_blocks, epoch, SLOT_BUCKET0 + b, self._wait_cycles,
                                           self.status.data_ptr(), st), "reduce_bucket")
        self._early_partials += self.bucket_blocks
        self._reduced[b] = 1

    def step(self, lr=None):
        """One optimizer step on the accumulated gradients.  Returns the device tensor
        `ctrl` = [global grad norm, clip coefficient, skipped (0/1), 0]; nothing here
        synchronises with the host."""
        h = self._hyper(self.lr if lr is None else lr)
        if not self.use_kernel:
            self._step_host(h)
            return self.ctrl
        plan = _Plan()
        plan.n_buckets, plan.n_segs = len(self.layout.buckets), self.seg_start.numel()
        for b in range(plan.n_buckets):
            plan.bucket_off[b], plan.bucket_len[b] = self.layout.bucket_off[b], self.layout.bucket_len[b]
            plan.moment_off[b], plan.reduced[b] = self.moment_off[b], self._reduced[b]
        hp = _Hyper(epoch=self.epoch, wait_cycles=self._wait_cycles, **h)
        # early partials sit first; the cooperative kernel appends one partial per block
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            _ck(self.lib.dmb_opt_fused_step(
                ctypes.byref(self._comm), ctypes.byref(plan), ctypes.byref(hp), self.seg_start.data_ptr(),
                self.seg_wd.data_ptr(), self.seg_lr.data_ptr(), self.m.data_ptr(), self.v.data_ptr(),
                self.partial.data_ptr(), self._early_partials, self.ctrl.data_ptr(), self.status.data_ptr(),
                self.blocks, st), "fused step")
        self._reduced = [0] * len(self.layout.buckets)
        self._early_partials = 0
        return self.ctrl

    def check_status(self, code=None):
        """Raises `PeerWaitExpired` if a cross-GPU wait of the kernels ran out.  `code`: the error code already
        on the host (ctrl[7] of the last step, read together with the step's verdict); None reads the status
        word from the device.  The word is sticky: once a wait has run out every later step is voided, so
        the caller should checkpoint from host state and stop."""
        if code is None:
            code = self.status[0].item()
        if code:
            peer = self.status[1].item()
            where = {1: "opening barrier", 2: "norm exchange", 3: "closing barrier"}.get(int(code), "?")
            raise PeerWaitExpired(f"fused optimizer: rank {self.rank} gave up waiting for rank {peer} at the {where}")

    @torch.no_grad()
    def _step_host(self, h):
        """Torch statement of the kernel (CPU / gloo ranks, and the kernel's test oracle)."""
        W, r = self.world, self.rank
        g = self.flat_grads
        if W > 1:
            dist.all_reduce(g, group=self.group)            # fixed-order sum on every rank
        g.mul_(h["grad_scale"])
        ss = torch.zeros((), dtype=torch.float32, device=self.device)
        for b in range(len(self.layout.buckets)):
            lo, hi = self.layout.slice_of(b, r)
            ss += g[lo:hi].square().sum()
        if W > 1:
            parts = [torch.zeros_like(ss) for _ in range(W)]
            dist.all_gather(parts, ss, group=self.group)
            tot = sum(parts)
        else:
            tot = ss
        gn = tot.sqrt()
        coef = torch.clamp(h["max_norm"] / (gn + 1e-6), max=1.0) if h["max_norm"] > 0 else torch.ones_like(gn)
        skip = (~torch.isfinite(gn)) | ((gn > h["skip_norm"]) if h["skip_norm"] > 0 else torch.zeros_like(gn, dtype=torch.bool))
        skip = skip | bool(self.status[0] != 0)
        self.ctrl[0], self.ctrl[1], self.ctrl[2] = gn, coef, skip.float()
        self.ctrl[7] = self.status[0].float()
        if bool(skip):
            return
        self.step_count += 1
        self.status[3] = self.step_count
        h = dict(h, bias1=1 - h["beta1"] ** self.step_count, bias2=1 - h["beta2"] ** self.step_count)
        self.ctrl[4], self.ctrl[5], self.ctrl[6] = float(self.step_count), h["bias1"], h["bias2"]
        wd_full, lr_full = self._expand_segments()
        for b in range(len(self.layout.buckets)):
            lo, hi = self.layout.slice_of(b, r)
            mo = self.moment_off[b]
            ge = g[lo:hi] * coef
            m, v = self.m[mo:mo + hi - lo], self.v[mo:mo + hi - lo]
            m.mul_(h["beta1"]).add_(ge, alpha=1 - h["beta1"])
            v.mul_(h["beta2"]).addcmul_(ge, ge, value=1 - h["beta2"])
            denom = v.sqrt() / math.sqrt(h["bias2"]) + h["eps"]
            p = self.flat_params[lo:hi]
            p.mul_(1 - h["lr"] * lr_full[lo:hi] * wd_full[lo:hi])
            p.sub_(h["lr"] / h["bias1"] * lr_full[lo:hi] * m / denom)
        if W > 1:                                            # all-gather of the updated slices
            for b in range(len(self.layout.buckets)):
                n = self.layout.bucket_len[b] // W
                whole = self.flat_params[self.layout.bucket_off[b]:self.layout.bucket_off[b] + n * W]
                dist.all_gather_into_tensor(whole, whole[r * n:(r + 1) * n].clone(), group=self.group)

    def _expand_segments(self):
        n = self.layout.numel
        idx = torch.searchsorted(self.seg_start, torch.arange(n, device=self.device), right=True) - 1
        return self.seg_wd[idx], self.seg_lr[idx]

    # ---- checkpoint interchange -------------------------------------------------------------------------
    def _gather_moments(self, local):
        """Full flat moment array from the per-rank slices."""
        W = self.world
        full = torch.zeros(self.layout.numel, dtype=torch.float32, device=self.device)
        for b in range(len(self.layout.buckets)):
            n, mo, off = self.layout.bucket_len[b] // W, self.moment_off[b], self.layout.bucket_off[b]
            if W > 1:
                dist.all_gather_into_tensor(full[off:off + n * W], local[mo:mo + n].contiguous(), group=self.group)
            else:
                full[off:off + n] = local[mo:mo + n]
        return full

    def state_dict(self):
        """Unsharded state in the layout of `torch.optim.AdamW.state_dict()`; parameter
        indices follow the order of `param_groups`."""
        m_full, v_full = self._gather_moments(self.m), self._gather_moments(self.v)
        self.applied_steps()
        state, groups, idx = {}, [], 0
        for g in self.param_groups:
            ids = []
            for p in g["params"]:
                state[idx] = {"step": torch.tensor(float(self.step_count)),
                              "exp_avg": self.layout.view(m_full, p).clone().cpu(),
                              "exp_avg_sq": self.layout.view(v_full, p).clone().cpu()}
                ids.append(idx)
                idx += 1
            groups.append({"lr": self.lr * g["lr_mult"], "betas": self.betas, "eps": self.eps,
                           "weight_decay": g["weight_decay"], "amsgrad": False, "params": ids})
        return {"state": state, "param_groups": groups}

    def load_state_dict(self, sd):
        m_full = torch.zeros(self.layout.numel, dtype=torch.float32, device=self.device)
        v_full = torch.zeros_like(m_full)
        idx = 0
        for g in self.param_groups:
            for p in g["params"]:
                st = sd["state"].get(idx)
                if st is not None:
                    self.layout.view(m_full, p).copy_(st["exp_avg"])
                    self.layout.view(v_full, p).copy_(st["exp_avg_sq"])
                    self.step_count = int(float(st["step"]))
                idx += 1
        self.status[3] = self.step_count
        for b in range(len(self.layout.buckets)):
            lo, hi = self.layout.slice_of(b, self.rank)
            mo = self.moment_off[b]
            self.m[mo:mo + hi - lo] = m_full[lo:hi]
            self.v[mo:mo + hi - lo] = v_full[lo:hi]

    def close(self):
        if self.use_kernel:
            torch.cuda.synchronize(self.device)
            if self.nvls:
                dist.barrier(group=self.group)       # nobody unmaps while a peer may still store through the multicast address
            for pb in (self._pb_grads, self._pb_params, self._pb_flags, self._pb_norms):
                pb.close()


class NcclAdamW:
    """The baseline chain behind the same interface: library all-reduce of the flat
    gradient buffer, global-norm clip, skip decision, `torch.optim.AdamW`."""

    def __init__(self, param_groups, *, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, max_norm=1.0,
                 skip_norm=0.0, grad_accum=1, process_group=None, bitwise_sync=False):
        self.group = process_group
        self.world = dist.get_world_size(process_group) if dist.is_available() and dist.is_initialized() else 1
        groups = [{"params": unique_params(g["params"]), "weight_decay": g.get("weight_decay", 0.0),
                   "lr": lr * g.get("lr_mult", 1.0)} for g in param_groups]
        self.params = [p for g in groups for p in g["params"]]
        dev = self.params[0].device
        self.opt = torch.optim.AdamW(groups, lr=lr, betas=betas, eps=eps, fused=dev.type == "cuda")
        self.base_lrs = [g["lr"] / lr for g in groups]
        self.lr, self.max_norm, self.skip_norm, self.grad_accum = lr, max_norm, skip_norm, grad_accum
        self.grad_scale_override = None
        self.bitwise_sync = bitwise_sync
        self.grads = GradBuffers(self.params)
        self.ctrl = torch.zeros(4, dtype=torch.float32, device=dev)

    def grad_buffers(self):
        return self.grads

    def zero_grad(self):
        self.grads.zero_()

    def step(self, lr=None):
        flat = self.grads.flat
        if self.world > 1:
            if self.bitwise_sync:
                dist.reduce(flat, dst=0, group=self.group)
                dist.broadcast(flat, src=0, group=self.group)
            else:
                dist.all_reduce(flat, group=self.group)
        flat.mul_(self.grad_scale_override or 1.0 / (self.world * self.grad_accum))
        self.grads.to_param_grads()
        gn = flat.norm()
        if self.max_norm and self.max_norm > 0:
            flat.mul_(torch.clamp(self.max_norm / (gn + 1e-6), max=1.0))
        skip = (~torch.isfinite(gn)) | ((gn > self.skip_norm) if self.skip_norm > 0 else False)
        self.ctrl[0], self.ctrl[2] = gn, float(skip)
        if bool(skip):
            return self.ctrl
        for g, mult in zip(self.opt.param_groups, self.base_lrs):
            g["lr"] = (self.lr if lr is None else lr) * mult
        self.opt.step()
        return self.ctrl

    def state_dict(self):
        return self.opt.state_dict()

    def load_state_dict(self, sd):
        self.opt.load_state_dict(sd)
