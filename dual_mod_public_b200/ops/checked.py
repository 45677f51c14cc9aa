"""Launch-argument checker: a wrapper around an op table that validates every call on the host.

    ops = CheckedOps(CudaOps(device))        # or: DMB_CHECK_ARGS=1 (the engines wrap their table themselves)

No memory-checking tool runs on the kernels' target machines, so the errors such a tool would catch are
caught one level up, from the arguments of each launch, before it happens:

  layout      no negative strides; with `strict_layout=True` (DMB_CHECK_LAYOUT=1) also: every tensor argument
              has a dense last dimension, rows that start on 16-byte boundaries (the kernels use 16-byte
              vector accesses) and a base address aligned likewise.  The kernel table itself falls back to the
              torch statement for layouts a kernel cannot take, so the strict form asks "would every launch of
              this run have been a kernel launch?"
  aliasing    tensors a call writes (`out=`, `*_acc`, `*_out`, `dW`, the per-layer arrays of `cell_finish`
              and `split_partials`) do not overlap any tensor the same call reads
  ranges      positions and extents agree with the tape: 0 <= pos0 <= T, pos0 + rows <= T where rows are
              written at pos0, window and offsets non-negative, chunk lengths divide window lengths,
              q_start <= q_end <= T
  shapes      rows of queries / partials / gradients agree; head count and head size agree across arguments
  finite      with `check_finite=True` (DMB_CHECK_FINITE=1) every floating tensor written by the call is
              scanned for NaN / Inf afterwards (one host sync per call: a debugging aid, not for timing)

A violation raises `OpArgumentError` naming the op, the argument and the rule.  The wrapper forwards
everything else (`launches`, `name`, `gemm`, ...) to the inner table.
"""

from __future__ import annotations

import inspect
import os

import torch


class OpArgumentError(ValueError):
    pass


WRITTEN = {"out", "dq_acc", "dks_acc", "dv_acc", "doc_acc", "dlsec_acc", "dk_acc", "dglx_acc", "dvgx_acc", "dcg_out",
           "uhat_out", "dW", "dw_acc", "gw", "doc", "corr", "lsec", "dks", "dv", "DOf", "DLf", "docn", "corrn", "lsen",
           "dvc_out", "dkg_out", "dcg"}
# ops whose named argument is an accumulator that may legitimately alias nothing else; (op, arg) pairs that are
# read-write on purpose and must not be reported as "written tensor overlaps a read tensor" against themselves
READ_ONLY_DCG = {"mrk_vin_bwd"}                       # there `dcg` is read-modify-write by design (adds into it)


def _extent(t):
    """[first byte, last byte + 1) of the memory a view can touch."""
    if t.numel() == 0:
        return t.data_ptr(), t.data_ptr()
    span = sum((s - 1) * st for s, st in zip(t.shape, t.stride())) + 1
    return t.data_ptr(), t.data_ptr() + span * t.element_size()


def _overlap(a, b):
    if a.device != b.device or a.numel() == 0 or b.numel() == 0:
        return False
    a0, a1 = _extent(a)
    b0, b1 = _extent(b)
    if not (a0 < b1 and b0 < a1):
        return False
    # two row slices [B, R, ...] of the same [B, T, ...] buffer interleave in memory without sharing a byte:
    # same batch stride and dense rows -> compare the per-batch runs
    if (a.dim() >= 2 and a.dim() == b.dim() and a.dtype == b.dtype and a.stride() == b.stride()
            and a.shape[0] == b.shape[0] and a.shape[2:] == b.shape[2:] and a.shape[0] > 1):
        run_a, run_b = a.shape[1] * a.stride(1), b.shape[1] * b.stride(1)
        bs = a.stride(0)
        if max(run_a, run_b) <= bs:
            off = (b0 - a0) // a.element_size()              # elements from a's first row to b's first row
            off %= bs
            return off < run_a or off + run_b > bs
    return True


class CheckedOps:
    def __init__(self, inner, check_finite=None, strict_layout=None, align=16):
        self._inner = inner
        self._finite = (os.environ.get("DMB_CHECK_FINITE", "0") == "1") if check_finite is None else check_finite
        self._strict = (os.environ.get("DMB_CHECK_LAYOUT", "0") == "1") if strict_layout is None else strict_layout
        self._align = align
        self.calls_checked = 0
        self._sigs = {}

    # ---- forwarding ---------------------------------------------------------------------------------
    def __getattr__(self, name):
        target = getattr(self._inner, name)
        if name.startswith("_") or not callable(target) or inspect.isclass(target):
            return target
        sig = self._sigs.get(name)
        if sig is None:
            try:
                sig = self._sigs[name] = inspect.signature(target)
            except (TypeError, ValueError):
                return target

        def call(*args, **kwargs):
            bound = sig.bind(*args, **kwargs)
            bound.apply_defaults()
            self._check(name, bound.arguments)
            result = target(*args, **kwargs)
            if self._finite:
                self._check_finite(name, bound.arguments, result)
            return result

        return call

    def __setattr__(self, name, value):
        if name.startswith("_") or name == "calls_checked":
            object.__setattr__(self, name, value)
        else:
            setattr(self._inner, name, value)

    # ---- rules ----------------------------------------------------------------------------------------
    def _fail(self, op, arg, rule):
        raise OpArgumentError(f"{op}({arg}): {rule}")

    def _tensors(self, arguments):
        for k, v in arguments.items():
            if torch.is_tensor(v):
                yield k, v
            elif isinstance(v, (tuple, list)) and v and all(torch.is_tensor(x) for x in v):
                for i, x in enumerate(v):
                    yield f"{k}[{i}]", x

    def _check(self, op, arguments):
        self.calls_checked += 1
        named = list(self._tensors(arguments))
        for k, t in named:
            if t.dim() == 0 or t.numel() == 0:
                continue
            if any(st < 0 for st in t.stride()):
                self._fail(op, k, f"negative stride {tuple(t.stride())}")
            if not self._strict:
                continue
            if t.shape[-1] > 1 and t.stride(-1) != 1:
                self._fail(op, k, f"last dimension is not dense (strides {tuple(t.stride())})")
            if t.is_floating_point() and t.dim() >= 2 and t.shape[-1] * t.element_size() >= self._align:
                if t.data_ptr() % self._align:
                    self._fail(op, k, f"base address is not {self._align}-byte aligned")
                for size, st in zip(t.shape[:-1], t.stride()[:-1]):
                    if size > 1 and (st * t.element_size()) % self._align:
                        self._fail(op, k, f"a stride of {st} elements leaves rows off a {self._align}-byte boundary")
        written = [(k, t) for k, t in named if k.split("[")[0] in WRITTEN and not (op in READ_ONLY_DCG and k == "dcg")]
        for kw, tw in written:
            for kr, tr in named:
                if kr == kw or kr.split("[")[0] in WRITTEN:
                    continue
                if _overlap(tw, tr):
                    self._fail(op, kw, f"written tensor overlaps the read tensor `{kr}`")
        for i, (k1, t1) in enumerate(written):
            for k2, t2 in written[i + 1:]:
                if _overlap(t1, t2):
                    self._fail(op, k1, f"written tensor overlaps the written tensor `{k2}`")
        rule = getattr(self, "_rule_" + op, None)
        if rule is not None:
            rule(op, arguments)

    def _check_finite(self, op, arguments, result):
        outs = [(k, t) for k, t in self._tensors(arguments) if k.split("[")[0] in WRITTEN]
        if torch.is_tensor(result):
            outs.append(("result", result))
        elif isinstance(result, (tuple, list)):
            outs += [(f"result[{i}]", r) for i, r in enumerate(result) if torch.is_tensor(r)]
        for k, t in outs:
            if t.is_floating_point() and t.numel() and not bool(torch.isfinite(t).all()):
                self._fail(op, k, "non-finite values after the call")

    # ---- per-op range and shape rules -----------------------------------------------------------------------
    def _need(self, op, cond, arg, rule):
        if not cond:
            self._fail(op, arg, rule)

    def _tape(self, op, a, rows_key="q_r"):
        Kc, Vc = a["Kc"], a["Vc"]
        self._need(op, Kc.shape == Vc.shape, "Vc", f"shape {tuple(Vc.shape)} differs from Kc {tuple(Kc.shape)}")
        q = a[rows_key]
        self._need(op, q.shape[0] == Kc.shape[0] and q.shape[2:] == Kc.shape[2:], rows_key,
                   f"batch / heads / head size {tuple(q.shape)} do not match the tape {tuple(Kc.shape)}")
        self._need(op, a.get("window", 0) >= 0, "window", "negative")
        return Kc.shape[1]

    def _rule_prefix_fwd(self, op, a):
        T = self._tape(op, a)
        self._need(op, 0 <= a["pos0"] <= T, "pos0", f"{a['pos0']} outside the tape of {T} rows")
        self._need(op, a["qoff"] >= 0, "qoff", "negative")

    def _rule_prefix_dq(self, op, a):
        self._rule_prefix_fwd(op, a)
        q = a["q_r"]
        self._need(op, a["dq_acc"].shape == q.shape, "dq_acc", f"shape {tuple(a['dq_acc'].shape)} != queries {tuple(q.shape)}")
        self._need(op, a["lse_c"].shape == q.shape[:3] and a["corr"].shape == q.shape[:3], "lse_c / corr",
                   "one value per (batch, row, head) expected")

    def _rule_prefix_dkv(self, op, a):
        T = self._tape(op, a, "q_all")
        q_end = T if a["q_end"] is None else a["q_end"]
        self._need(op, a["c"] > 0 and 0 <= a["pos0"] and a["pos0"] + a["c"] <= T, "pos0",
                   f"key rows [{a['pos0']}, {a['pos0'] + a['c']}) outside the tape of {T} rows")
        self._need(op, 0 <= a["q_start"] <= q_end <= a["q_all"].shape[1], "q_start",
                   f"query rows [{a['q_start']}, {q_end}) outside {a['q_all'].shape[1]} rows")

    def _rule_tail_fwd(self, op, a):
        q = a["q_r"]
        for k in ("kself_r", "v_raw", "K_in", "V_in", "o_c"):
            self._need(op, a[k].shape == q.shape, k, f"shape {tuple(a[k].shape)} != queries {tuple(q.shape)}")
        self._need(op, a["lse_c"].shape == q.shape[:3], "lse_c", "one value per (batch, row, head) expected")
        self._need(op, a.get("window", 0) >= 0, "window", "negative")

    def _rule_tail_bwd(self, op, a):
        self._rule_tail_fwd(op, a)
        q = a["q_r"]
        for k in ("dO", "o", "dq_acc", "dks_acc", "dv_acc", "doc_acc"):
            self._need(op, a[k].shape == q.shape, k, f"shape {tuple(a[k].shape)} != queries {tuple(q.shape)}")

    def _window(self, op, a, key="q_win"):
        rows, C = a[key].shape[1], a["C"]
        self._need(op, C > 0 and rows % C == 0, key, f"{rows} window rows are not a whole number of chunks of {C}")

    def _rule_win_near_fwd(self, op, a):
        T = self._tape(op, a, "q_win")
        self._window(op, a)
        G = a["q_win"].shape[1] // a["C"]
        self._need(op, 0 <= a["pos0"] and a["pos0"] + (G - 1) * a["C"] <= T, "pos0",
                   f"the last group's keys end at {a['pos0'] + (G - 1) * a['C']}, past the tape of {T} rows")
        self._need(op, a["lo"] <= a["pos0"], "lo", "the key range starts after it ends")

    _rule_win_near_dq = _rule_win_near_fwd

    def _rule_win_tail_fwd(self, op, a):
        self._window(op, a)

    def _rule_win_tail_bwd(self, op, a):
        self._window(op, a)

    def _rule_refine_fwd(self, op, a):
        k = a["k"]
        self._need(op, k.shape[-1] % a["h"] == 0, "h", f"{a['h']} heads do not divide the width {k.shape[-1]}")
        self._need(op, a["raw"].shape[:2] == k.shape[:2] and a["raw"].shape[-1] == 4 * k.shape[-1], "raw",
                   f"shape {tuple(a['raw'].shape)} is not [B, c, 4d] for rows {tuple(k.shape)}")
        self._need(op, a["cos"].shape[0] == k.shape[1], "cos", f"{a['cos'].shape[0]} positions for {k.shape[1]} rows")
        self._need(op, 0 <= a["pin_cols"] <= k.shape[-1], "pin_cols", "outside [0, d]")

    def _rule_embed_bwd(self, op, a):
        self._need(op, a["idx"].numel() == a["dx"].numel() // a["dx"].shape[-1], "idx", "one id per gradient row expected")
        self._need(op, a["gw"].shape[-1] == a["dx"].shape[-1], "gw", "row width differs from the gradient rows")
        if a["idx"].numel():
            lo, hi = int(a["idx"].min()), int(a["idx"].max())
            self._need(op, 0 <= lo and hi < a["gw"].shape[0], "idx", f"ids in [{lo}, {hi}] outside the table of {a['gw'].shape[0]} rows")

    def _rule_linear(self, op, a):
        x, w, out = a["x"], a["w"], a["out"]
        self._need(op, x.shape[-1] == w.shape[1], "w", f"inner sizes {x.shape[-1]} and {w.shape[1]} differ")
        if out is not None:
            self._need(op, out.shape[-1] == w.shape[0] and out.numel() // out.shape[-1] == x.numel() // x.shape[-1], "out",
                       f"shape {tuple(out.shape)} is not [rows, {w.shape[0]}]")

    def _rule_linear_dx(self, op, a):
        dy, w, out = a["dy"], a["w"], a["out"]
        self._need(op, dy.shape[-1] == w.shape[0], "w", f"inner sizes {dy.shape[-1]} and {w.shape[0]} differ")
        if out is not None:
            self._need(op, out.shape[-1] == w.shape[1], "out", f"width {out.shape[-1]} != {w.shape[1]}")

    def _rule_linear_dw_acc(self, op, a):
        dW, dy, x = a["dW"], a["dy"], a["x"]
        self._need(op, dW.shape == (dy.shape[-1], x.shape[-1]), "dW", f"shape {tuple(dW.shape)} != [{dy.shape[-1]}, {x.shape[-1]}]")
        self._need(op, dy.numel() // dy.shape[-1] == x.numel() // x.shape[-1], "x", "row counts of dy and x differ")
        self._need(op, dW.dtype == torch.float32, "dW", "the accumulator must be fp32")


def maybe_checked(ops):
    """`ops` wrapped in `CheckedOps` when DMB_CHECK_ARGS=1, else `ops` itself."""
    return CheckedOps(ops) if os.environ.get("DMB_CHECK_ARGS", "0") == "1" and not isinstance(ops, CheckedOps) else ops
