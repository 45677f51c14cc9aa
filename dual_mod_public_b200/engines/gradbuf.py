"""Flat gradient storage.

Every parameter's gradient is a view into one contiguous buffer (per dtype), so
data-parallel reduction is a few large transfers and the fused
reduce-scatter + AdamW kernels can treat the model as a 1-D array.  Tied
parameters share one view.  Reference parity: `GradBuffers`
(engines/wavescan/engine/backward.py:27-84).  Differences: views are padded to
`align` elements so every parameter starts on a 16-byte boundary, and the buffer
may be allocated by a caller-supplied function (peer-mapped symmetric memory).
"""

from __future__ import annotations

from typing import Callable, Iterable

import torch


def unique_params(params: Iterable[torch.nn.Parameter]) -> list:
    seen, out = set(), []
    for p in params:
        if id(p) not in seen:
            seen.add(id(p))
            out.append(p)
    return out


class FlatLayout:
    """Offsets of a parameter list inside a flat array."""

    def __init__(self, params, align: int = 64, pad_total_to: int = 1):
        self.params = unique_params(params)
        self.offsets, off = {}, 0
        for p in self.params:
            self.offsets[id(p)] = off
            off += -(-p.numel() // align) * align
        self.numel = -(-off // pad_total_to) * pad_total_to

    def view(self, flat: torch.Tensor, p) -> torch.Tensor:
        o = self.offsets[id(p)]
        return flat[o:o + p.numel()].view_as(p)

    def segments(self):
        """[(param, offset, numel)] in layout order."""
        return [(p, self.offsets[id(p)], p.numel()) for p in self.params]


class GradBuffers:
    def __init__(self, params, bf16_ids=None, align: int = 64, pad_total_to: int = 1,
                 alloc: Callable[[int, torch.dtype, torch.device], torch.Tensor] | None = None):
        """bf16_ids: ids of parameters whose gradient accumulates in bf16 (a second
        flat bucket); all others accumulate in fp32."""
        uniq = unique_params(params)
        bf16_ids = bf16_ids or set()
        dev = uniq[0].device
        alloc = alloc or (lambda n, dt, dv: torch.zeros(n, dtype=dt, device=dv))
        self.order = uniq
        self.buf, self.flats, self.layouts = {}, [], []
        groups = [(torch.float32, [p for p in uniq if id(p) not in bf16_ids])]
        if bf16_ids:
            groups.append((torch.bfloat16, [p for p in uniq if id(p) in bf16_ids]))
        for dt, plist in groups:
            if not plist:
                continue
            lay = FlatLayout(plist, align=align, pad_total_to=pad_total_to)
            flat = alloc(lay.numel, dt, dev)
            flat.zero_()
            self.flats.append(flat)
            self.layouts.append(lay)
            for p in plist:
                self.buf[id(p)] = lay.view(flat, p)
        self.flat = self.flats[0]

    @classmethod
    def from_flat(cls, params, layout, flat):
        """Views into an existing flat array placed by `layout` (anything with
        `.view(flat, p)`), e.g. the fused optimizer's peer-mapped gradient buffer."""
        self = cls.__new__(cls)
        self.order = unique_params(params)
        self.flats, self.layouts = [flat], [layout]
        self.buf = {id(p): layout.view(flat, p) for p in self.order}
        self.flat = flat
        return self

    def zero_(self):
        for f in self.flats:
            f.zero_()

    def add(self, param, g):
        if g is not None:
            self.buf[id(param)].add_(g.to(self.buf[id(param)].dtype))

    def get(self, param) -> torch.Tensor:
        return self.buf[id(param)]

    def to_param_grads(self):
        """Expose the buffers as `p.grad` (aliasing the view when dtypes agree)."""
        for p in self.order:
            b = self.buf[id(p)]
            if b.dtype == p.dtype:
                p.grad = b
            elif p.grad is None:
                p.grad = b.to(p.dtype)
            else:
                p.grad.copy_(b)

    def global_norm(self) -> torch.Tensor:
        return torch.sqrt(sum(f.float().square().sum() for f in self.flats))
