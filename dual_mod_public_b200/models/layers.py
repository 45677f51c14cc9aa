"""Small building blocks shared by every model in the package.

Reference parity: `RMSNorm` (models/dualmod/attention.py:74-83), the factored
projections `LoRAGate` / `LoRALinear` (attention.py:24-71) and `SwiGLU`
(models/dualmod/model.py:103-112).  State-dict keys are the same as the
reference's (`a.weight`, `b.weight`, `b.bias`; `down.weight`, `up.weight`,
`up.bias`; `w1/w2/w3.weight`).
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


def rms_normalize(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / rms(x) over the last dim, computed and returned in fp32."""
    xf = x.float()
    return xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)


class RMSNorm(nn.Module):
    """Root-mean-square norm with a learned gain; math in fp32, output in x.dtype."""

    def __init__(self, d: int, eps: float = 1e-5):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.eps = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return (rms_normalize(x, self.eps) * self.weight.float()).to(x.dtype)


def head_rms(x: torch.Tensor, n_heads: int, gain: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Per-head RMS norm of a flat [..., h*dh] tensor with one gain per head."""
    lead = x.shape[:-1]
    xh = x.reshape(*lead, n_heads, -1)
    out = rms_normalize(xh, eps) * gain.float().unsqueeze(-1)
    return out.to(x.dtype).reshape(*lead, -1)


class LoRAGate(nn.Module):
    """Gate projection factored as in -> r (no bias) -> out (bias).

    `.weight` / `.bias` expose the second factor so init and telemetry code that
    addresses a dense gate keeps working.
    """

    def __init__(self, d_in: int, rank: int, d_out: int):
        super().__init__()
        self.a = nn.Linear(d_in, rank, bias=False)
        self.b = nn.Linear(rank, d_out, bias=True)

    def forward(self, x):
        return self.b(self.a(x))

    @property
    def weight(self):
        return self.b.weight

    @property
    def bias(self):
        return self.b.bias

    def dense_weight(self) -> torch.Tensor:
        """The composed [d_out, d_in] matrix (engines pack this for their GEMMs)."""
        return self.b.weight @ self.a.weight


class LoRALinear(nn.Module):
    """Context operator factored as d_in -> r -> d_out.

    `.weight` materialises the product `up @ down` so kernels that want a dense
    matrix can read one; the module itself applies the two factors in sequence.
    """

    def __init__(self, d_in: int, rank: int, d_out: int, bias: bool = False):
        super().__init__()
        self.down = nn.Linear(d_in, rank, bias=False)
        self.up = nn.Linear(rank, d_out, bias=bias)

    def forward(self, x):
        return self.up(self.down(x))

    @property
    def weight(self):
        return self.up.weight @ self.down.weight

    @property
    def bias(self):
        return self.up.bias


class SwiGLU(nn.Module):
    """w2( silu(w1 x) * w3 x ), no biases."""

    def __init__(self, d_model: int, hidden: int):
        super().__init__()
        self.w1 = nn.Linear(d_model, hidden, bias=False)
        self.w3 = nn.Linear(d_model, hidden, bias=False)
        self.w2 = nn.Linear(hidden, d_model, bias=False)

    def forward(self, x):
        return self.w2(F.silu(self.w1(x)) * self.w3(x))
