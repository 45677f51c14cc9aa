"""Rotary position embedding, half-split pairing (dim i pairs with i + dh/2).

Queries are rotated when they read; a blended key k'' is rotated once, when it
is written to the tape, so the tape holds rotated keys and scores are plain dot
products (reference: models/dualmod/rope.py:1-33).
"""

from __future__ import annotations

import torch


def build_rope_cache(max_seq_len: int, head_dim: int, theta: float, device=None):
    """(cos, sin), each [max_seq_len, head_dim // 2] in fp32."""
    exponent = torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim
    inv_freq = theta ** (-exponent)
    angle = torch.arange(max_seq_len, device=device, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return angle.cos(), angle.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate x [..., T, dh] by the angles of cos/sin [T, dh/2]; fp32 math."""
    half = x.shape[-1] // 2
    xf = x.float()
    lo, hi = xf[..., :half], xf[..., half:]
    return torch.cat((lo * cos - hi * sin, hi * cos + lo * sin), dim=-1).to(x.dtype)


def unapply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Inverse rotation (the transpose of `apply_rope`); used by manual backward passes."""
    return apply_rope(x, cos, -sin)
