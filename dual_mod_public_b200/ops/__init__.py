"""Device op tables.  `default_ops(device)` returns the sm_100a kernel table on a
CUDA device (and raises if the extension is missing there: a silent fallback
would hide that the kernels are not running) and the plain-torch table on CPU."""

from __future__ import annotations

import torch

from .torch_ops import TorchOps

_cache = {}


def default_ops(device):
    device = torch.device(device)
    key = (device.type, device.index)
    if key not in _cache:
        if device.type == "cuda":
            from .cuda_ops import CudaOps
            _cache[key] = CudaOps(device)
        else:
            _cache[key] = TorchOps()
    return _cache[key]


__all__ = ["TorchOps", "default_ops"]
