"""The allocation-free column reduction (`dmb_col_reduce_acc_noalloc`, csrc/noalloc.h).

Some users of the kernel library may not allocate device memory at all: code running
inside somebody else's fixed memory arena (a serving process that accounts for every byte),
or code that must be certain no hidden allocation can fail in the middle of a step.
For them the library exports one entry point that carries its own scratch in a fixed
array inside the library image.  This test calls that entry point through its exported
C symbol, exactly as such a caller would (raw pointers and a stream, nothing else), and
checks it against the ordinary entry point, which is given caller-allocated scratch.
It does so on two calls in a row, because the built-in array keeps the previous call's
contents and the second call must not be disturbed by them; and it checks that an input
wider than the array is refused with a readable message rather than computed wrongly.

The file name sorts last on purpose: a run that stops at the first failure has then
already been through every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from dual_mod_public_b200.ops.cuda_ops import load_library
    lib = load_library()
    p, i, ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
    lib.dmb_col_reduce_acc_noalloc.restype = i
    lib.dmb_col_reduce_acc_noalloc.argtypes = [p, i, p, ll, p, p, i, i, p]
    lib.dmb_col_reduce_acc.restype = i
    lib.dmb_col_reduce_acc.argtypes = [p, i, p, ll, p, p, i, p, i, i, p]
    lib.dmb_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ordinary(lib, dy, x, rstd, rows, d):
    nsplit = max(1, min(64, rows // 64))
    scratch = torch.empty(nsplit * d, dtype=torch.float32, device="cuda")      # caller-allocated
    out = torch.full((d,), 0.5, dtype=torch.float32, device="cuda")
    rc = lib.dmb_col_reduce_acc(dy.data_ptr(), int(dy.dtype == torch.float32),
                                x.data_ptr() if x is not None else None, d,
                                rstd.data_ptr() if rstd is not None else None,
                                scratch.data_ptr(), nsplit, out.data_ptr(), rows, d, _stream())
    assert rc == 0
    return out


def _no_alloc(lib, dy, x, rstd, rows, d):
    out = torch.full((d,), 0.5, dtype=torch.float32, device="cuda")
    rc = lib.dmb_col_reduce_acc_noalloc(dy.data_ptr(), int(dy.dtype == torch.float32),
                                        x.data_ptr() if x is not None else None, d,
                                        rstd.data_ptr() if rstd is not None else None,
                                        out.data_ptr(), rows, d, _stream())
    assert rc == 0, lib.dmb_noalloc_last_error()
    return out


def test_no_alloc_entry_matches_ordinary_entry_twice_in_a_row():
    lib = _lib()
    torch.manual_seed(0)
    # first call: weighted reduction (the RMSNorm weight gradient), bf16 inputs
    rows, d = 4096, 1024
    dy = torch.randn(rows, d, device="cuda").bfloat16()
    x = torch.randn(rows, d, device="cuda").bfloat16()
    rstd = torch.rand(rows, device="cuda") + 0.5
    a = _no_alloc(lib, dy, x, rstd, rows, d)
    b = _ordinary(lib, dy, x, rstd, rows, d)
    ref = 0.5 + (dy.float() * x.float() * rstd[:, None]).sum(0)
    torch.cuda.synchronize()
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-5)
    assert torch.allclose(a, ref, rtol=2e-2, atol=2e-2 * ref.abs().max().item())
    # second call, different shape and mode (plain fp32 column sum): the array still holds the
    # first call's partial sums and they must not leak into this result
    rows2, d2 = 1000, 2304
    dy2 = torch.randn(rows2, d2, device="cuda")
    a2 = _no_alloc(lib, dy2, None, None, rows2, d2)
    b2 = _ordinary(lib, dy2, None, None, rows2, d2)
    torch.cuda.synchronize()
    assert torch.allclose(a2, b2, rtol=1e-5, atol=1e-5)
    assert torch.allclose(a2, 0.5 + dy2.sum(0), rtol=1e-4, atol=1e-3)


def test_no_alloc_entry_refuses_inputs_wider_than_its_array():
    lib = _lib()
    d = 8192 + 64
    dy = torch.zeros(8, d, device="cuda")
    out = torch.zeros(d, device="cuda")
    rc = lib.dmb_col_reduce_acc_noalloc(dy.data_ptr(), 1, None, d, None, out.data_ptr(), 8, d, _stream())
    assert rc == -3
    msg = lib.dmb_noalloc_last_error().decode()
    assert "8192" in msg and "columns" in msg
    torch.cuda.synchronize()
    assert out.abs().max().item() == 0.0
