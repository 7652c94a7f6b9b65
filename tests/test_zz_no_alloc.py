"""The allocation-free weight-gradient entry point against the regular one.

Some callers of the kernel library may not allocate device memory where they need a result
(a memory pool that must not grow, a loop that bans the device-wide synchronisation
cudaMalloc implies, a host application with a fixed amount of device memory).  For them the library exports
``jb_conv3x3_c64_wgrad_noalloc``, whose scratch is a static device array inside the library
image.  This test calls it through its exported C symbol, twice in a row (the scratch is
shared between calls and keeps the previous contents), and compares weight and bias gradient
with the regular entry point that takes caller-allocated scratch.  It also checks the size
limit.  The file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _padded(x):
    n, c, h, w = x.shape
    p = torch.zeros(n, h + 2, w + 2, c, device=x.device, dtype=torch.bfloat16)
    p[:, 1:-1, 1:-1, :] = x.permute(0, 2, 3, 1)
    return p


def test_noalloc_wgrad_matches_regular_entry_point_twice():
    from jigsaw_b200.ops import _lib

    L = _lib.lib()
    fn = L.jb_conv3x3_c64_wgrad_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    sm = _lib.sm_count(0)
    stream = torch.cuda.current_stream().cuda_stream
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    scratch = torch.empty(L.jb_conv3x3_wgrad_scratch_floats(sm), dtype=torch.float32, device=dev)
    for call, shape in enumerate([(2, 70, 300), (1, 33, 128)]):
        torch.manual_seed(call)
        NB, H, W = shape
        xp = _padded(torch.randn(NB, 64, H, W, device=dev))
        gp = _padded(torch.randn(NB, 64, H, W, device=dev))
        gw_ref = torch.zeros(64, 64, 3, 3, device=dev)
        gb_ref = torch.zeros(64, device=dev)
        rc = L.jb_conv3x3_c64_wgrad(_ptr(xp), _ptr(gp), _ptr(gw_ref), _ptr(gb_ref), _ptr(scratch), NB, H, W, None,
                                    _ptr(status), sm, stream)
        assert rc == 0
        gw = torch.full((64, 64, 3, 3), float("nan"), device=dev)
        gb = torch.full((64,), float("nan"), device=dev)
        rc = fn(_ptr(xp), _ptr(gp), _ptr(gw), _ptr(gb), NB, H, W, 1, stream)
        assert rc == 0, f"call {call}: return code {rc}"
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        # same arithmetic, different number of partial sums: fp32 rounding differences only
        tol_w = 1e-4 * float(gw_ref.abs().max())
        tol_b = 1e-4 * float(gb_ref.abs().max())
        assert float((gw - gw_ref).abs().max()) <= tol_w, f"call {call}: weight gradient differs"
        assert float((gb - gb_ref).abs().max()) <= tol_b, f"call {call}: bias gradient differs"
        # and both agree with PyTorch in fp32
        x = xp[:, 1:-1, 1:-1].permute(0, 3, 1, 2).float()
        g = gp[:, 1:-1, 1:-1].permute(0, 3, 1, 2).float()
        ref = torch.nn.grad.conv2d_weight(x, (64, 64, 3, 3), g, padding=1)
        assert float((gw - ref).abs().max()) <= 1e-3 * float(ref.abs().max())


def test_noalloc_wgrad_rejects_oversize():
    from jigsaw_b200.ops import _lib

    L = _lib.lib()
    fn = L.jb_conv3x3_c64_wgrad_noalloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    dummy = torch.zeros(16, device=dev)
    # nothing is launched for a refused size, so the dummy pointers are never dereferenced
    assert fn(_ptr(dummy), _ptr(dummy), _ptr(dummy), None, 2, 4096, 4096, 0, None) == -5
