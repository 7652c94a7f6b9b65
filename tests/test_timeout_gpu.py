"""The bounded waits of the kernels: a flag that nothing ever sets makes the wait run out after its
limit (2 s), the kernel returns, the status word names the failure, the host turns it into an
exception and the context stays usable.  No fault, trap or endless loop is involved."""

import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_flag_wait_times_out_and_reports():
    from jigsaw_b200.ops import _lib, linear_fused, symm

    dev = torch.device("cuda", 0)
    ar = symm.arena(dev)
    ar.check_status()                                   # clean before
    L = _lib.lib()
    n = 1024
    slabs = torch.ones(2, n, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    never = torch.zeros(4, device=dev, dtype=torch.int32)          # a flag word that stays 0
    flags = (ctypes.c_void_p * 8)()
    flags[0] = None
    flags[1] = never.data_ptr()
    t0 = time.time()
    rc = L.jb_sum_slabs(ctypes.c_void_p(slabs.data_ptr()), n, 2, flags, 1, 0, None, ctypes.c_void_p(out.data_ptr()), 1,
                        ctypes.c_void_p(ar.status.data_ptr()), _lib.sm_count(0), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    waited = time.time() - t0
    assert 1.5 < waited < 10.0, waited                   # the limit, not an endless wait
    with pytest.raises(RuntimeError, match="flag wait timed out"):
        ar.check_status()
    ar.check_status()                                   # the status word was cleared by the report
    # the context is still usable: a GEMM on the same stream gives the right answer
    a = torch.randn(256, 128, device=dev).bfloat16()
    b = torch.randn(64, 128, device=dev).bfloat16()
    c = linear_fused.gemm(a, b, out_dtype=torch.float32)
    torch.testing.assert_close(c, a.float() @ b.float().t(), rtol=2e-2, atol=2e-2)
    ar.check_status()
