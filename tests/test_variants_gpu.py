"""Single-GPU checks that are sorted last on purpose, because they reach kernel variants that no other test
reaches: the scatter epilogue of the tcgen05 GEMM with both slabs on this GPU (column part ``p`` of the product
goes to slab ``p``), and the Adam kernel that reads its learning rate from device memory."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("staged", [False, True])
@pytest.mark.parametrize("M,K,part_cols,b_mn", [(300, 256, 256, False), (9516, 128, 256, True), (520, 192, 64, False), (520, 192, 64, True), (1000, 128, 128, True)])
def test_scatter_epilogue_into_local_slabs(M, K, part_cols, b_mn, staged):
    """The GEMM whose epilogue stores column part ``p`` of the product into slab ``p``; here both slabs
    are buffers of this GPU, so that the epilogue's addressing is checked without peers.  Both forms
    of the epilogue: row-per-thread stores, and the staged one (tiles leave through shared memory as
    128-byte row pieces) that the library uses."""
    import ctypes

    from jigsaw_b200.ops import _lib, symm

    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    parts = 2
    N = parts * part_cols
    A = torch.randn(M, K, device=dev).bfloat16()
    B = torch.randn(N, K, device=dev).bfloat16()
    b = B.t().contiguous() if b_mn else B
    slabs = [torch.full((M, part_cols), float("nan"), device=dev, dtype=torch.bfloat16) for _ in range(parts)]
    c_part = (ctypes.c_void_p * 8)()
    for i, t in enumerate(slabs):
        c_part[i] = t.data_ptr()
    L = _lib.lib()
    ar = symm.arena(dev)
    fn = L.jb_gemm_bf16_scatter_staged if staged else L.jb_gemm_bf16_scatter
    rc = fn(ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(b.data_ptr()), c_part, parts, part_cols, M, K, A.stride(0),
            b.stride(0), 0, 1 if b_mn else 0, _lib.sm_count(0), ctypes.c_void_p(ar.status.data_ptr()), _lib.stream_ptr())
    assert rc == 0
    torch.cuda.synchronize()
    ar.check_status()
    ref = A.float() @ B.float().t()
    for i, t in enumerate(slabs):
        assert not torch.isnan(t).any(), f"slab {i} has rows the epilogue did not write"
        assert _rel(t, ref[:, i * part_cols:(i + 1) * part_cols]) < 1e-2


def test_fused_adam_learning_rate_from_device_memory():
    """The Adam kernel that reads its learning rate from device memory against the one that takes it by
    value, including a change of the rate between steps."""
    from jigsaw_b200.optim import FusedAdam

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(n, device=dev)) for n in (1000, 70000, 33)]
    qs = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    lr = torch.full((), 1e-2, device=dev)
    oa = FusedAdam(ps, lr=1e-2, weight_decay=0.05, decoupled_weight_decay=True)
    ob = FusedAdam(qs, lr=lr, weight_decay=0.05, decoupled_weight_decay=True)
    for i in range(4):
        if i == 2:
            oa.param_groups[0]["lr"] = 3e-3
            lr.fill_(3e-3)
        for p, q in zip(ps, qs):
            p.grad = torch.randn_like(p)
            q.grad = p.grad.clone()
        oa.step()
        ob.step()
    torch.cuda.synchronize()
    for p, q in zip(ps, qs):
        assert torch.allclose(p, q, atol=1e-7, rtol=1e-6)
