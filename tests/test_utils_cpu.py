"""Small runtime utilities on CPU: buffer cache, activation offloader (pass-through without CUDA),
autocast policy helpers, config checks, shard descriptions."""

import pytest
import torch


def test_preallocated_buffers_are_cached_per_call_site():
    from jigsaw_b200._core import buffers

    buffers.clear_preallocated_buffers()

    def site(shape, **kw):
        return buffers.preallocated_buffer(shape, torch.float32, "cpu", depth=1, **kw)

    a = site((4, 8))
    a.fill_(3.0)
    b = site((4, 8))
    assert a.data_ptr() == b.data_ptr() and float(b.sum()) == 96.0         # same line -> same storage, contents kept
    c = site((2, 8), zero=True)
    assert c.data_ptr() == a.data_ptr() and float(c.sum()) == 0.0
    big = site((16, 16))
    assert big.numel() == 256                                               # grows when needed
    other = buffers.preallocated_buffer((4, 8), torch.float32, "cpu", index=1)
    assert other.data_ptr() != big.data_ptr()
    buffers.clear_preallocated_buffers()
    assert not buffers._cache


def test_buffer_cache_keys_and_growth():
    """What tells two buffers apart: the calling line, the dtype, the device and the index; not the shape."""
    from jigsaw_b200._core import buffers

    buffers.clear_preallocated_buffers()
    try:
        first = buffers.preallocated_buffer((3, 3), torch.float32, "cpu")
        second = buffers.preallocated_buffer((3, 3), torch.float32, "cpu")       # another line: its own storage
        assert first.data_ptr() != second.data_ptr() and not first.any() and first.shape == (3, 3)
        first.fill_(1.0)
        second.fill_(2.0)
        assert bool((first == 1.0).all()) and bool((second == 2.0).all())

        def site(shape=(8,), dtype=torch.float32, device="cpu", index=0):
            return buffers.preallocated_buffer(shape, dtype, device, index, depth=1)

        before = len(buffers._cache)
        a = site()
        assert len(buffers._cache) == before + 1
        for _ in range(50):
            assert site().data_ptr() == a.data_ptr()                              # steady state: no new storage
        assert len(buffers._cache) == before + 1
        assert site(dtype=torch.float64).data_ptr() != a.data_ptr() and site(dtype=torch.float64).dtype == torch.float64
        assert site(index=1).data_ptr() != a.data_ptr()
        assert site(device="meta").device.type == "meta"
        assert len(buffers._cache) == before + 4
        # one entry serves every shape asked for at the line: grown once, then trimmed views of it
        big = site((4, 16))
        assert big.shape == (4, 16) and not big.any() and big.data_ptr() != a.data_ptr()
        big.fill_(7.0)
        small = site((2, 3))
        assert small.data_ptr() == big.data_ptr() and float(small.sum()) == 42.0   # contents are the caller's business
        assert float(site((2, 3), ).sum()) == 42.0
        assert len(buffers._cache) == before + 4
        volume = site((2, 3, 4))
        volume[1, 2, 3] = 5.0
        assert float(volume[1, 2, 3]) == 5.0 and volume.is_contiguous()
    finally:
        buffers.clear_preallocated_buffers()


def test_offloader_is_transparent_on_cpu():
    from jigsaw_b200._core.offload import ActivationOffloader

    off = ActivationOffloader("cpu")
    t = torch.randn(5)
    assert off.offload(t) is t
    off.wait_offloads()
    dev, ev = off.prefetch(t)
    assert dev is t and ev is None and off.consume(dev, ev) is t


def test_autocast_helpers():
    from jigsaw_b200._core import autocast as A

    x, w = torch.randn(3, dtype=torch.bfloat16), torch.randn(3)
    assert A.autocast_dtype("cpu") is None
    assert A.cast_to_autocast_dtype(x, None, w) == (x, None, w)
    assert A.promote_to_fp32_under_autocast(x)[0].dtype == torch.bfloat16
    assert A.resolve_matmul_dtype(torch.device("cpu"), x, w) == torch.float32
    with torch.autocast("cpu", dtype=torch.bfloat16):
        assert A.autocast_dtype("cpu") == torch.bfloat16
        cx, none, cw = A.cast_to_autocast_dtype(x, None, w)
        assert cx.dtype == cw.dtype == torch.bfloat16 and none is None
        px, pd = A.promote_to_fp32_under_autocast(x, torch.randn(2, dtype=torch.float64))
        assert px.dtype == torch.float32 and pd.dtype == torch.float64
        assert A.resolve_matmul_dtype(torch.device("cpu"), w, w) == torch.bfloat16


def test_config_check_and_shard_repr():
    from jigsaw_b200._core.config import check_config
    from jigsaw_b200._core.shard_repr import shard_repr

    class Cfg:
        _layer_key = {"kernel_size": (3, 3), "bias": True}

    check_config(Cfg(), {"kernel_size": (3, 3), "bias": True})
    with pytest.raises(ValueError, match="different layer"):
        check_config(Cfg(), {"kernel_size": (5, 5)})
    assert shard_repr(row=None, col=4) == "row=1, col=4"
    assert shard_repr(spatial=(None, 2)) == "spatial=(1, 2)"


def test_ring_attention_config_validation():
    from jigsaw_b200.modules.attention import Offload, RingAttentionConfig, SaveScope, SendOp

    cfg = RingAttentionConfig(device="cpu", send_op="hybrid", intra_size=2, save_scope="local")
    assert cfg.send_op is SendOp.HYBRID and cfg.save_scope is SaveScope.LOCAL
    with pytest.raises(ValueError, match="must be one of"):
        RingAttentionConfig(device="cpu", send_op="zigzag")
    with pytest.raises(ValueError, match="save_scope=GLOBAL"):
        RingAttentionConfig(device="cuda", offload=Offload.CPU, save_scope="local")
    with pytest.raises(ValueError, match="CUDA"):
        RingAttentionConfig(device="cpu", offload="cpu")
    with pytest.raises(ValueError, match="intra_size"):
        RingAttentionConfig(device="cpu", send_op="hybrid", intra_size=0)


def test_chunk_owner_schedules_visit_every_chunk_once():
    from jigsaw_b200.modules.attention import SendOp
    from jigsaw_b200.modules.attention._ring import chunk_owner

    for op, P, A in ((SendOp.RING, 6, 1), (SendOp.BROADCAST, 5, 1), (SendOp.HYBRID, 8, 4), (SendOp.HYBRID, 6, 2)):
        for p in range(P):
            owners = [chunk_owner(op, p, s, P, A) for s in range(P)]
            assert sorted(owners) == list(range(P)), (op, P, A, p, owners)
    with pytest.raises(ValueError):
        chunk_owner(SendOp.HYBRID, 0, 0, 6, 4)
    # every ring size up to 12 with every intra size that divides it, all four schedules
    for P in range(1, 13):
        for A in [a for a in range(1, P + 1) if P % a == 0]:
            for op in SendOp:
                for p in range(P):
                    owners = [chunk_owner(op, p, s, P, A) for s in range(P)]
                    assert sorted(owners) == list(range(P)), (op, P, A, p, owners)
                if op in (SendOp.RING, SendOp.HYBRID):
                    # at each step the positions read from distinct owners: no owner serves two readers at once
                    for step in range(P):
                        assert len({chunk_owner(op, p, step, P, A) for p in range(P)}) == P, (op, P, A, step)
                else:
                    # the broadcast forms: at each step all positions of an intra group read one and the same owner
                    for step in range(P):
                        width = P if op is SendOp.BROADCAST else A
                        for first in range(0, P, width):
                            assert len({chunk_owner(op, p, step, P, A) for p in range(first, first + width)}) == 1
                if op in (SendOp.HYBRID, SendOp.HYBRID_BROADCAST):
                    # the first A steps stay inside the own intra group
                    for p in range(P):
                        assert all(chunk_owner(op, p, step, P, A) // A == p // A for step in range(A))


def _worker_status_agreement(rank, world):
    """A kernel error code seen by one rank reaches every rank (host-side part of the bounded waits:
    the device tensor is replaced by a CPU tensor, the reduction is the same)."""
    import torch
    from jigsaw_b200.ops import symm

    mine = torch.tensor([2 if rank == 1 else 0], dtype=torch.int32)
    assert symm.agree_on_status(mine) == 2
    assert int(mine) == (2 if rank == 1 else 0), "the local status word is left as it was"
    assert symm.agree_on_status(torch.zeros(1, dtype=torch.int32)) == 0


def test_kernel_status_is_agreed_over_ranks():
    from dist_utils import run_distributed

    run_distributed(_worker_status_agreement, 3, backend="gloo", timeout=120)


def test_block_range_check():
    """Host-side guard of every copy into a peer's copy of a block (pure arithmetic, no device needed)."""
    from jigsaw_b200.ops.symm import Block

    blk = Block(None, 0, 4096, 1 << 20, torch.empty(0))
    blk.check_range(256, 1 << 10)
    blk.check_range(256, 128, pitch=2048, rows=512)              # last row ends at 256 + 511 * 2048 + 128 = 1046912
    blk.check_range(0, 1 << 20)
    for bad in ((-1, 16, 0, 1), (0, 0, 0, 1), ((1 << 20) - 8, 16, 0, 1), (256, 128, 2048, 513), (0, 128, 64, 4), (0, 16, 0, 0)):
        with pytest.raises(ValueError):
            blk.check_range(*bad)
