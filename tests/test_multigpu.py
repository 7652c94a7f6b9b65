"""Multi-GPU tests of the fused halo-exchange convolution chain (peer stores over NVLink):
the fused chain on a tiled image must match the unfused torch + NCCL path of the same model,
which in turn is pinned against the undivided torch layers by the CPU tests."""

import pytest
import torch

from dist_utils import assert_close, run_distributed

pytestmark = pytest.mark.gpu


def _worker_chain(rank, world, mesh_shape):
    import os

    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import jigsaw_b200 as jb
    from jigsaw_b200.models import DomainCNN
    from jigsaw_b200.ops import symm

    dev = torch.device("cuda", rank)
    mesh = jb.make_process_mesh({"sh": mesh_shape[0], "sw": mesh_shape[1], "col": 1})
    torch.manual_seed(0)
    fused = DomainCNN(mesh, dev, depth=4)
    plain = DomainCNN(mesh, dev, depth=4, fuse=False)
    plain.load_state_dict(fused.state_dict())
    loss_fn = jb.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(2, 3, 40, 136, generator=g).to(dev)
    y = torch.randn(2, 3, 40, 136, generator=g).to(dev)
    for step in range(2):      # twice: buffers, flag slots and epochs are recycled
        for m in (fused, plain):
            m.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out_f = fused(x)
        loss_f = loss_fn(out_f.float(), y)
        loss_f.backward()
        out_p = plain(x)                       # fp32 oracle through torch + NCCL halo exchange
        loss_p = loss_fn(out_p, y)
        loss_p.backward()
        symm.arena(dev).check_status()
        scale = float(out_p.abs().max())
        assert_close(out_f.float(), out_p, f"step {step}: output", 0.0, 3e-2 * scale)
        assert_close(loss_f, loss_p, f"step {step}: loss", 2e-2, 0.0)
        for (n, p), q in zip(fused.named_parameters(), plain.parameters()):
            gs = float(q.grad.abs().max())
            assert_close(p.grad, q.grad, f"step {step}: grad {n}", 0.0, 6e-2 * gs + 1e-7)
    jb.debug.assert_replica_consistency(fused, mesh)


@pytest.mark.multigpu(2)
def test_fused_chain_two_gpus_rows():
    run_distributed(_worker_chain, 2, (2, 1), backend="nccl", timeout=300)


@pytest.mark.multigpu(2)
def test_fused_chain_two_gpus_cols():
    run_distributed(_worker_chain, 2, (1, 2), backend="nccl", timeout=300)


@pytest.mark.multigpu(4)
def test_fused_chain_four_gpus_with_corners():
    run_distributed(_worker_chain, 4, (2, 2), backend="nccl", timeout=300)
