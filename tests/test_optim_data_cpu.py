"""FusedAdam's PyTorch fallback path (CPU parameters), the gradient norm helper, the tile dataset
and the device prefetcher on CPU."""

import numpy as np
import torch

from dist_utils import run_distributed


def test_fused_adam_cpu_path_matches_torch():
    from jigsaw_b200.optim import FusedAdam, fused_grad_norm

    torch.manual_seed(0)
    for adamw in (False, True):
        ours = [torch.randn(5, 7, requires_grad=True), torch.randn(11, requires_grad=True)]
        theirs = [p.detach().clone().requires_grad_(True) for p in ours]
        kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.05)
        a = FusedAdam(ours, decoupled_weight_decay=adamw, **kw)
        b = (torch.optim.AdamW if adamw else torch.optim.Adam)(theirs, **kw)
        for _ in range(5):
            for p, q in zip(ours, theirs):
                g = torch.randn_like(p)
                p.grad, q.grad = g.clone(), g.clone()
            n = fused_grad_norm([p.grad for p in ours])
            torch.testing.assert_close(n, torch.sqrt(sum(q.grad.pow(2).sum() for q in theirs)))
            a.step()
            b.step()
        for p, q in zip(ours, theirs):
            torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


def _worker_data(rank, world, tmp):
    import jigsaw_b200 as jb
    from jigsaw_b200.data import DevicePrefetcher, TileDataset, replica_sampler
    from torch.utils.data import DataLoader

    mesh = jb.make_process_mesh({"dp": 2, "sh": 2, "col": 1}, model_parallel_axes=("sh", "col"))
    path = f"{tmp}/samples.npy"
    if rank == 0:
        np.save(path, np.arange(12 * 2 * 8 * 6, dtype=np.float32).reshape(12, 2, 8, 6))
    import torch.distributed as dist

    dist.barrier()
    ds = TileDataset(path, splits={1: mesh["sh"]})
    assert len(ds) == 12 and ds[3][0].shape == (2, 4, 6) and ds[3][1] == 3
    full = np.load(path)
    h0 = mesh["sh"].rank() * 4
    assert np.array_equal(ds[5][0].numpy(), full[5][:, h0:h0 + 4])
    sampler = replica_sampler(ds, mesh, seed=1)
    sampler.set_epoch(0)
    loader = DataLoader(ds, batch_size=2, sampler=sampler, drop_last=True)
    pre = DevicePrefetcher(loader, "cpu")
    seen = [idx for _, idx in pre]
    assert len(seen) == 3 and all(len(i) == 2 for i in seen)
    mine = torch.cat(seen)
    both = [torch.empty_like(mine) for _ in range(2)]
    dist.all_gather(both, mine, group=mesh["dp"])
    assert not set(both[0].tolist()) & set(both[1].tolist())
    same = [torch.empty_like(mine) for _ in range(2)]
    dist.all_gather(same, mine, group=mesh["sh"])
    assert torch.equal(same[0], same[1])


def test_tile_dataset_and_sampler(tmp_path):
    run_distributed(_worker_data, 4, str(tmp_path))


def test_fused_adam_with_tensor_learning_rate_on_cpu():
    """A learning rate given as a one-element tensor (the form that a CUDA graph can read at replay time)
    gives the same updates as the float, and changing it in place changes the next step."""
    from jigsaw_b200.optim import FusedAdam

    torch.manual_seed(0)
    a = torch.nn.Parameter(torch.randn(7))
    b = torch.nn.Parameter(a.detach().clone())
    lr = torch.tensor(1e-2)
    oa = FusedAdam([a], lr=1e-2, weight_decay=0.1, decoupled_weight_decay=True)
    ob = FusedAdam([b], lr=lr, weight_decay=0.1, decoupled_weight_decay=True)
    for i in range(4):
        if i == 2:                                   # a schedule: the float is replaced, the tensor overwritten
            oa.param_groups[0]["lr"] = 5e-3
            lr.fill_(5e-3)
        g = torch.randn(7)
        a.grad, b.grad = g.clone(), g.clone()
        oa.step()
        ob.step()
    assert torch.allclose(a, b, atol=1e-7)
