"""A dataloader for a domain-parallel model: each rank reads only its tile (``jigsaw_b200.data``).

1. ``TileDataset`` slices the memory-mapped file, so a rank never holds a whole sample.
2. ``replica_sampler`` keys the shuffling by the data-parallel index: the ranks of a copy draw the same
   samples in the same order, different copies draw different ones; ``drop_last`` keeps the number of
   steps (and of collectives) equal.
3. Per-sample randomness must be seeded by the sample index, not by the rank.
4. ``DevicePrefetcher`` stages batches in pinned memory and copies them on a side stream.

The mesh is 2 copies of a model cut in two along the height.  The script checks that the tiles of a
copy fit together into the stored sample and that the copies never see the same sample.

    torchrun --nproc-per-node 4 examples/dataloader.py

Counterpart of the reference tutorial examples/dataloader.py.
"""

import tempfile
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
from torch.utils.data import DataLoader

from _common import setup

import jigsaw_b200 as jb
from jigsaw_b200.data import DevicePrefetcher, TileDataset, replica_sampler

N, C, H, W = 16, 2, 16, 16


def main(num_workers: int = 2) -> None:
    device, rank, world = setup()
    mesh = jb.make_process_mesh({"dp": 2, "sh": 2, "sw": 1, "col": 1}, model_parallel_axes=("sh", "sw", "col"))
    holder = [None]
    if rank == 0:                                   # a node-local directory; use a shared file system across nodes
        root = Path(tempfile.mkdtemp())
        arr = np.lib.format.open_memmap(root / "samples.npy", mode="w+", dtype=np.float32, shape=(N, C, H, W))
        arr[:] = np.random.default_rng(0).standard_normal((N, C, H, W))
        arr.flush()
        holder = [root]
    dist.broadcast_object_list(holder, src=0)
    path = holder[0] / "samples.npy"

    dataset = TileDataset(path, splits={1: mesh["sh"], 2: mesh["sw"]})          # sample dims (C, H, W) = (0, 1, 2)
    sampler = replica_sampler(dataset, mesh, seed=0)
    loader = DataLoader(dataset, batch_size=2, sampler=sampler, num_workers=num_workers, drop_last=True)
    full = np.load(path, mmap_mode="r")
    for epoch in range(2):
        sampler.set_epoch(epoch)
        seen = []
        for x, idx in DevicePrefetcher(loader, device):
            idx_dev = idx.to(device)
            same = [torch.empty_like(idx_dev) for _ in range(mesh["model"].size())]
            dist.all_gather(same, idx_dev, group=mesh["model"])
            assert all(torch.equal(s, idx_dev) for s in same), "ranks of one copy drew different samples"
            whole = jb.gather.gather_results(x, mesh, pm_key_row="sh", pm_key_col="sw")
            assert np.array_equal(whole.cpu().numpy(), full[idx.cpu().numpy()]), "tiles do not fit together"
            seen.append(idx_dev)
        mine = torch.cat(seen)
        both = [torch.empty_like(mine) for _ in range(2)]
        dist.all_gather(both, mine, group=mesh["dp"])
        assert not set(both[0].tolist()) & set(both[1].tolist()), "two copies saw the same sample"
        assert len(set(both[0].tolist()) | set(both[1].tolist())) == N
    jb.log.info("all checks passed")


if __name__ == "__main__":
    main()
