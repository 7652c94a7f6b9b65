"""The CPU / gloo workload: a two-layer domain-parallel CNN in fp32 on four CPU ranks, for this framework
and for the unmodified reference (``--impl reference``, from ``baseline/_ref``), with parity against the
undivided PyTorch model trained on the whole images.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29620 \\
        benchmarks/cpu_cnn.py [--impl reference]

Mesh ``{sh: 2, sw: 2, col: 1}``, global batch 2 x 3 x 512 x 512 (tiles of 256 x 256),
Conv2d(3 -> 16, k3, p1) -> GELU -> Conv2d(16 -> 3, k3, p1), DistributedMSELoss over (sh, sw), Adam lr 1e-3,
seed 0.  The first ten steps are compared with the undivided model (loss curve, final parameters); wall-clock
per step is taken over ``--steps`` further steps between barriers.  Rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch
import torch.distributed as dist
from torch import nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--image", type=int, default=512)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if world != 4:
        raise SystemExit("this workload is defined for 4 ranks")
    torch.set_num_threads(max(1, (os.cpu_count() or 4) // world))
    dist.init_process_group("gloo")
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import jigsaw as lib
    else:
        import jigsaw_b200 as lib
    dev = torch.device("cpu")
    mesh = lib.make_process_mesh({"sh": 2, "sw": 2, "col": 1})
    groups = (mesh["sh"], mesh["sw"])

    torch.manual_seed(0)
    serial = nn.Sequential(nn.Conv2d(3, 16, 3, padding=1), nn.GELU(), nn.Conv2d(16, 3, 3, padding=1))
    conv = lambda i, o: lib.modules.DistributedConv2d(i, o, kernel_size=3, padding=1, device=dev, spatial_group=groups,  # noqa: E731
                                                     channel_group=mesh["col"])
    model = nn.Sequential(conv(3, 16), nn.GELU(), conv(16, 3))
    with torch.no_grad():
        for p, q in zip(model.parameters(), serial.parameters()):
            p.copy_(q)
    loss_fn = lib.modules.DistributedMSELoss(reduce_groups=groups)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    opt_s = torch.optim.Adam(serial.parameters(), lr=1e-3)

    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 3, args.image, args.image, generator=g)
    y = torch.randn(2, 3, args.image, args.image, generator=g)
    th, tw = args.image // 2, args.image // 2
    r, c = mesh["sh"].rank(), mesh["sw"].rank()
    xt = x[:, :, r * th:(r + 1) * th, c * tw:(c + 1) * tw].contiguous()
    yt = y[:, :, r * th:(r + 1) * th, c * tw:(c + 1) * tw].contiguous()

    def step() -> float:
        loss = loss_fn(model(xt), yt)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return float(loss.detach())

    losses, losses_s = [], []
    for _ in range(10):
        losses.append(step())
        ls = nn.functional.mse_loss(serial(x), y)
        opt_s.zero_grad(set_to_none=True)
        ls.backward()
        opt_s.step()
        losses_s.append(float(ls))
    loss_diff = max(abs(a - b) for a, b in zip(losses, losses_s))
    param_diff = max(float((p.detach() - q.detach()).abs().max()) for p, q in zip(model.parameters(), serial.parameters()))

    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dist.barrier()
    ms = torch.tensor([(time.perf_counter() - t0) / args.steps * 1e3], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(json.dumps({
            "impl": args.impl, "workload": "cpu_gloo_cnn", "world": world, "dtype": "fp32", "threads_per_rank": torch.get_num_threads(),
            "ms_per_step": round(float(ms), 2), "steps": args.steps, "loss_first": losses[0], "loss_step10": losses[-1],
            "max_loss_diff_vs_undivided": loss_diff, "max_param_diff_vs_undivided": param_diff,
        }))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
