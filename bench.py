"""Headline benchmark: images/s of the domain-parallel CNN training step on N B200s.

Configuration (fixed global problem, strong scaling): 8 ``DistributedConv2d`` layers (k3, p1,
64 channels, 3 input / 3 output channels) with GELU between, bf16 autocast, one global image
1 x 3 x 4096 x 4096 ~ N(0,1) tiled over the mesh, MSE loss against an N(0,1) target, Adam.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 10 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference through its own API

Rank 0 prints one JSON line.  ``value`` is timed on the device (CUDA events around exactly
``steps`` steps, barrier + synchronize on both sides, max over ranks) with the inputs
resident on the device; ``e2e`` repeats the measurement with the per-step host-to-device copy
of the input / target tiles from pinned memory and the device-to-host read of the loss inside
the timed region.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
MESHES = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (4, 2)}
IMAGE = 4096
DEPTH, WIDTH, CIN, COUT = 8, 64, 3, 3


def parse() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying a CUDA graph")
    ap.add_argument("--image", type=int, default=IMAGE, help="global image edge (default: the benchmark size)")
    ap.add_argument("--model", choices=("domaincnn", "sequential"), default="sequential",
                    help="ours: the same nn.Sequential of DistributedConv2d + nn.GELU layers that the reference arm builds "
                         "(default; the layers join into one fused chain), or the DomainCNN model class")
    return ap.parse_args()


def init_dist(n: int) -> tuple[int, int, torch.device]:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n:
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}; launch with torch.distributed.run for N > 1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    return rank, world, dev


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi (read-only) during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc, self.path = index, None, f"/tmp/jb_clocks_{os.getpid()}.csv"

    def start(self) -> None:
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=self.out, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [c.strip() for c in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def build(impl: str, mesh_shape: tuple[int, int], dev: torch.device, model_kind: str = "sequential"):
    """Model, loss and mesh of the chosen implementation, through its public API."""
    if impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import jigsaw as lib
    else:
        import jigsaw_b200 as lib
    mesh = lib.make_process_mesh({"sh": mesh_shape[0], "sw": mesh_shape[1], "col": 1})
    torch.manual_seed(0)
    if impl == "reference" or model_kind == "sequential":
        chans = [CIN] + [WIDTH] * (DEPTH - 1) + [COUT]
        layers = []
        for i in range(DEPTH):
            layers.append(lib.modules.DistributedConv2d(chans[i], chans[i + 1], kernel_size=3, padding=1, device=dev,
                                                        spatial_group=(mesh["sh"], mesh["sw"]), channel_group=mesh["col"]))
            if i + 1 < DEPTH:
                layers.append(torch.nn.GELU())
        model = torch.nn.Sequential(*layers)
    else:
        from jigsaw_b200.models import DomainCNN

        model = DomainCNN(mesh, dev, CIN, COUT, WIDTH, DEPTH)
    loss_fn = lib.modules.DistributedMSELoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    return model, loss_fn, mesh


def main() -> None:
    args = parse()
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "jigsaw")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
        return
    if args.gpus not in MESHES:
        raise SystemExit("--gpus must be 1, 2, 4 or 8")
    rank, world, dev = init_dist(args.gpus)
    ph, pw = MESHES[args.gpus]
    model, loss_fn, _mesh = build(args.impl, (ph, pw), dev, args.model)
    if args.impl == "ours":
        from jigsaw_b200.ops import _lib as _jb_lib

        _jb_lib.set_strict(True)       # a fused operation that declines its inputs raises: no silent library fallback
    graphed = args.impl == "ours" and not args.no_graph
    if args.impl == "ours":
        from jigsaw_b200.optim import FusedAdam

        opt = FusedAdam(model.parameters(), lr=1e-3)          # multi-tensor kernel, device-side step counter
    else:
        opt = torch.optim.Adam(model.parameters(), lr=1e-3, fused=True)
    H, W = args.image // ph, args.image // pw
    # every rank draws its own tile (synthetic data; the global image is 1 x 3 x image x image)
    g = torch.Generator().manual_seed(1234 + rank)
    x_host = torch.randn(1, CIN, H, W, generator=g).pin_memory()
    y_host = torch.randn(1, COUT, H, W, generator=g).pin_memory()
    x_dev, y_dev = x_host.to(dev), y_host.to(dev)

    def step(x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(x)
        # the reference's loss wants fp32 predictions; ours reads the bf16 channels-last output in place
        loss = loss_fn(out if args.impl == "ours" else out.float(), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    run = None
    if graphed:
        # the framework's whole-step CUDA graph: static inputs, one replay per step
        from jigsaw_b200.utils import GraphedStep

        run = GraphedStep(step, (x_dev, y_dev), warmup=max(args.warmup, 3))

    sizes = {"loss": 4}

    def timed(n_steps: int, e2e: bool) -> tuple[float, float]:
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        last = 0.0
        e0.record()
        if e2e and run is not None:
            # The framework's input pipeline: every step's inputs travel from pinned host memory on a side
            # stream while the previous step computes (DevicePrefetcher), land in the graph's static inputs,
            # and every step's loss is read back to the host a few steps behind its launch, so that neither the
            # read nor a late wake-up of one rank's host thread stalls the launches (the ranks wait for each
            # other's halos inside every step, so one late rank would hold up all of them).
            from jigsaw_b200.data import DevicePrefetcher

            lag = 3                                    # steps between a launch and the read of its loss
            host_loss = [torch.empty((), dtype=run.outputs.dtype).pin_memory() for _ in range(lag + 1)]
            done = [torch.cuda.Event() for _ in range(lag + 1)]
            sizes["loss"] = run.outputs.element_size()
            batches = ((x_host, y_host) for _ in range(n_steps))
            for i, (xb, yb) in enumerate(DevicePrefetcher(batches, dev, depth=lag + 1, reuse_buffers=True)):
                x_dev.copy_(xb)
                y_dev.copy_(yb)
                out = run.replay()
                host_loss[i % (lag + 1)].copy_(out, non_blocking=True)
                done[i % (lag + 1)].record()
                if i >= lag:
                    done[(i - lag) % (lag + 1)].synchronize()
                    last = float(host_loss[(i - lag) % (lag + 1)].item())
            for i in range(max(n_steps - lag, 0), n_steps):          # the losses still in flight
                done[i % (lag + 1)].synchronize()
                last = float(host_loss[i % (lag + 1)].item())
        for _ in range(0 if (e2e and run is not None) else n_steps):
            if e2e:
                x = x_host.to(dev, non_blocking=True)
                y = y_host.to(dev, non_blocking=True)
                out = step(x, y)
                sizes["loss"] = out.element_size()
                last = float(out.item())
            elif run is not None:
                loss = run.replay()
            else:
                loss = step(x_dev, y_dev)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        if not e2e:
            last = float(loss.item())
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()) / n_steps, last

    for _ in range(max(args.warmup, 0)):
        run.replay() if run is not None else step(x_dev, y_dev)
    torch.cuda.synchronize()
    launches0 = 0
    if args.impl == "ours":
        from jigsaw_b200.ops import _lib

        launches0 = _lib.LAUNCHES
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    ms_dev, loss_val = timed(args.steps, e2e=False)
    launches = (_lib.LAUNCHES - launches0) if args.impl == "ours" else 0
    if run is not None:
        launches = run.launches_per_step * args.steps      # replayed launches do not pass through Python
    timed(max(args.warmup, 6), e2e=True)   # untimed: the input pipeline's ring of staging buffers (5 slots) and streams come into being here
    ms_e2e, _ = timed(args.steps, e2e=True)
    clocks = sampler.stop() if rank == 0 else {}
    if args.impl == "ours":
        from jigsaw_b200.ops import symm

        symm.arena(dev).check_status(collective=True)      # every rank raises if any rank saw a kernel error
    if rank == 0:
        h2d = (x_host.numel() + y_host.numel()) * 4
        loss_bytes = sizes["loss"]
        line = {
            "metric": "CNN images/sec (domain-parallel 8x Conv2d(64ch,k3)+GELU, 1x3x4096x4096, fwd+bwd+Adam)",
            "value": 1000.0 / ms_dev,
            "unit": "images/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": ms_dev,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "bf16",
            "data": "synthetic N(0,1) image and target, random-init weights",
            "impl": args.impl,
            "config": {
                "model": f"CNN {DEPTH}xConv2d(k3,p1,{WIDTH}ch,{CIN}->{COUT})+GELU, MSE, Adam",
                "global_batch": 1,
                "image": [args.image, args.image],
                "seq_len": None,
                "parallelism": f"domain sh{ph} x sw{pw}",
                "cuda_graph": bool(graphed),
                "model_api": args.model if args.impl == "ours" else "sequential",
                "l2": "per-rank activations (>= 270 MB per layer) exceed the 126 MB L2; no explicit flush",
            },
            "clocks": clocks,
            "e2e": {"value": 1000.0 / ms_e2e, "unit": "images/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": loss_bytes},
            "gpu_launches": launches,
            "dispatch": _jb_lib.dispatch_counts() if args.impl == "ours" else None,
            "loss": loss_val,
        }
        print(json.dumps(line), flush=True)
    if run is not None:
        run.close()           # a live graph with captured collectives would stall the teardown
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
