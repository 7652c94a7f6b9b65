"""Secondary benchmark workloads: the Vision Transformer, Swin and the 3-D encoder-decoder, for this
framework and for the unmodified reference (``--impl reference``, from ``baseline/_ref``).

Both arms build the *same* architecture from their own public layer API (the two APIs share
signatures), run ``--warmup`` untimed and ``--steps`` timed training steps (forward, loss,
backward, optimizer) on synthetic data under bf16 autocast, time on the device with CUDA events
(max over ranks) and print one JSON line.

    python benchmarks/workloads.py --config vit --gpus 1
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        --master-port 29600 benchmarks/workloads.py --config vit --gpus 2 [--impl reference]

Configurations (``--scale small`` shrinks depth / width for quick runs):
  vit     24 blocks, width 1024, 16 heads, MLP 4096, 1024x1024 image, patch 16 (4096 tokens), batch 8,
          4 input channels, 1000-class cross-entropy; mesh row x col = {1: 1x1, 2: 1x2, 4: 2x2, 8: 4x2}
  swin    1536^2 image, patch 4 (384^2 tokens), widths 128-256-512-1024, depths 2-2-18-2, heads 4-8-16-32,
          window 16 (the largest window that divides a stage's tile), 19-class map at 1/4 resolution, batch 2;
          replicated weights, tiles sh x sw = {1: 1x1, 2: 2x1, 4: 2x2, 8: 4x2}
  unet3d  channels 1-32-64-128, stride-2 Conv3d / ConvTranspose3d, GroupNorm(8) + GELU, BCE,
          volume 128^3 (256^3 with --scale full); mesh sh x sw = {1: 1x1, 2: 2x1, 4: 2x2, 8: 4x2}
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
from torch import nn

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
MESH2D = {1: (1, 1), 2: (1, 2), 4: (2, 2), 8: (4, 2)}
SEQUENCE_PARALLEL = "ring"          # how attention sees the whole sequence when rows split it: "ring" | "ulysses" (--seq)
TILES = {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (4, 2)}


def load(impl: str):
    if impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import jigsaw as lib
    else:
        import jigsaw_b200 as lib
    return lib


# ----------------------------------------------------------------------------- ViT (either API)
class Block(nn.Module):
    def __init__(self, lib, mesh, dev, dim, heads, hidden, ring):
        super().__init__()
        row, col, model = mesh["row"], mesh["col"], mesh["model"]
        M = lib.modules
        self.norm1 = M.DistributedLayerNorm(dim, model.rank(), dev, row, col)
        self.norm2 = M.DistributedLayerNorm(dim, model.rank(), dev, row, col)
        cfg = None
        if ring:
            from importlib import import_module

            att = import_module(lib.__name__ + ".modules.attention")
            cfg = M.RingAttentionConfig(device=dev, send_in_forward=att.SendForward.KV, save_for_backward=att.SaveBackward.KV)
        ulysses = ring and SEQUENCE_PARALLEL == "ulysses"
        self.attn = M.DistributedAttention(dim, dim, dim, heads, model.rank(), dev, spatial_group=row, channel_group=col,
                                           ring=ring and not ulysses, ulysses=ulysses, config=None if ulysses else cfg)
        self.fc1 = M.DistributedLinear(dim, hidden, device=dev, model_group=model, row_group=row, col_group=col, bias=True)
        self.fc2 = M.DistributedLinear(hidden, dim, device=dev, model_group=model, row_group=row, col_group=col, bias=True)

    def forward(self, x):
        x = x + self.attn(self.norm1(x))
        return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.norm2(x))))


class ViT(nn.Module):
    def __init__(self, lib, mesh, dev, image, patch, chans, dim, heads, depth, hidden, classes):
        super().__init__()
        row, col, model = mesh["row"], mesh["col"], mesh["model"]
        M = lib.modules
        self.row, self.patch = row, patch
        self.embed = M.DistributedConv2d(chans, dim, kernel_size=patch, stride=patch, device=dev, spatial_group=row,
                                         channel_group=col)
        self.blocks = nn.ModuleList(Block(lib, mesh, dev, dim, heads, hidden, row.size() > 1) for _ in range(depth))
        self.norm = M.DistributedLayerNorm(dim, model.rank(), dev, row, col)
        self.head = M.DistributedLinear(dim, classes, device=dev, model_group=col, row_group=row, col_group=col, bias=True)
        hp, wp, e = image // patch, image // patch // row.size(), dim // col.size()
        self.pos = nn.Parameter(torch.zeros(hp * wp, e, device=dev))
        self.tokens = hp * wp * row.size()

    def forward(self, x):
        z = self.embed(x)
        b, e, hp, wp = z.shape
        z = z.permute(0, 2, 3, 1).reshape(b, hp * wp, e).contiguous() + self.pos.to(z.dtype)
        for blk in self.blocks:
            z = blk(z)
        pooled = self.norm(z).sum(dim=1)
        if self.row.size() > 1:
            import torch.distributed.nn.functional as dfn

            pooled = dfn.all_reduce(pooled, group=self.row)
        return self.head(pooled / self.tokens)


MESH_OVERRIDE: tuple[int, int] | None = None   # --mesh RxC for the ViT (e.g. 2x1: ring attention on two GPUs)


def build_vit(lib, n, dev, scale):
    r, c = MESH_OVERRIDE or MESH2D[n]
    mesh = lib.make_process_mesh({"row": r, "col": c})
    small = scale == "small"
    image, patch, chans = (256 if small else 1024), 16, 4
    dim, heads, depth, hidden, classes, batch = (256, 4, 2, 1024, 1000, 8) if small else (1024, 16, 24, 4096, 1000, 8)
    torch.manual_seed(mesh["model"].rank())
    model = ViT(lib, mesh, dev, image, patch, chans, dim, heads, depth, hidden, classes)
    loss_fn = lib.modules.DistributedCrossEntropyLoss(mesh["col"], (mesh["row"],))
    g = torch.Generator().manual_seed(7)
    x = torch.randn(batch, chans, image, image, generator=g)
    x = x[:, mesh["col"].rank() * chans // c:(mesh["col"].rank() + 1) * chans // c]
    w = image // r
    x = x[..., mesh["row"].rank() * w:(mesh["row"].rank() + 1) * w].contiguous()
    y = torch.randint(0, classes, (batch,), generator=g)
    desc = {"model": f"ViT depth {depth} width {dim} heads {heads} mlp {hidden}, {image}x{image} patch {patch}",
            "global_batch": batch, "seq_len": (image // patch) ** 2, "parallelism": f"row{r} x col{c}" + (f", {SEQUENCE_PARALLEL} attention" if r > 1 else "")}
    return model, loss_fn, x, y, desc, batch


# ----------------------------------------------------------------------------- Swin (either API)
def _windows(x, ws):
    b, h, w, c = x.shape
    return x.view(b, h // ws, ws, w // ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(b, (h // ws) * (w // ws), ws * ws, c)


def _unwindows(x, ws, h, w):
    b, _, _, c = x.shape
    return x.view(b, h // ws, w // ws, ws, ws, c).permute(0, 1, 3, 2, 4, 5).reshape(b, h, w, c)


def _shift_mask(h, w, ws, shift, sh, sw):
    def region(local, group):
        g = group.rank() * local + torch.arange(local)
        total = group.size() * local
        return (g >= total - ws).long() + (g >= total - shift).long()

    label = region(h, sh)[:, None] * 3 + region(w, sw)[None, :]
    win = _windows(label[None, :, :, None].float(), ws)[0, :, :, 0]
    return torch.zeros(win.shape[0], ws * ws, ws * ws).masked_fill(win[:, :, None] != win[:, None, :], -100.0)


class SwinBlock(nn.Module):
    def __init__(self, lib, mesh, dev, dim, heads, tile, ws, shift):
        super().__init__()
        sh, sw = mesh["sh"], mesh["sw"]
        self.tile, self.ws, self.heads, self.shift = tile, ws, heads, shift
        self.norm1, self.norm2 = nn.LayerNorm(dim, device=dev), nn.LayerNorm(dim, device=dev)
        self.qkv, self.proj = nn.Linear(dim, 3 * dim, device=dev), nn.Linear(dim, dim, device=dev)
        self.fc1, self.fc2 = nn.Linear(dim, 4 * dim, device=dev), nn.Linear(4 * dim, dim, device=dev)
        self.bias = nn.Parameter(torch.zeros(heads, ws * ws, ws * ws, device=dev))
        mask = _shift_mask(tile[0], tile[1], ws, shift, sh, sw) if shift else torch.zeros(1, ws * ws, ws * ws)
        self.register_buffer("mask", mask.to(dev), persistent=False)
        if shift:
            M = lib.modules
            self.roll_in = M.DistributedRoll((-shift, -shift), (1, 2), (1, 2), (sh, sw), dev)
            self.roll_out = M.DistributedRoll((shift, shift), (1, 2), (1, 2), (sh, sw), dev)

    def forward(self, x):
        h, w = self.tile
        y = self.norm1(x)
        if self.shift:
            y = self.roll_in(y.contiguous())
        win = _windows(y, self.ws)
        b, nw, n, c = win.shape
        qkv = self.qkv(win).view(b, nw, n, 3, self.heads, c // self.heads).permute(3, 0, 1, 4, 2, 5)
        bias = (self.bias[None] + self.mask[:, None]).to(qkv.dtype)
        att = torch.nn.functional.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2], attn_mask=bias)
        y = _unwindows(self.proj(att.transpose(2, 3).reshape(b, nw, n, c)), self.ws, h, w)
        if self.shift:
            y = self.roll_out(y.contiguous())
        x = x + y
        return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.norm2(x))))


class Merge(nn.Module):
    def __init__(self, dev, dim, out):
        super().__init__()
        self.norm, self.reduce = nn.LayerNorm(4 * dim, device=dev), nn.Linear(4 * dim, out, bias=False, device=dev)

    def forward(self, x):
        return self.reduce(self.norm(torch.cat([x[:, i::2, j::2] for i in (0, 1) for j in (0, 1)], dim=-1)))


class Swin(nn.Module):
    """Tiled Swin with replicated weights: plain torch layers whose parameters are marked replicated over
    the tile groups and synchronised through the library (the pattern of the reference's Swin tutorial)."""

    def __init__(self, lib, mesh, dev, image, patch, chans, dims, heads, depths, window, classes):
        super().__init__()
        self.lib = lib
        sh, sw = mesh["sh"], mesh["sw"]
        M = lib.modules
        kw = dict(device=dev, spatial_group=(sh, sw), channel_group=mesh["col"])
        self.embed = M.DistributedConv2d(chans, dims[0], kernel_size=patch, stride=patch, **kw)
        tile = (image // patch // sh.size(), image // patch // sw.size())
        layers = []
        for i, (dim, hd, depth) in enumerate(zip(dims, heads, depths)):
            ws = max(d for d in range(1, window + 1) if tile[0] % d == 0 and tile[1] % d == 0)
            for j in range(depth):
                layers.append(SwinBlock(lib, mesh, dev, dim, hd, tile, ws, 0 if j % 2 == 0 else ws // 2))
            if i + 1 < len(dims):
                layers.append(Merge(dev, dim, dims[i + 1]))
                tile = (tile[0] // 2, tile[1] // 2)
        self.layers = nn.Sequential(*layers)
        self.norm = nn.LayerNorm(dims[-1], device=dev)
        up = 2 ** (len(dims) - 1)
        self.decode = M.DistributedConvTranspose2d(dims[-1], classes, kernel_size=up, stride=up, **kw)
        live = [g for g in (sh, sw) if g.size() > 1]
        if live:
            for mod in [self.layers, self.norm]:
                for p in mod.parameters():
                    lib.parallel.mark_replicated(p, live)
            lib.parallel.broadcast_replicas(self)

    def forward(self, x):
        synced = self.lib.parallel.synced_parameters(self)
        if synced:
            return torch.func.functional_call(self, synced, (x,))
        z = self.embed(x).permute(0, 2, 3, 1).contiguous()
        z = self.norm(self.layers(z)).permute(0, 3, 1, 2).contiguous()
        return self.decode(z)


def build_swin(lib, n, dev, scale):
    sh, sw = TILES[n]
    mesh = lib.make_process_mesh({"sh": sh, "sw": sw, "col": 1})
    small = scale == "small"
    image, patch, chans, classes, batch = (256 if small else 1536), 4, 3, 19, 2
    dims, heads, depths, window = ((32, 64), (2, 4), (2, 2), 8) if small else ((128, 256, 512, 1024), (4, 8, 16, 32), (2, 2, 18, 2), 16)
    torch.manual_seed(0)
    model = Swin(lib, mesh, dev, image, patch, chans, dims, heads, depths, window, classes)
    loss_fn = lib.modules.DistributedCrossEntropyLoss(None, (mesh["sh"], mesh["sw"]))
    g = torch.Generator().manual_seed(11)
    x = torch.randn(batch, chans, image, image, generator=g)
    y = torch.randint(0, classes, (batch, image // patch, image // patch), generator=g)
    h, w = image // sh, image // sw

    def tile(t, f=1):
        return t[..., mesh["sh"].rank() * h // f:(mesh["sh"].rank() + 1) * h // f,
                 mesh["sw"].rank() * w // f:(mesh["sw"].rank() + 1) * w // f].contiguous()

    desc = {"model": f"Swin {image}^2 patch {patch} dims {dims} depths {depths} window {window}, {classes}-class map at 1/{patch}",
            "global_batch": batch, "seq_len": (image // patch) ** 2, "parallelism": f"sh{sh} x sw{sw}"}
    return model, loss_fn, tile(x), tile(y, patch), desc, batch


DATA_PARALLEL = 1          # --dp N: N data-parallel replicas of the 3-D model (wrap_ddp with the joint hook)


def build_unet3d(lib, n, dev, scale):
    dp = DATA_PARALLEL
    sh, sw = TILES[n // dp]
    if dp > 1:
        mesh = lib.make_process_mesh({"dp": dp, "sh": sh, "sw": sw, "col": 1}, model_parallel_axes=("sh", "sw", "col"))
    else:
        mesh = lib.make_process_mesh({"sh": sh, "sw": sw, "col": 1})
    M = lib.modules
    size = {"small": 64, "default": 128, "full": 256}[scale]
    widths = (32, 64, 128)
    spatial = (None, mesh["sh"], mesh["sw"])
    kw = dict(device=dev, spatial_group=spatial, channel_group=mesh["col"])
    torch.manual_seed(0)

    def norm(ch):
        return M.DistributedGroupNorm(8, ch, dev, channel_group=mesh["col"], spatial_group=spatial)

    chans = (1, *widths)
    layers = []
    for i in range(3):
        layers += [M.DistributedConv3d(chans[i], chans[i + 1], 3, stride=2, padding=1, **kw), norm(chans[i + 1]), nn.GELU()]
    ups = (64, 32, 1)
    ins = (128, 64, 32)
    for i in range(3):
        layers.append(M.DistributedConvTranspose3d(ins[i], ups[i], 4, stride=2, padding=1, **kw))
        if i < 2:
            layers += [norm(ups[i]), nn.GELU()]
    model = nn.Sequential(*layers)
    if dp > 1:
        # every replica sees its own volume; DDP averages over dp and the joint hook folds the sum over the tile ranks in
        model = lib.parallel.wrap_ddp(model, mesh, dp_key="dp", joint_hook=True)
    loss_fn = M.DistributedBCEWithLogitsLoss(reduce_groups=(mesh["sh"], mesh["sw"]))
    g = torch.Generator().manual_seed(3 + (mesh["dp"].rank() if dp > 1 else 0))
    x = torch.randn(1, 1, size, size, size, generator=g)
    y = (torch.rand(1, 1, size, size, size, generator=g) > 0.5).float()
    h, w = size // sh, size // sw

    def tile(t):
        return t[..., mesh["sh"].rank() * h:(mesh["sh"].rank() + 1) * h, mesh["sw"].rank() * w:(mesh["sw"].rank() + 1) * w].contiguous()

    desc = {"model": f"3-D enc-dec 1-32-64-128, {size}^3", "global_batch": dp, "seq_len": None,
            "parallelism": (f"dp{dp} x " if dp > 1 else "") + f"sh{sh} x sw{sw}" + (", DDP with the joint hook" if dp > 1 else "")}
    return model, loss_fn, tile(x), tile(y), desc, dp


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", choices=("vit", "swin", "unet3d"), default="vit")
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--scale", default="default")
    ap.add_argument("--seq", choices=("ring", "ulysses"), default="ring", help="sequence parallelism of the ViT's attention")
    ap.add_argument("--dp", type=int, default=1, help="unet3d only: data-parallel replicas (the tile grid uses gpus / dp ranks)")
    ap.add_argument("--mesh", default=None, help="ViT only: rows x columns of the mesh, e.g. 2x1 (default: 1x1, 1x2, 2x2, 4x2)")
    ap.add_argument("--profile", default=None, metavar="FILE",
                    help="after the timed steps, run two more under torch.profiler and write rank 0's kernel table to FILE")
    ap.add_argument("--graph", action="store_true",
                    help="replay the whole step as one CUDA graph (this framework only; GraphedStep)")
    args = ap.parse_args()
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "jigsaw")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", 0)))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    lib = load(args.impl)
    global SEQUENCE_PARALLEL, MESH_OVERRIDE, DATA_PARALLEL
    SEQUENCE_PARALLEL = args.seq
    DATA_PARALLEL = args.dp
    if args.mesh:
        r, c = (int(v) for v in args.mesh.lower().split("x"))
        if r * c != args.gpus:
            raise SystemExit(f"--mesh {args.mesh} does not have {args.gpus} ranks")
        MESH_OVERRIDE = (r, c)
    builders = {"vit": build_vit, "swin": build_swin, "unet3d": build_unet3d}
    model, loss_fn, x, y, desc, batch = builders[args.config](lib, args.gpus, dev, args.scale)
    x, y = x.to(dev), y.to(dev)
    if args.impl == "ours":
        from jigsaw_b200.optim import FusedAdam

        opt = FusedAdam(model.parameters(), lr=1e-4, decoupled_weight_decay=True)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.0, fused=True)

    def step():
        with torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(x)
        loss = loss_fn(out.float(), y)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    run = step
    graphed = None
    if args.graph and args.impl == "ours":
        from jigsaw_b200.utils import GraphedStep

        graphed = GraphedStep(lambda a, b: step(), (x, y), warmup=max(args.warmup, 3))
        run = graphed.replay
    for _ in range(0 if graphed is not None else args.warmup):
        loss = run()
    launches0 = 0
    if args.impl == "ours":
        from jigsaw_b200.ops import _lib

        launches0 = _lib.LAUNCHES
    from bench import ClockSampler       # nvidia-smi clock / throttle-reason samples during the timed region (read-only)

    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = run()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], device=dev)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else {}
    dispatch = None
    launches = (_lib.LAUNCHES - launches0) if args.impl == "ours" else 0
    if graphed is not None:
        launches = graphed.launches_per_step * args.steps
    if args.impl == "ours":
        from jigsaw_b200.ops import symm

        symm.arena(dev).check_status(collective=True)      # every rank raises if any rank saw a kernel error
        dispatch = _lib.dispatch_counts()                   # per operation: calls on the fused kernels / declined
    if rank == 0:
        print(json.dumps({"metric": f"{args.config} samples/sec (fwd+bwd+AdamW)", "value": batch * 1000.0 / float(ms), "unit": "samples/s",
                          "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(ms), "impl": args.impl,
                          "dtype": "bf16", "data": "synthetic", "config": desc, "gpu_launches": launches,
                          "graph": graphed is not None, "loss": float(loss), "clocks": clocks, "dispatch": dispatch}), flush=True)
    if args.profile:
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            for _ in range(2):
                run()
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.profile, "w") as f:
                f.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=40, max_name_column_width=90))
    if graphed is not None:
        graphed.close()                      # a live graph that holds collectives blocks the teardown
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
