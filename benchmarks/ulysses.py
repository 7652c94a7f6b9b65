"""Ulysses projections with their exchanges on P GPUs, device-timed (max over ranks).

QKV projection + sequence -> head exchange, three ways:

* ``fused``    - one tcgen05 GEMM whose epilogue stores every tile into the destination rank's inbox
                 (``jigsaw_b200.ops.ulysses_fused``), flag publish, bounded wait, layout copy;
* ``unfused``  - the same GEMM kernel into local memory, then the peer-memory all-to-all kernel;
* ``library``  - cuBLAS (``F.linear``) followed by NCCL ``all_to_all_single``.

Head -> sequence exchange + output projection (``out_*`` keys): ``fused`` is one GEMM that loads the heads
of rank ``p`` by TMA from rank ``p``'s staging block, ``unfused`` the all-to-all kernel followed by the GEMM
kernel, ``library`` NCCL followed by cuBLAS.

    torchrun --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/ulysses.py [--out result.json]

The roofline target is the slower of (FLOPs / measured cuBLAS bf16 rate) and (bytes that leave this GPU /
770 GB/s measured peer copy rate).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def timed(fn, warmup: int, reps: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096, help="tokens of the whole sequence")
    ap.add_argument("--dim", type=int, default=1024)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention._ulysses import heads_to_seq, seq_to_heads
    from jigsaw_b200.ops import linear_fused, symm, ulysses_fused

    ulysses_fused.FUSE_QKV_PROJECTION = ulysses_fused.FUSE_OUTPUT_PROJECTION = True      # measure them, whatever the defaults
    mesh = jb.make_process_mesh({"row": world, "col": 1})
    group = mesh["row"]
    P, b, h = world, args.batch, args.heads
    d = args.dim // h
    sl, hl = args.seq // P, h // P
    torch.manual_seed(0)
    x = torch.randn(b, sl, args.dim, device=dev).bfloat16()
    w = (torch.randn(3 * h * d, args.dim, device=dev) * 0.03).bfloat16()
    xb = x.view(b * sl, args.dim)

    def fused():
        return ulysses_fused.maybe_fused_ulysses_qkv(x, w, group, h, d)

    def unfused():
        y = linear_fused.gemm(xb, w)
        return seq_to_heads(y.view(b, sl, 3, h, d).permute(2, 0, 1, 3, 4), group)

    def library():
        y = F.linear(xb, w)
        send = y.view(b, sl, 3, P, hl, d).permute(3, 2, 0, 1, 4, 5).contiguous()
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        return recv.permute(1, 2, 0, 3, 4, 5).reshape(3, b, P * sl, hl, d)

    a, c = fused(), unfused()
    assert a is not None, "the fused path did not apply"
    same = torch.equal(a, c)
    err = float((a.float() - library().float()).abs().max())
    res = {"world": P, "batch": b, "seq": args.seq, "dim": args.dim, "heads": h, "fused_equals_unfused": bool(same),
           "max_abs_diff_vs_library": err}
    for name, fn in (("fused", fused), ("unfused", unfused), ("library", library)):
        res[name + "_ms"] = round(timed(fn, args.warmup, args.reps), 4)
    # ---- head -> sequence exchange + output projection
    o = torch.randn(b, hl, P * sl, d, device=dev).bfloat16().transpose(1, 2)          # (b, s, hl, d) as the core returns it
    wo = (torch.randn(args.dim, h * d, device=dev) * 0.03).bfloat16()
    bo = torch.randn(args.dim, device=dev)

    def out_fused():
        return ulysses_fused.maybe_fused_ulysses_out(o, wo, bo, group)

    def out_unfused():
        mine = heads_to_seq(o.contiguous(), group)
        return linear_fused.gemm(mine.view(b * sl, h * d), wo, bias=bo).view(b, sl, -1)

    def out_library():
        send = o.unflatten(1, (P, sl)).permute(1, 0, 2, 3, 4).contiguous()              # (P, b, sl, hl, d)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)
        mine = recv.permute(1, 2, 0, 3, 4).reshape(b * sl, h * d)
        return F.linear(mine, wo, bo.bfloat16()).view(b, sl, -1)

    ya, yc = out_fused(), out_unfused()
    assert ya is not None, "the fused output projection did not apply"
    res["out_fused_equals_unfused"] = bool(torch.equal(ya, yc))
    res["out_max_abs_diff_vs_library"] = float((ya.float() - out_library().float()).abs().max())
    for name, fn in (("out_fused", out_fused), ("out_unfused", out_unfused), ("out_library", out_library)):
        res[name + "_ms"] = round(timed(fn, args.warmup, args.reps), 4)
    symm.arena(dev).check_status(collective=True)
    flops = 2.0 * b * sl * args.dim * 3 * h * d
    sent = b * sl * 3 * h * d * 2 * (P - 1) / P
    peaks = {}
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        peaks = json.load(open(path))
    tf = float(peaks.get("bf16_tflops", 1590.0))
    target = max(flops / tf / 1e9, sent / 770e9 * 1e3)
    res.update(gemm_tflop=flops / 1e12, bytes_sent_per_gpu=sent, target_ms=round(target, 4),
               fused_of_target=round(target / res["fused_ms"], 3))
    if rank == 0:
        print(json.dumps(res))
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            json.dump(res, open(args.out, "w"))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
