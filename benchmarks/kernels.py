"""Per-kernel roofline report on one GPU: every own kernel on a workload larger than L2, timed with
CUDA events (warm-up, then ``--reps`` launches), as achieved GB/s or TFLOP/s and as a fraction of the
measured peaks in ``MEASURED_PEAKS.json`` (copy bandwidth, cuBLAS bf16).

    python benchmarks/kernels.py                 # all kernels
    python benchmarks/kernels.py --only layer_norm_fwd --reps 1 --warmup 1      # one kernel, e.g. under ncu

The multi-GPU variants of the same kernels (peer exchange) need several ranks and are timed by
``bench.py`` and ``benchmarks/workloads.py``.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks() -> tuple[float, float]:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"])
    return 6650.0, 1590.0            # earlier measurement on the same pool


def timed(fn, warmup: int, reps: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None)
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--small", action="store_true", help="a few hundred MB per case (profiler captures)")
    args = ap.parse_args()
    import jigsaw_b200  # noqa: F401  (package import registers the kernel library path)
    from jigsaw_b200.ops import _lib, linear_fused, loss_fused, norm_fused, symm
    from jigsaw_b200.optim import FusedAdam

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    hbm, tf = peaks()
    L = _lib.lib()
    SM = _lib.sm_count(0)
    scale = 4 if args.small else 1
    cases: dict = {}

    def case(name):
        def deco(f):
            cases[name] = f
            return f
        return deco

    def P(t):
        return None if t is None else ctypes.c_void_p(t.data_ptr())

    # ---- LayerNorm (rows x 1024, bf16 in, fp32 out as under autocast)
    R, n = 131072 // scale, 1024
    x_ln = torch.randn(R, n, device=dev).bfloat16().requires_grad_(True)
    w_ln, b_ln = torch.ones(n, device=dev, requires_grad=True), torch.zeros(n, device=dev, requires_grad=True)

    @case("layer_norm_fwd")
    def _():
        with torch.autocast("cuda", dtype=torch.bfloat16), torch.no_grad():
            f = lambda: norm_fused.maybe_fused_layer_norm(x_ln, w_ln, b_ln, None, 1e-5)
            return timed(f, args.warmup, args.reps), R * n * (2 + 4), None

    @case("layer_norm_bwd")
    def _():
        y = norm_fused.maybe_fused_layer_norm(x_ln, w_ln, b_ln, None, 1e-5)
        g = torch.randn_like(y)
        f = lambda: torch.autograd.grad(y, [x_ln, w_ln, b_ln], g, retain_graph=True)
        return timed(f, args.warmup, args.reps), R * n * (2 + 2 + 2), None

    # ---- GroupNorm (8 groups of a 32-channel volume)
    xg = torch.randn(1, 32, 128 // scale, 128, 128, device=dev).bfloat16().requires_grad_(True)
    wg, bg = torch.ones(32, device=dev, requires_grad=True), torch.zeros(32, device=dev, requires_grad=True)

    @case("group_norm_fwd")
    def _():
        with torch.no_grad():
            f = lambda: norm_fused.maybe_fused_group_norm(xg, 8, wg, bg, [], 1e-5)
            return timed(f, args.warmup, args.reps), xg.numel() * (2 + 2 + 2), None      # statistics pass re-reads x

    @case("group_norm_bwd")
    def _():
        y = norm_fused.maybe_fused_group_norm(xg, 8, wg, bg, [], 1e-5)
        g = torch.randn_like(y)
        f = lambda: torch.autograd.grad(y, [xg, wg, bg], g, retain_graph=True)
        return timed(f, args.warmup, args.reps), xg.numel() * 2 * 5, None

    # ---- cross-entropy (per-pixel, 20 classes) and squared error
    xc = torch.randn(8, 20, 1024 // scale, 1024, device=dev).bfloat16().requires_grad_(True)
    tc = torch.randint(0, 20, (8, 1024 // scale, 1024), device=dev)

    @case("cross_entropy_fwd")
    def _():
        with torch.no_grad():
            f = lambda: loss_fused.maybe_fused_cross_entropy(xc, tc, 1, None, -100)
            return timed(f, args.warmup, args.reps), xc.numel() * 2 * 2 + tc.numel() * (8 + 8), None

    @case("cross_entropy_bwd")
    def _():
        rows = loss_fused.maybe_fused_cross_entropy(xc, tc, 1, None, -100)
        g = torch.ones_like(rows)
        f = lambda: torch.autograd.grad(rows, [xc], g, retain_graph=True)
        return timed(f, args.warmup, args.reps), xc.numel() * 2 * 2 + tc.numel() * 16, None

    # the shape of the CNN benchmark's loss: a 3-channel bf16 channels-last prediction against an fp32 NCHW target
    xm = torch.randn(1, 3, 4096 // scale, 4096, device=dev).bfloat16().permute(0, 2, 3, 1).contiguous().permute(0, 3, 1, 2)
    xm.requires_grad_(True)
    ym = torch.randn(1, 3, 4096 // scale, 4096, device=dev)

    @case("mse_fwd")
    def _():
        with torch.no_grad():
            f = lambda: loss_fused.maybe_fused_sq_diff_sum(xm, ym)
            return timed(f, args.warmup, args.reps), xm.numel() * (2 + 4), None

    @case("mse_bwd")
    def _():
        s = loss_fused.maybe_fused_sq_diff_sum(xm, ym)
        f = lambda: torch.autograd.grad(s, [xm], retain_graph=True)
        return timed(f, args.warmup, args.reps), xm.numel() * (2 + 4 + 2), None

    # ---- multi-tensor Adam (40 tensors of 8 Mi floats)
    params = [torch.randn(8 * 1024 * 1024 // scale, device=dev, requires_grad=True) for _ in range(40)]
    for p in params:
        p.grad = torch.randn_like(p)
    opt = FusedAdam(params, lr=1e-3)

    @case("adam")
    def _():
        return timed(opt.step, args.warmup, args.reps), sum(p.numel() for p in params) * 4 * 7, None

    # ---- online-softmax merge
    o1 = torch.randn(8, 16, 4096 // scale, 64, device=dev)
    l1 = torch.randn(8, 16, 4096 // scale, device=dev)
    o2 = torch.randn(8, 16, 4096 // scale, 64, device=dev).bfloat16()
    l2 = torch.randn(8, 16, 4096 // scale, device=dev)

    @case("merge_chunks")
    def _():
        from jigsaw_b200.ops import attention_fused

        f = lambda: attention_fused.maybe_fused_merge(o1, l1, o2, l2)
        return timed(f, args.warmup, args.reps), o1.numel() * (4 + 4 + 2), None

    # ---- tcgen05 attention against the library kernels: PyTorch's default SDPA dispatch and the flash kernel
    #      that the reference's ring core calls directly (aten._scaled_dot_product_flash_attention)
    if True:
        qa = torch.randn(8, 16, 4096 // scale, 64, device=dev).bfloat16()
        ka, va = torch.randn_like(qa), torch.randn_like(qa)
        fa_flops = 4.0 * qa.shape[0] * qa.shape[1] * qa.shape[2] * qa.shape[2] * 64

        @case("flash_attn_fwd")
        def _():
            from jigsaw_b200.ops import attention_fused

            f = lambda: attention_fused.flash_attention_forward(qa, ka, va, 0.125)
            return timed(f, args.warmup, args.reps), None, fa_flops

        @case("flash_attn_bwd")
        def _():
            from jigsaw_b200.ops import attention_fused

            out, lse = attention_fused.flash_attention_forward(qa, ka, va, 0.125)
            go = torch.randn_like(out)
            f = lambda: attention_fused.flash_attention_backward(go, qa, ka, va, out, lse, 0.125)
            return timed(f, args.warmup, args.reps), None, 2.5 * fa_flops      # five products, two of them recomputed twice: 3.5x issued

        @case("sdpa_fwd_library")
        def _():
            with torch.no_grad():
                f = lambda: torch.nn.functional.scaled_dot_product_attention(qa, ka, va, scale=0.125)
                return timed(f, args.warmup, args.reps), None, fa_flops

        @case("aten_flash_fwd_library")
        def _():
            with torch.no_grad():
                f = lambda: torch.ops.aten._scaled_dot_product_flash_attention(qa, ka, va, 0.0, False, False, scale=0.125)
                return timed(f, args.warmup, args.reps), None, fa_flops

        @case("aten_flash_bwd_library")
        def _():
            res = torch.ops.aten._scaled_dot_product_flash_attention(qa, ka, va, 0.0, False, False, scale=0.125)
            out, lse, ps, po = res[0], res[1], res[6], res[7]
            go = torch.randn_like(out)
            S = qa.shape[2]
            f = lambda: torch.ops.aten._scaled_dot_product_flash_attention_backward(
                go, qa, ka, va, out, lse, None, None, S, S, 0.0, False, ps, po, scale=0.125)
            return timed(f, args.warmup, args.reps), None, 2.5 * fa_flops

        @case("sdpa_bwd_library")
        def _():
            ql, kl, vl = (t.clone().requires_grad_(True) for t in (qa, ka, va))
            out = torch.nn.functional.scaled_dot_product_attention(ql, kl, vl, scale=0.125)
            go = torch.randn_like(out)
            f = lambda: torch.autograd.grad(out, [ql, kl, vl], go, retain_graph=True)
            return timed(f, args.warmup, args.reps), None, 2.5 * fa_flops

    # ---- GEMM
    for (M, N, K) in ((8192, 8192, 8192), (8192, 4096, 1024), (8192, 1024, 4096)):
        if args.small and M * N * K > 2 ** 36:
            continue
        A = torch.randn(M, K, device=dev).bfloat16()
        B = torch.randn(N, K, device=dev).bfloat16()

        def g(A=A, B=B, M=M, N=N, K=K):
            return timed(lambda: linear_fused.gemm(A, B), args.warmup, args.reps), None, 2.0 * M * N * K

        cases[f"gemm_{M}x{N}x{K}"] = g

    # ---- 3x3 convolution kernels on a 64-channel tile
    NB, H, W = 1, 2048 // scale, 4096
    ar = symm.arena(dev)
    xp = torch.randn(NB, H + 2, W + 2, 64, device=dev).bfloat16()
    gp = torch.randn(NB, H + 2, W + 2, 64, device=dev).bfloat16()
    po = torch.zeros(NB, H + 2, W + 2, 64, device=dev, dtype=torch.bfloat16)
    pre = torch.zeros(NB, H, W, 64, device=dev, dtype=torch.bfloat16)
    wt = (torch.randn(9 * 64, 64, device=dev) * 0.05).bfloat16()
    bias = torch.randn(64, device=dev)
    gw, gb = torch.zeros(64, 64, 3, 3, device=dev), torch.zeros(64, device=dev)
    scratch = torch.zeros(L.jb_conv3x3_wgrad_scratch_floats(SM), device=dev)
    flop = 2.0 * 9 * 64 * 64 * NB * H * W
    st = _lib.stream_ptr

    @case("conv3x3_fwd_plain")
    def _():
        f = lambda: L.jb_conv3x3_c64(P(xp), P(wt), P(bias), None, None, P(po), None, NB, H, W, 64, 64, 0, 0, None,
                                     P(ar.done_counter), P(ar.status), SM, st())
        return timed(f, args.warmup, args.reps), None, flop

    @case("conv3x3_fwd_gelu")
    def _():
        f = lambda: L.jb_conv3x3_c64(P(xp), P(wt), P(bias), None, P(pre), P(po), None, NB, H, W, 64, 64, 1, 0, None,
                                     P(ar.done_counter), P(ar.status), SM, st())
        return timed(f, args.warmup, args.reps), None, flop

    @case("conv3x3_dgrad_gelu")
    def _():
        f = lambda: L.jb_conv3x3_c64(P(gp), P(wt), None, P(pre), None, P(po), None, NB, H, W, 64, 64, 0, 1, None,
                                     P(ar.done_counter), P(ar.status), SM, st())
        return timed(f, args.warmup, args.reps), None, flop

    @case("conv3x3_wgrad")
    def _():
        f = lambda: L.jb_conv3x3_c64_wgrad(P(xp), P(gp), P(gw), P(gb), P(scratch), NB, H, W, None, P(ar.status), SM, st())
        return timed(f, args.warmup, args.reps), None, flop

    @case("halo_pack")
    def _():
        src = torch.randn(1, 3, H, W, device=dev)
        f = lambda: L.jb_halo_pack(P(src), 1, *src.stride(), NB, 3, H, W, 64, 4, P(po), None, P(ar.done_counter), st())
        return timed(f, args.warmup, args.reps), NB * H * W * (12 + 32), None      # 8-byte stores land in 32-byte sectors

    print(f"peaks of measured: {hbm:.0f} GB/s copy, {tf:.1f} TFLOP/s cuBLAS bf16")
    for name, fn in cases.items():
        if args.only and args.only != name:
            continue
        ms, nbytes, flops = fn()
        if flops is not None:
            rate = flops / ms / 1e9
            print(f"{name:28s} {ms:8.3f} ms  {rate:8.1f} TFLOP/s  {rate / tf:5.2f} of measured")
        else:
            rate = nbytes / ms / 1e6
            print(f"{name:28s} {ms:8.3f} ms  {rate:8.0f} GB/s     {rate / hbm:5.2f} of measured")
    ar.check_status()


if __name__ == "__main__":
    main()
