"""Fused halo-exchange convolution chains on the sm_100a kernels.

A *chain* is a sequence of 3x3 / stride 1 / padding 1 convolutions, each optionally followed
by GELU, whose channel counts fit the kernels: a thin first layer (<= 4 input channels to 64),
any number of 64 -> 64 layers, and optionally a thin last layer (64 to <= 4 channels).  A single
layer is a chain of length one.  The whole chain runs in bf16 with fp32 accumulation (the
numerics of ``torch.autocast(dtype=bfloat16)``), fp32 master weights and fp32 weight
gradients.

Forward.  The input is packed once into a padded NHWC buffer; every layer's epilogue writes
the next layer's padded input (bias + GELU fused) and stores its edge pixels directly into
the neighbouring ranks' buffers, so no halo exchange, padded copy, activation kernel or
layout change runs between the layers.  Backward.  The data-gradient kernel of layer ``i``
multiplies by GELU'(pre-activation of layer ``i - 1``) in its epilogue and writes the padded
gradient (with halo push) that both the weight-gradient kernel of layer ``i - 1`` and the next
data-gradient kernel consume; the halo scatter-add of the reference disappears because the
gradient halo is read instead.  The weight-gradient kernel also yields the bias gradient.

Reference parity: jigsaw/modules/convolution/_conv/distributed.py:212-396 (forward and
backward with halo exchange), _conv/functional.py:28-169 (autograd Function).
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch

from . import _lib, symm


def _p(t: torch.Tensor | None) -> ctypes.c_void_p | None:
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _bp(b: "symm.Block | None") -> ctypes.c_void_p | None:
    return None if b is None else ctypes.c_void_p(b.ptr)


def _check(rc: int, what: str) -> None:
    _lib.count_launches(2 if what == "wgrad" else 1)
    if rc != 0:
        raise RuntimeError(f"jigsaw_b200 kernel launch failed ({what}): code {rc}")


class Geometry:
    """Local tile shape plus the neighbourhood it exchanges halos with."""

    def __init__(self, NB: int, H: int, W: int, device: torch.device, group_h: Any, group_w: Any) -> None:
        self.NB, self.H, self.W = NB, H, W
        self.device = device
        self.arena = symm.arena(device)
        self.nbrs = symm.neighbour_table(group_h, group_w)
        self.sm = _lib.sm_count(device.index if device.index is not None else torch.cuda.current_device())

    def padded(self, channels: int, live: int | None = None) -> "symm.Block":
        """A padded buffer.  ``live`` (< channels) asks for one whose channels beyond ``live`` are
        and stay zero: such buffers are only ever recycled among themselves."""
        n = self.NB * (self.H + 2) * (self.W + 2) * channels * 2
        return self.arena.alloc(n, tag=("padded", self.NB, self.H, self.W, channels, live))

    def padded4(self) -> "symm.Block":
        """A padded buffer with four channels per pixel (thin first / last layers)."""
        n = self.NB * (self.H + 2) * (self.W + 2) * 4 * 2
        return self.arena.alloc(n, tag=("padded4", self.NB, self.H, self.W))

    def halo(self, produce: "symm.Block | None", consume: "symm.Block | None") -> Any:
        return symm.make_halo(self.arena, self.nbrs, produce, consume)


def chain_kinds(channels: list[tuple[int, int]]) -> list[str] | None:
    """Classify the layers of a chain or return ``None`` if the kernels do not cover it."""
    kinds = []
    for i, (cin, cout) in enumerate(channels):
        if cin == 64 and cout == 64:
            kinds.append("mid")
        elif cin <= 4 and cout == 64 and i == 0:
            kinds.append("thin_in")
        elif cin == 64 and cout <= 4 and i == len(channels) - 1:
            kinds.append("thin_out")
        else:
            return None
    return kinds


def _prep_weights(kind: str, w: torch.Tensor, b: torch.Tensor | None, thin: bool = False) -> dict:
    """Kernel-side weight layouts of one layer (small tensors, rebuilt every step).

    ``thin``: the layer's few channels live in a four-channel padded buffer and the thin-channel kernels run
    (one [64][64] weight tile whose column ``tap * 4 + c`` holds channel ``c`` of the thin side).  Otherwise thin
    layers run on the 64-channel kernels with their missing channels zero-filled (odd tile widths, which the
    16-byte granularity of the four-channel rows does not cover).
    """
    dev = w.device
    cout, cin = w.shape[0], w.shape[1]
    out: dict = {}
    if thin and kind == "thin_in":
        t = torch.zeros(64, 9, 4, device=dev, dtype=torch.bfloat16)
        t[:, :, :cin] = w.detach().permute(0, 2, 3, 1).reshape(64, 9, cin).to(torch.bfloat16)      # [co][tap][ci]
        out["w"] = t.view(64, 36).contiguous()
        out["w"] = torch.nn.functional.pad(out["w"], (0, 28))                                     # [64][64]
        out["b"] = None if b is None else b.detach().float().contiguous()
        return out
    wt = w.detach().permute(2, 3, 0, 1).to(torch.bfloat16)                                  # [3,3,co,ci]
    if kind == "mid":
        out["w"] = wt.contiguous()
        out["b"] = None if b is None else b.detach().float().contiguous()
    elif kind == "thin_in":
        t = torch.zeros(3, 3, 64, 64, device=dev, dtype=torch.bfloat16)
        t[:, :, :, :cin] = wt
        out["w"] = t
        out["b"] = None if b is None else b.detach().float().contiguous()
    else:  # thin_out
        t = torch.zeros(3, 3, 16, 64, device=dev, dtype=torch.bfloat16)
        t[:, :, :cout] = wt
        out["w"] = t                                                                        # forward: 16 output columns
        bb = torch.zeros(16, device=dev, dtype=torch.float32)
        if b is not None:
            bb[:cout] = b.detach().float()
        out["b"] = bb
        if thin:
            # data gradient on the thin-input kernel: row = input channel, column = mirrored tap * 4 + output channel
            t = torch.zeros(64, 9, 4, device=dev, dtype=torch.bfloat16)
            t[:, :, :cout] = w.detach().flip(2, 3).permute(1, 2, 3, 0).reshape(64, 9, cout).to(torch.bfloat16)
            out["w_dgrad"] = torch.nn.functional.pad(t.view(64, 36), (0, 28)).contiguous()
        else:
            d = torch.zeros(3, 3, 64, 64, device=dev, dtype=torch.bfloat16)
            d[:, :, :cout] = wt
            out["w_dgrad"] = d                                                              # backward: 64 (zero-filled) gradient channels
    return out


class _BlockHolder:
    """Returns the saved padded buffers to the arena after backward, or when the autograd
    graph that owns them is dropped without a backward pass."""

    def __init__(self, ar: "symm.PeerArena", blocks: list) -> None:
        self.ar, self.blocks = ar, list(blocks)

    def release(self) -> None:
        for b in self.blocks:
            self.ar.free(b)
        self.blocks = []

    def __del__(self) -> None:
        self.release()


class _ConvChain(torch.autograd.Function):
    @staticmethod
    def forward(ctx: Any, x: torch.Tensor, geom: Geometry, kinds: tuple, acts: tuple, reduce_ranks: tuple | None,
                *params: torch.Tensor | None) -> torch.Tensor:
        L = _lib.lib()
        ar, st = geom.arena, _lib.stream_ptr()
        NB, H, W = geom.NB, geom.H, geom.W
        n = len(kinds)
        weights = [params[2 * i] for i in range(n)]
        biases = [params[2 * i + 1] for i in range(n)]
        need_grad = any(ctx.needs_input_grad)      # grad mode itself is always off inside forward
        if acts[-1]:
            raise ValueError("the last layer of a fused chain must not have an activation")
        if x.dtype not in (torch.float32, torch.bfloat16):
            x = x.float()
        thin = W % 2 == 0          # the four-channel rows are read in 16-byte units (pixel pairs)
        prep = [_prep_weights(kinds[i], weights[i], biases[i], thin) for i in range(n)]
        cin0 = weights[0].shape[1]
        thin_first = thin and kinds[0] == "thin_in"
        # ---- pack the input into the padded layout (+ halo push)
        sn, sc, sh, sw = x.stride()
        if thin_first:
            a = geom.padded4()
            _check(L.jb_halo_pack(_p(x), int(x.dtype == torch.float32), sn, sc, sh, sw, NB, cin0, H, W, 4, 4, _bp(a),
                                  geom.halo(a, None), _p(ar.done_counter), st), "halo_pack")
        else:
            cw0 = min(64, (cin0 + 3) // 4 * 4)
            a = geom.padded(64, None if cw0 == 64 else cw0)
            _check(L.jb_halo_pack(_p(x), int(x.dtype == torch.float32), sn, sc, sh, sw, NB, cin0, H, W, 64, cw0, _bp(a),
                                  geom.halo(a, None), _p(ar.done_counter), st), "halo_pack")
        acts_in: list[symm.Block] = [a]
        pres: list[torch.Tensor | None] = []
        out = None
        for i in range(n):
            last = i == n - 1
            cout = weights[i].shape[0]
            nxt = None if last else geom.padded(64)
            pre = None
            if need_grad and not last and acts[i]:
                pre = torch.empty(NB, H, W, 64, device=x.device, dtype=torch.bfloat16)
            if last:
                out = torch.empty(NB, H, W, cout, device=x.device, dtype=torch.bfloat16)
            halo = geom.halo(nxt, acts_in[i])
            act = 1 if acts[i] else 0
            nout = 16 if kinds[i] == "thin_out" else 64
            if i == 0 and thin_first:
                _check(L.jb_conv3x3_thin_in(_bp(acts_in[0]), _p(prep[0]["w"]), _p(prep[0]["b"]), None, _p(pre), _bp(nxt),
                                            _p(out) if last else None, NB, H, W, act, halo, _p(ar.done_counter),
                                            _p(ar.status), geom.sm, st), "conv3x3_thin_in")
            else:
                _check(L.jb_conv3x3_c64(_bp(acts_in[i]), _p(prep[i]["w"]), _p(prep[i]["b"]), None, _p(pre), _bp(nxt),
                                        _p(out) if last else None, NB, H, W, nout, cout, act, 0, halo,
                                        _p(ar.done_counter), _p(ar.status), geom.sm, st), "conv3x3_c64")
            pres.append(pre)
            if nxt is not None:
                acts_in.append(nxt)
        if need_grad:
            ctx.geom, ctx.kinds, ctx.acts, ctx.prep = geom, kinds, acts, prep
            ctx.acts_in, ctx.pres = acts_in, pres
            ctx.shapes = [tuple(w.shape) for w in weights]
            ctx.has_bias = [b is not None for b in biases]
            ctx.x_needs_grad = ctx.needs_input_grad[0]
            ctx.thin = thin
            ctx.reduce_ranks = reduce_ranks
            ctx.holder = _BlockHolder(ar, acts_in)
        else:
            for blk in acts_in:
                ar.free(blk)
        return out.permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx: Any, gout: torch.Tensor) -> tuple:
        L = _lib.lib()
        geom: Geometry = ctx.geom
        ar, st = geom.arena, _lib.stream_ptr()
        NB, H, W = geom.NB, geom.H, geom.W
        kinds, acts, prep, acts_in, pres = ctx.kinds, ctx.acts, ctx.prep, ctx.acts_in, ctx.pres
        n = len(kinds)
        dev = gout.device
        grads: list[torch.Tensor | None] = [None] * (2 * n)
        cout_last = ctx.shapes[-1][0]
        thin = ctx.thin
        thin_last = thin and kinds[-1] == "thin_out"
        thin_first = thin and kinds[0] == "thin_in"
        sn, sc, sh, sw = gout.stride()
        if thin_last:
            g = geom.padded4()
            _check(L.jb_halo_pack(_p(gout), int(gout.dtype == torch.float32), sn, sc, sh, sw, NB, cout_last, H, W, 4, 4,
                                  _bp(g), geom.halo(g, None), _p(ar.done_counter), st), "halo_pack(grad)")
        else:
            cwg = min(64, (cout_last + 3) // 4 * 4)
            g = geom.padded(64, None if cwg == 64 else cwg)
            _check(L.jb_halo_pack(_p(gout), int(gout.dtype == torch.float32), sn, sc, sh, sw, NB, cout_last, H, W, 64, cwg,
                                  _bp(g), geom.halo(g, None), _p(ar.done_counter), st), "halo_pack(grad)")
        scratch = None
        scratch_thin = None
        gx = None
        # replicated weights: every layer's gradient is summed over the tile ranks on a side stream as soon
        # as its kernel has been launched, under the remaining data- and weight-gradient kernels
        reducer = None
        if ctx.reduce_ranks is not None:
            from . import reduce_fused

            reducer = reduce_fused.OverlappedReducer(dev, ctx.reduce_ranks)
        for i in range(n - 1, -1, -1):
            kind = kinds[i]
            cout, cin = ctx.shapes[i][0], ctx.shapes[i][1]
            # gradient of the layer above flows through the GELU that precedes this layer's input
            src = pres[i - 1] if i > 0 else None
            # ---- weight / bias gradient
            thin_here = (kind == "thin_out" and thin_last) or (kind == "thin_in" and thin_first and i == 0)
            if thin_here:
                # one side of the layer has at most four channels: the thin-channel kernel pairs the interior of the
                # 64-channel tensor with the shifted pixels of the four-channel one (read with its halo)
                side = 0 if kind == "thin_in" else 1
                cs = cin if side == 0 else cout
                big, small = (g, acts_in[i]) if side == 0 else (acts_in[i], g)
                gw = torch.empty((64, cs, 3, 3) if side == 0 else (cs, 64, 3, 3), device=dev, dtype=torch.float32)
                gb = torch.empty(64 if side == 0 else cs, device=dev, dtype=torch.float32)
                if scratch_thin is None:
                    scratch_thin = torch.empty(L.jb_conv3x3_wgrad_thin_scratch_floats(geom.sm), device=dev, dtype=torch.float32)
                _check(L.jb_conv3x3_wgrad_thin(_bp(big), _bp(small), _p(gw), _p(gb), _p(scratch_thin), NB, H, W, side, cs,
                                               geom.halo(None, small), _p(ar.status), geom.sm, st), "wgrad")
            else:
                gw = torch.empty(64, 64, 3, 3, device=dev, dtype=torch.float32)
                gb = torch.empty(64, device=dev, dtype=torch.float32)
                if scratch is None:
                    scratch = torch.empty(L.jb_conv3x3_wgrad_scratch_floats(geom.sm), device=dev, dtype=torch.float32)
                _check(L.jb_conv3x3_c64_wgrad(_bp(acts_in[i]), _bp(g), _p(gw), _p(gb), _p(scratch), NB, H, W,
                                              geom.halo(None, g), _p(ar.status), geom.sm, st), "wgrad")
                if kind == "thin_in":
                    gw = gw[:, :cin].contiguous()
                elif kind == "thin_out":
                    gw, gb = gw[:cout].contiguous(), gb[:cout].contiguous()
            grads[2 * i] = gw
            grads[2 * i + 1] = gb if ctx.has_bias[i] else None
            if reducer is not None:
                reducer.add([gw, gb] if ctx.has_bias[i] else [gw])
            # ---- data gradient
            if i == 0:
                if ctx.x_needs_grad and kind == "mid":
                    gx = torch.empty(NB, H, W, 64, device=dev, dtype=torch.bfloat16)
                    _check(L.jb_conv3x3_c64(_bp(g), _p(prep[i]["w"]), None, None, None, None, _p(gx), NB, H, W, 64, 64, 0,
                                            1, geom.halo(None, g), _p(ar.done_counter), _p(ar.status), geom.sm, st),
                           "dgrad(input)")
                    gx = gx.permute(0, 3, 1, 2)
                ar.free(g)
                break
            gnext = geom.padded(64)
            halo = geom.halo(gnext, g)
            gsrc = src if acts[i - 1] else None
            wd = prep[i]["w_dgrad"] if kind == "thin_out" else prep[i]["w"]
            if kind == "thin_out" and thin_last:
                _check(L.jb_conv3x3_thin_in(_bp(g), _p(wd), None, _p(gsrc), None, _bp(gnext), None, NB, H, W, 0, halo,
                                            _p(ar.done_counter), _p(ar.status), geom.sm, st), "dgrad")
            else:
                _check(L.jb_conv3x3_c64(_bp(g), _p(wd), None, _p(gsrc), None, _bp(gnext), None, NB, H, W, 64, 64,
                                        0, 1, halo, _p(ar.done_counter), _p(ar.status), geom.sm, st), "dgrad")
            ar.free(g)
            g = gnext
        ctx.holder.release()
        if reducer is not None:
            reducer.finish()
        return (gx, None, None, None, None, *grads)


@_lib.traced("jb.conv_chain")
def conv_chain(x: torch.Tensor, geom: Geometry, kinds: list[str], acts: list[bool], weights: list, biases: list,
               reduce_ranks: list[int] | None = None) -> torch.Tensor:
    """Run an eligible chain on the fused kernels.  ``x``: ``(N, C, H, W)`` local tile (any
    strides, fp32 or bf16).  Returns the output tile as a bf16 ``(N, C_out, H, W)`` tensor in
    channels-last memory.  With ``reduce_ranks`` (world ranks holding copies of the weights, see
    ``parallel.overlapped_sum_plan``) the weight and bias gradients come back already summed over those
    ranks, each layer's sum overlapped with the rest of the backward pass; the parameters must then NOT
    also go through ``sync_grad``."""
    flat: list = []
    for w, b in zip(weights, biases):
        flat += [w, b]
    return _ConvChain.apply(x, geom, tuple(kinds), tuple(acts), None if reduce_ranks is None else tuple(reduce_ranks), *flat)


_geoms: dict[tuple, Geometry] = {}


def geometry_for(x: torch.Tensor, group_h: Any, group_w: Any) -> Geometry:
    key = (x.shape[0], x.shape[2], x.shape[3], x.device.index, id(group_h), id(group_w))
    if key not in _geoms:
        _geoms[key] = Geometry(x.shape[0], x.shape[2], x.shape[3], x.device, group_h, group_w)
    return _geoms[key]


def layer_is_eligible(layer: Any, x: torch.Tensor) -> bool:
    """3x3 / stride 1 / padding 1 / dilation 1 / groups 1, unsplit channels, bf16 numerics."""
    if not (x.is_cuda and x.dim() == 4 and layer._n_spatial == 2 and not layer._transposed):
        return False
    if layer.kernel_size != (3, 3) or layer.stride != (1, 1) or layer.padding != (1, 1) or layer.dilation != (1, 1):
        return False
    if layer.groups != 1 or layer.channel_group.size() != 1:
        return False
    bf16 = x.dtype == torch.bfloat16 or (
        torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16
    )
    if not bf16 or x.shape[2] > 65535 or x.shape[0] > 65535:
        return False
    return _lib.available()


# ----------------------------------------------------------------------------- chains written as separate layers
def _run_lazy_chain(source: torch.Tensor, layers: tuple, acts: tuple) -> torch.Tensor:
    """Materialise a :class:`lazy_chain.LazyConvChain`: the layers as one fused chain.  A trailing
    activation (a chain whose last GELU feeds something other than a convolution) runs as a separate
    kernel, because the chain's last epilogue writes the dense output without one."""
    from .. import parallel

    kinds = chain_kinds([(m.in_channels, m.out_channels) for m in layers])
    geom = geometry_for(source, *layers[0].spatial_groups)
    raw = [t for m in layers for t in (m.weight, m.bias)]
    inner = list(acts[:-1]) + [False]
    ranks = parallel.overlapped_sum_plan(raw)
    if ranks is not None:
        out = conv_chain(source, geom, kinds, inner, raw[0::2], raw[1::2], reduce_ranks=ranks)
    else:
        params = list(parallel.sync_grad(*raw))
        out = conv_chain(source, geom, kinds, inner, params[0::2], params[1::2])
    return torch.nn.functional.gelu(out) if acts[-1] else out


def lazy_conv2d(layer: Any, x: torch.Tensor) -> tuple[Any, torch.Tensor]:
    """Entry point of ``DistributedConv2d.forward``.  Returns ``(result, x)``: ``result`` is a pending
    :class:`lazy_chain.LazyConvChain` that ends with ``layer`` (a new chain, or the chain ``x`` extended), or
    ``None`` when the fused kernels do not cover the layer; ``x`` is then the input to continue with (the
    computed tensor if it came in as a pending chain that ``layer`` cannot join)."""
    from .lazy_chain import LazyConvChain

    act = getattr(layer, "fused_activation", None) == "gelu"
    grad_mode = torch.is_grad_enabled()
    if isinstance(x, LazyConvChain) and x.pending:
        prev = x
        same_place = layer.spatial_groups == prev.layers[0].spatial_groups and prev.grad_mode == grad_mode
        channels = [(m.in_channels, m.out_channels) for m in prev.layers] + [(layer.in_channels, layer.out_channels)]
        if same_place and layer_is_eligible(layer, x) and chain_kinds(channels) is not None:
            shape = (x.shape[0], layer.out_channels, x.shape[2], x.shape[3])
            return prev.extended(layer, act, shape), x
        x = prev.materialize()
    elif isinstance(x, LazyConvChain):
        x = x.materialize()
    if not layer_is_eligible(layer, x):
        return None, x
    kinds = chain_kinds([(layer.in_channels, layer.out_channels)])
    if kinds is None:
        return _lib.decline(f"{layer.in_channels} -> {layer.out_channels} channels (covered: <= 4 -> 64, 64 -> 64, 64 -> <= 4)"), x
    if kinds[0] != "mid" and x.requires_grad:
        return _lib.decline("a thin first layer whose input needs a gradient"), x
    shape = (x.shape[0], layer.out_channels, x.shape[2], x.shape[3])
    return LazyConvChain(x, (layer,), (act,), shape, grad_mode, _run_lazy_chain), x


@_lib.traced("jb.fused_or_lazy_conv2d")
def fused_or_lazy_conv2d(layer: Any, x: torch.Tensor) -> tuple[Any, torch.Tensor]:
    """:func:`lazy_conv2d` with the dispatch audit (counted as ``conv2d``; raises under strict dispatch when
    the kernels do not cover the layer)."""
    result, x = lazy_conv2d(layer, x)
    _lib.record("conv2d", result is not None)
    return result, x


@_lib.traced("jb.maybe_fused_patch_embed")
@_lib.audited("patch_embed")
def maybe_fused_patch_embed(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None, patch: tuple) -> torch.Tensor | None:
    """Convolution whose kernel equals its stride (no padding, no dilation): every output pixel sees its own
    patch, so the layer is a matrix product.  The patches are gathered into rows by one strided copy (in
    bf16) and multiplied with the ``(C_out, C_in * prod(patch))`` weight on the tcgen05 GEMM (bias in its
    epilogue; differentiable through the fused linear Function).  ``x``: ``(N, C_in, *spatial)`` with every
    spatial extent a multiple of the patch; returns ``(N, C_out, *spatial / patch)`` (channels-last memory),
    or ``None`` when the GEMM does not cover the shapes.

    Reference parity: the kernel == stride fast path of jigsaw/modules/convolution/_conv/distributed.py:39-106
    (there: a cuDNN convolution without halo exchange)."""
    from . import linear_fused

    if not x.is_cuda:
        return None
    nd = len(patch)
    if x.dim() != nd + 2 or any(x.shape[2 + i] % patch[i] for i in range(nd)):
        return _lib.decline("the spatial extents must be multiples of the patch")
    bf16 = x.dtype == torch.bfloat16 or (torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16)
    if not bf16:
        return _lib.decline("needs bf16 numerics")
    N, C = x.shape[0], x.shape[1]
    grid = [x.shape[2 + i] // patch[i] for i in range(nd)]
    # (N, C, g0, p0, g1, p1, ...) -> (N, g0, g1, ..., C, p0, p1, ...)
    split: list[int] = []
    for i in range(nd):
        split += [grid[i], patch[i]]
    v = x.reshape(N, C, *split)
    order = [0] + [2 + 2 * i for i in range(nd)] + [1] + [3 + 2 * i for i in range(nd)]
    K = C
    for p_ in patch:
        K *= p_
    rows = v.permute(*order).to(torch.bfloat16).reshape(-1, K)            # one copy: gather + cast
    out = linear_fused.maybe_fused_linear(rows, w.reshape(w.shape[0], K), b)
    if out is None:
        return _lib.decline("the GEMM does not cover these sizes (C_in * prod(patch) >= 64 and multiples of 8 are needed)")
    out = out.view(N, *grid, w.shape[0])
    back = [0, nd + 1] + list(range(1, nd + 1))
    return out.permute(*back)
