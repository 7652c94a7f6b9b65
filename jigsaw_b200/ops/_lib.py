"""ctypes loader of the in-tree sm_100a kernel library.

``lib()`` returns the loaded library or raises: on a machine with a CUDA device the
kernels are the product, so a missing or stale ``libjb_kernels.so`` is an error, never a
silent fall back to PyTorch ops.  ``available()`` answers without raising, for code that
must also run on CPU-only machines.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_int, c_longlong, c_uint, c_void_p, c_float
from functools import lru_cache

import torch

from . import _build


class JbHalo(ctypes.Structure):
    """Mirror of the C ``JbHalo`` struct: peer buffers / flags of the 3x3 neighbourhood."""

    _fields_ = [
        ("push_buf", c_void_p * 9),
        ("push_flag", c_void_p * 9),
        ("wait_flag", c_void_p * 9),
        ("push_epoch", c_uint),
        ("wait_epoch", c_uint),
        ("push_enabled", c_uint),
        ("wait_enabled", c_uint),
        ("push_stride", c_uint),
        ("wait_stride", c_uint),
        ("replay", c_void_p),
    ]


class JbLnExchange(ctypes.Structure):
    """Mirror of the C ``JbLnExchange`` struct: inboxes / flags of the column ranks of a LayerNorm."""

    _fields_ = [
        ("inbox_local", c_void_p),
        ("inbox_peer", c_void_p * 8),
        ("flag_local", c_void_p),
        ("flag_peer", c_void_p * 8),
        ("epoch", c_uint),
        ("stride", c_uint),
        ("replay", c_void_p),
        ("parts", c_int),
        ("me", c_int),
    ]


class JbGather(ctypes.Structure):
    """A operand of a GEMM whose reduction dimension is split over GPUs (see ``jb_gemm_bf16_gather``)."""

    _fields_ = [("a_part", c_void_p * 8), ("flag", c_void_p * 8), ("epoch", c_uint), ("stride", c_uint),
                ("replay", c_void_p), ("parts", c_int), ("k_part", c_int), ("lda_part", c_longlong)]


class JbRoll(ctypes.Structure):
    """Arguments of the fused distributed roll (see ``csrc/roll.cu``)."""

    _fields_ = [("x", c_void_p), ("A", c_longlong), ("M", c_longlong), ("I16", c_longlong), ("H", c_int), ("W", c_int),
                ("rem_h", c_int), ("rem_w", c_int), ("out", c_void_p * 4), ("flag_out", c_void_p * 4),
                ("flag_in", c_void_p * 4), ("epoch", c_uint), ("stride", c_uint), ("replay", c_void_p)]


class JbA2a(ctypes.Structure):
    """Arguments of the fused re-sharding all-to-all (see ``csrc/alltoall.cu``)."""

    _fields_ = [("x", c_void_p), ("dim", c_longlong * 5), ("split", c_int), ("cat", c_int), ("parts", c_int), ("me", c_int),
                ("out", c_void_p * 8), ("flag_out", c_void_p * 8), ("flag_in", c_void_p * 8), ("epoch", c_uint),
                ("stride", c_uint), ("replay", c_void_p)]


class JbAllReduce(ctypes.Structure):
    """Arguments of the peer-memory all-reduce (see ``csrc/allreduce.cu``)."""

    _fields_ = [("buf", c_void_p * 8), ("notice_out", c_void_p * 8), ("notice_in", c_void_p * 8), ("epoch", c_uint),
                ("stride", c_uint), ("replay", c_void_p), ("ranks", c_int), ("me", c_int), ("n", c_longlong), ("scale", c_float)]


class JbStrided4(ctypes.Structure):
    """A tensor of up to four dimensions: base pointer, element type, element strides."""

    _fields_ = [("ptr", c_void_p), ("is_bf16", c_int), ("stride", c_longlong * 4)]


class JbAdamTensors(ctypes.Structure):
    """Parameter / gradient / moment pointers of up to 48 fp32 tensors."""

    _fields_ = [("p", c_void_p * 48), ("g", c_void_p * 48), ("m", c_void_p * 48), ("v", c_void_p * 48),
                ("numel", c_longlong * 48), ("count", c_int)]


def _declare(L: ctypes.CDLL) -> None:
    L.jb_abi_version.restype = c_int
    L.jb_gemm_bf16.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p,  # A B C bias
        c_int, c_int, c_int,  # M N K
        c_longlong, c_longlong, c_longlong,  # lda ldb ldc
        c_int, c_int, c_int, c_int, c_int,  # a_mn b_mn act out_fp32 accumulate
        c_int, c_void_p, c_void_p,  # sm_count status stream
    ]
    L.jb_gemm_bf16.restype = c_int
    L.jb_conv3x3_c64.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p,  # in weights bias gelu_src
        c_void_p, c_void_p, c_void_p,  # dense_pre padded_out dense_out
        c_int, c_int, c_int,  # NB H W
        c_int, c_int, c_int, c_int,  # nout_pad cout_real act mode
        POINTER(JbHalo), c_void_p, c_void_p, c_int, c_void_p,  # halo done_counter status sm_count stream
    ]
    L.jb_conv3x3_c64.restype = c_int
    L.jb_conv3x3_wgrad_scratch_floats.argtypes = [c_int]
    L.jb_conv3x3_wgrad_scratch_floats.restype = c_longlong
    L.jb_conv3x3_c64_wgrad.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # x gy gw gb scratch
        c_int, c_int, c_int,  # NB H W
        POINTER(JbHalo), c_void_p, c_int, c_void_p,  # halo status sm_count stream
    ]
    L.jb_conv3x3_c64_wgrad.restype = c_int
    L.jb_halo_pack.argtypes = [
        c_void_p, c_int, c_longlong, c_longlong, c_longlong, c_longlong,  # src is_fp32 strides
        c_int, c_int, c_int, c_int, c_int, c_int,  # NB C H W CP CW
        c_void_p, POINTER(JbHalo), c_void_p, c_void_p,  # dst halo done_counter stream
    ]
    L.jb_halo_pack.restype = c_int
    L.jb_conv3x3_thin_in.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # in4 w bias gelu_src pre padded dense
        c_int, c_int, c_int, c_int,  # NB H W act
        POINTER(JbHalo), c_void_p, c_void_p, c_int, c_void_p,
    ]
    L.jb_conv3x3_thin_in.restype = c_int
    L.jb_conv3x3_wgrad_thin_scratch_floats.argtypes = [c_int]
    L.jb_conv3x3_wgrad_thin_scratch_floats.restype = c_longlong
    L.jb_conv3x3_wgrad_thin.argtypes = [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # big small gw gb scratch
        c_int, c_int, c_int, c_int, c_int,  # NB H W side cs
        POINTER(JbHalo), c_void_p, c_int, c_void_p,
    ]
    L.jb_conv3x3_wgrad_thin.restype = c_int
    L.jb_gemm_bf16_gather.argtypes = [POINTER(JbGather), c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong,
                                      c_int, c_int, c_int, c_void_p, c_void_p]
    L.jb_gemm_bf16_gather.restype = c_int
    L.jb_gemm_bf16_scatter.argtypes = [c_void_p, c_void_p, POINTER(c_void_p), c_int, c_int, c_int, c_int, c_longlong, c_longlong,
                                       c_int, c_int, c_int, c_void_p, c_void_p]
    L.jb_gemm_bf16_scatter.restype = c_int
    L.jb_gemm_bf16_scatter_staged.argtypes = L.jb_gemm_bf16_scatter.argtypes
    L.jb_gemm_bf16_scatter_staged.restype = c_int
    L.jb_set_staged_epilogue.argtypes = [c_int]
    L.jb_set_staged_epilogue.restype = None
    L.jb_sum_slabs.argtypes = [c_void_p, c_longlong, c_int, POINTER(c_void_p), c_uint, c_uint, c_void_p, c_void_p, c_int,
                               c_void_p, c_int, c_void_p]
    L.jb_sum_slabs.restype = c_int
    L.jb_publish.argtypes = [POINTER(c_void_p), c_int, c_uint, c_uint, c_void_p, c_void_p]
    L.jb_publish.restype = c_int
    L.jb_all_to_all.argtypes = [POINTER(JbA2a), c_void_p, c_void_p, c_int, c_void_p]
    L.jb_all_to_all.restype = c_int
    L.jb_wait_flags.argtypes = [POINTER(c_void_p), c_int, c_uint, c_uint, c_void_p, c_void_p, c_void_p]
    L.jb_wait_flags.restype = c_int
    L.jb_softmax_apply.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    L.jb_softmax_apply.restype = c_int
    L.jb_softmax_rowdot.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
    L.jb_softmax_rowdot.restype = c_int
    L.jb_softmax_bwd.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int,
                                 c_void_p]
    L.jb_softmax_bwd.restype = c_int
    L.jb_all_reduce_sum.argtypes = [POINTER(JbAllReduce), c_void_p, c_void_p, c_int, c_void_p]
    L.jb_all_reduce_sum.restype = c_int
    L.jb_memcpy_async.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p]
    L.jb_memcpy_async.restype = c_int
    L.jb_memcpy2d_async.argtypes = [c_void_p, c_longlong, c_void_p, c_longlong, c_longlong, c_longlong, c_void_p]
    L.jb_memcpy2d_async.restype = c_int
    L.jb_slot_acquire.argtypes = [POINTER(c_void_p), c_int, c_void_p, c_uint, c_uint, c_void_p, c_void_p, c_void_p]
    L.jb_slot_acquire.restype = c_int
    L.jb_slot_release.argtypes = [POINTER(c_void_p), c_int, c_uint, c_uint, c_void_p, c_void_p]
    L.jb_slot_release.restype = c_int
    L.jb_flash_attn_fwd.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int] + [c_longlong] * 8 + [
        c_float, c_void_p, c_void_p]
    L.jb_flash_attn_fwd.restype = c_int
    L.jb_flash_attn_bwd.argtypes = [c_void_p] * 10 + [c_int, c_int, c_int, c_float, c_void_p, c_void_p]
    L.jb_flash_attn_bwd.restype = c_int
    L.jb_flash_attn_fwd_parts.argtypes = [c_void_p, POINTER(c_void_p), POINTER(c_void_p), POINTER(c_void_p), c_uint, c_uint,
                                          c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int] + [c_longlong] * 6 + [
        c_float, c_void_p, c_void_p]
    L.jb_flash_attn_fwd_parts.restype = c_int
    L.jb_flash_attn_delta.argtypes = [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p]
    L.jb_flash_attn_delta.restype = c_int
    L.jb_flash_attn_bwd_parts.argtypes = [c_void_p] * 4 + [POINTER(c_void_p)] * 7 + [c_uint, c_uint, c_void_p, c_int, c_int,
                                                                                  c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                                                  c_float, c_void_p, c_void_p]
    L.jb_flash_attn_bwd_parts.restype = c_int
    L.jb_peer_fetch.argtypes = [c_void_p, c_void_p, c_longlong, c_void_p, c_uint, c_uint, c_void_p, c_void_p, c_int, c_void_p]
    L.jb_peer_fetch.restype = c_int
    L.jb_roll.argtypes = [POINTER(JbRoll), c_void_p, c_void_p, c_int, c_void_p]
    L.jb_roll.restype = c_int
    L.jb_merge_chunks.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_longlong, c_int, c_void_p]
    L.jb_merge_chunks.restype = c_int
    L.jb_mse_grid.argtypes = [c_longlong, c_int]
    L.jb_mse_grid.restype = c_int
    L.jb_pair_loss_sum.argtypes = [POINTER(JbStrided4), POINTER(JbStrided4), POINTER(c_int), c_int, c_float, c_void_p, c_void_p,
                                   c_void_p, c_int, c_void_p]
    L.jb_pair_loss_sum.restype = c_int
    L.jb_pair_loss_grad.argtypes = [POINTER(JbStrided4), POINTER(JbStrided4), POINTER(c_int), c_int, c_float, c_void_p, c_void_p,
                                    c_int, c_int, c_void_p]
    L.jb_pair_loss_grad.restype = c_int
    L.jb_increment.argtypes = [c_void_p, c_void_p]
    L.jb_increment.restype = c_int
    L.jb_adam_multi.argtypes = [POINTER(JbAdamTensors), c_float, c_float, c_float, c_float, c_float, c_int, c_int, c_void_p,
                                c_void_p, c_void_p]
    L.jb_adam_multi.restype = c_int
    L.jb_adam_multi_lr.argtypes = [POINTER(JbAdamTensors), c_void_p, c_float, c_float, c_float, c_float, c_int, c_int, c_void_p,
                                   c_void_p, c_void_p]
    L.jb_adam_multi_lr.restype = c_int
    L.jb_sumsq_multi.argtypes = [POINTER(JbAdamTensors), c_void_p, c_void_p, c_void_p, c_void_p]
    L.jb_sumsq_multi.restype = c_int
    L.jb_chunks.argtypes = [c_longlong]
    L.jb_chunks.restype = c_int
    L.jb_cross_entropy_grid.argtypes = [c_int, c_int, c_int, c_int]
    L.jb_cross_entropy_grid.restype = c_int
    L.jb_cross_entropy_fwd.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                       POINTER(JbLnExchange), c_void_p, c_int, c_void_p]
    L.jb_cross_entropy_fwd.restype = c_int
    L.jb_cross_entropy_bwd.argtypes = [c_void_p, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                       c_void_p, c_int, c_int, c_void_p]
    L.jb_cross_entropy_bwd.restype = c_int
    L.jb_group_norm_splits.argtypes = [c_int, c_int]
    L.jb_group_norm_splits.restype = c_int
    L.jb_group_norm_fwd.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_int, c_int, c_int, c_longlong, c_float, POINTER(JbLnExchange), c_void_p, c_int, c_void_p]
    L.jb_group_norm_fwd.restype = c_int
    L.jb_group_norm_bwd.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                    c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, POINTER(JbLnExchange), c_void_p, c_int,
                                    c_void_p]
    L.jb_group_norm_bwd.restype = c_int
    L.jb_layer_norm_grid.argtypes = [c_int, c_int]
    L.jb_layer_norm_grid.restype = c_int
    L.jb_layer_norm_scratch_floats.argtypes = [c_int, c_int]
    L.jb_layer_norm_scratch_floats.restype = c_longlong
    L.jb_layer_norm_grid2.argtypes = [c_int, c_int, c_int, c_int]
    L.jb_layer_norm_grid2.restype = c_int
    L.jb_layer_norm_fwd.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,  # x x_bf16 y y_bf16 w b
        c_void_p, c_void_p, c_int, c_int, c_float,  # mean rstd R n eps
        POINTER(JbLnExchange), c_void_p, c_int, c_void_p,  # exchange status sm_count stream
    ]
    L.jb_layer_norm_fwd.restype = c_int
    L.jb_layer_norm_bwd.argtypes = [
        c_void_p, c_int, c_void_p, c_int, c_void_p, c_int,  # x g dx (+ bf16 flags)
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # w mean rstd dw db scratch
        c_int, c_int, POINTER(JbLnExchange), c_void_p, c_int, c_void_p,  # R n exchange status sm_count stream
    ]
    L.jb_layer_norm_bwd.restype = c_int


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    """Load (building first if the sources are newer) and return the kernel library."""
    override = os.environ.get("JIGSAW_B200_LIB")     # a pre-built library to load instead
    if override:
        L = ctypes.CDLL(override)
        _declare(L)
        return L
    if not _build.is_fresh():
        _build.build()
    L = ctypes.CDLL(str(_build.LIB_PATH))
    _declare(L)
    return L


def available() -> bool:
    """True when a CUDA device is present and the kernel library loads."""
    if not torch.cuda.is_available():
        return False
    try:
        lib()
    except (OSError, RuntimeError):
        return False
    return True


@lru_cache(maxsize=8)
def sm_count(device_index: int) -> int:
    return torch.cuda.get_device_properties(device_index).multi_processor_count


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


#: Number of kernels of this library launched so far in this process (benchmarks report it).
LAUNCHES = 0


def count_launches(n: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += n


# ----------------------------------------------------------------------------- audited dispatch
#: ``{operation: [calls that ran on the fused kernels, calls on CUDA tensors that were declined]}``
DISPATCH: dict[str, list[int]] = {}
_strict = os.environ.get("JIGSAW_STRICT_FUSED", "0") == "1"
_last_reason: str | None = None


class FusedPathDeclined(RuntimeError):
    """A fused operation declined CUDA inputs while strict dispatch was on."""


def set_strict(on: bool) -> bool:
    """Strict dispatch: a fused operation that declines CUDA inputs raises :class:`FusedPathDeclined`
    (with the reason) instead of handing the call to the ``torch.distributed`` path.  Benchmarks and
    GPU tests switch it on so that a number or a pass can never come from a silent library fallback;
    ``JIGSAW_STRICT_FUSED=1`` sets the initial state.  Returns the previous state."""
    global _strict
    prev, _strict = _strict, bool(on)
    return prev


class strict_fused:
    """``with strict_fused():`` - strict dispatch inside the block."""

    def __init__(self, on: bool = True) -> None:
        self.on = on

    def __enter__(self) -> None:
        self.prev = set_strict(self.on)

    def __exit__(self, *exc) -> None:
        set_strict(self.prev)


def decline(reason: str) -> None:
    """``return _lib.decline("why")`` inside a fused entry point: records why the kernels do not cover
    the call (reported by strict dispatch) and returns ``None``."""
    global _last_reason
    _last_reason = reason
    return None


def dispatch_counts(reset: bool = False) -> dict[str, dict[str, int]]:
    """``{operation: {"fused": n, "fallback": m}}`` since the start (or the last reset)."""
    out = {k: {"fused": v[0], "fallback": v[1]} for k, v in sorted(DISPATCH.items())}
    if reset:
        DISPATCH.clear()
    return out


def record(name: str, fused: bool) -> None:
    """Count one call of operation ``name`` on CUDA inputs; under strict dispatch a declined call raises."""
    rec = DISPATCH.setdefault(name, [0, 0])
    rec[0 if fused else 1] += 1
    if not fused and _strict:
        raise FusedPathDeclined(f"{name} declined CUDA inputs: {_last_reason or 'outside the coverage of the kernel'}")


def _any_batched(args: tuple) -> bool:
    """True when one of ``args`` is a tensor that ``torch.vmap`` has wrapped."""
    probe = getattr(getattr(torch._C, "_functorch", None), "is_batchedtensor", None)
    if probe is None:
        return False
    return any(isinstance(a, torch.Tensor) and probe(a) for a in args)


def audited(name: str):
    """Decorator of the ``maybe_fused_*`` entry points: counts, per operation, the calls that ran on the
    kernels and the calls with CUDA tensors that were declined, and raises on the latter under strict
    dispatch.  Calls without any CUDA tensor (the CPU / gloo path) are not counted."""

    def wrap(fn):
        import functools

        @functools.wraps(fn)
        def inner(*args, **kwargs):
            global _last_reason
            _last_reason = None
            # a pending fused convolution chain among the arguments is computed first
            if any(type(a).__name__ == "LazyConvChain" for a in args):
                from .lazy_chain import materialize

                args = tuple(materialize(a) for a in args)
            if _any_batched(args):
                # the kernels take raw pointers and have no batching rules: a call under torch.vmap goes to the
                # torch.distributed path, whose Functions carry them
                out = decline("called under torch.vmap")
            else:
                out = fn(*args, **kwargs)
            if out is not None:
                record(name, True)
                return out
            if any(isinstance(a, torch.Tensor) and a.is_cuda for a in args):
                record(name, False)
            return None

        return inner

    return wrap


def traced(name: str):
    """Decorator: an NVTX range named ``name`` around every call when ``JIGSAW_NVTX=1`` is set (for
    Nsight timelines); otherwise the function is returned unchanged and costs nothing."""
    if os.environ.get("JIGSAW_NVTX", "0") != "1":
        return lambda fn: fn

    def wrap(fn):
        import functools

        @functools.wraps(fn)
        def inner(*args, **kwargs):
            if not torch.cuda.is_available():
                return fn(*args, **kwargs)
            torch.cuda.nvtx.range_push(name)
            try:
                return fn(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()

        return inner

    return wrap
