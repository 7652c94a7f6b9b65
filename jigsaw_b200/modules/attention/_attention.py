"""Multi-head attention: the serial ``Attention`` and the head- and sequence-parallel
``DistributedAttention``.

Input ``x``: ``(batch, [extra axes, e.g. windows], seq / spatial, in_dim / channel)``.  Heads
are split over ``channel_group`` (the ``qkv`` and ``head_concat`` projections are
``DistributedLinear`` with ``model_group = channel_group``; plain ``nn.Linear`` when the
channel group has one rank); the sequence is split over ``spatial_group`` and mixed by ring
attention, Ulysses, hierarchical Ulysses, or not at all (window attention on local tiles,
optional additive mask).  No causal masking.

Parameter layout: ``qkv.weight`` rows are grouped per head shard as ``[C, 3, heads / C, d]``
so that output block ``j`` of the sharded projection is (q, k, v) of head shard ``j``;
``convert_to_torch`` restores the ``[3, heads, d]`` order.  Every parameter is replicated
over ``spatial_group`` (q/k norms also over ``channel_group``), marked and broadcast.

Reference parity: jigsaw/modules/attention/_attention.py:159-179 (core dtype), :198-1045
(DistributedAttention), :1048-1405 (Attention and its converter).
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ... import parallel
from ..._core.placement import gather_dim
from ..._core.shard_repr import shard_repr
from ..linear import DistributedLinear
from ._config import AttnBackend, Offload, RingAttentionConfig, SaveBackward, SaveScope, SendForward, coerce_enum, resolve_backend
from ._cores import MathCore
from ._ring import hybrid_subgroups, ring_attention
from ._ulysses import heads_to_seq, hierarchical_ulysses_attention, seq_to_heads


def attn_core_dtype(x: torch.Tensor) -> torch.dtype:
    """dtype the attention core runs in: the autocast dtype when active, bf16 for fp32 inputs
    on CUDA (the fused kernels are half-precision only), else the input dtype."""
    if torch.is_autocast_enabled(x.device.type):
        return torch.get_autocast_dtype(x.device.type)
    if x.is_cuda and x.dtype == torch.float32:
        return torch.bfloat16
    return x.dtype


def _dense_attention(q, k, v, scale: float, dropout_p: float, backend: AttnBackend, attn_mask=None, training=True):
    """``(..., h, s, d)`` attention on local data."""
    p = dropout_p if training else 0.0
    if backend is AttnBackend.MATH:
        if attn_mask is None:
            return MathCore.forward(q, k, v, scale, 0.0, 0)[0] if p == 0.0 and not torch.is_grad_enabled() else \
                _math_autograd(q, k, v, scale, p, None)
        return _math_autograd(q, k, v, scale, p, attn_mask)
    if attn_mask is None and q.is_cuda:
        from ...ops import _lib, attention_fused

        if not _lib._any_batched((q, k, v)) and attention_fused.flash_usable(q, k, p) and v.dtype == torch.bfloat16:
            return attention_fused.FlashAttention.apply(q, k, v, scale)       # own tcgen05 kernels
    return F.scaled_dot_product_attention(q, k, v, attn_mask=attn_mask, dropout_p=p, scale=scale)


def _math_autograd(q, k, v, scale, p, mask):
    acc = torch.promote_types(q.dtype, torch.float32)
    s = torch.matmul(q.to(acc), k.to(acc).transpose(-1, -2)) * scale
    if mask is not None:
        s = s + mask.to(acc) if mask.dtype != torch.bool else s.masked_fill(~mask, float("-inf"))
    a = torch.softmax(s, dim=-1)
    if p > 0.0:
        a = F.dropout(a, p)
    return torch.matmul(a, v.to(acc)).to(q.dtype)


def _split_heads(qkv: torch.Tensor, heads: int, bshd: bool) -> torch.Tensor:
    """``(..., s, 3 * h * d)`` -> ``(3, ..., s, h, d)`` (bshd) or ``(3, ..., h, s, d)``."""
    *lead, s, f = qkv.shape
    d = f // (3 * heads)
    t = qkv.reshape(*lead, s, 3, heads, d)
    t = t.movedim(-3, 0)                       # (3, ..., s, h, d)
    return t if bshd else t.transpose(-3, -2)


class Attention(torch.nn.Module):
    """Serial multi-head attention (bias-free fused qkv projection, output projection)."""

    def __init__(
        self, in_dim: int, embed_dim: int, out_dim: int, heads: int, device: torch.device | str, dropout_p: float = 0.0,
        qk_norm: bool = False, dtype: torch.dtype = torch.float32, out_bias: bool = True,
        attn_backend: AttnBackend | str = AttnBackend.SDPA,
    ) -> None:
        super().__init__()
        if embed_dim % heads:
            raise ValueError("embed_dim is not divisible by heads")
        self.in_dim, self.embed_dim, self.out_dim, self.heads = in_dim, embed_dim, out_dim, heads
        self.head_dim = embed_dim // heads
        self.device, self.dtype = torch.device(device), dtype
        self.dropout_p, self.qk_norm = dropout_p, qk_norm
        self.attn_backend = coerce_enum(AttnBackend, attn_backend, "attn_backend")
        self.attn_backend = resolve_backend(self.attn_backend)
        self.scale = self.head_dim**-0.5
        self.qkv = torch.nn.Linear(in_dim, 3 * embed_dim, bias=False, device=self.device, dtype=dtype)
        self.head_concat = torch.nn.Linear(embed_dim, out_dim, bias=out_bias, device=self.device, dtype=dtype)
        if qk_norm:
            self.q_norm = torch.nn.LayerNorm(self.head_dim, device=self.device, dtype=dtype)
            self.k_norm = torch.nn.LayerNorm(self.head_dim, device=self.device, dtype=dtype)

    def forward(self, x: torch.Tensor, attn_mask: torch.Tensor | None = None) -> torch.Tensor:
        q, k, v = _split_heads(self.qkv(x), self.heads, bshd=False).unbind(0)
        core = attn_core_dtype(x)
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k, v = q.to(core), k.to(core), v.to(core)
        if attn_mask is not None and attn_mask.dtype != torch.bool:
            attn_mask = attn_mask.to(core)
        out = _dense_attention(q, k, v, self.scale, self.dropout_p, self.attn_backend, attn_mask, self.training)
        out = out.transpose(-3, -2).reshape(*x.shape[:-1], self.embed_dim).to(x.dtype)
        return self.head_concat(out)

    def get_parameter_count(self) -> int:
        n = 3 * self.embed_dim * self.in_dim + self.embed_dim * self.out_dim
        n += self.out_dim if self.head_concat.bias is not None else 0
        return n + (4 * self.head_dim if self.qk_norm else 0)

    def extra_repr(self) -> str:
        return (
            f"in_dim={self.in_dim}, embed_dim={self.embed_dim}, out_dim={self.out_dim}, heads={self.heads}, "
            f"dropout_p={self.dropout_p}, qk_norm={self.qk_norm}"
        )

    @classmethod
    def convert_to_jigsaw(
        cls, attention: "Attention", process_mesh_dict: dict, device: torch.device | str, row_kw: str = "row",
        col_kw: str = "col", model_kw: str = "model", ring: bool = True, ulysses: bool = False,
        ulysses_intra_size: int = 0, ulysses_inter_save_scope: SaveScope | str = SaveScope.LOCAL,
        ulysses_inter_overlap: bool = False, ulysses_inter_offload: Offload | str = Offload.DISABLED,
        attn_backend: AttnBackend | str = AttnBackend.SDPA, config: RingAttentionConfig | None = None, **kwargs: Any,
    ) -> "DistributedAttention":
        """Shard a serial ``Attention``: regroup the qkv rows per head shard, slice the input
        columns of both projections, broadcast over the spatial group."""
        channel, spatial = process_mesh_dict[col_kw], process_mesh_dict[row_kw]
        C, c = channel.size(), channel.rank()
        if attention.heads % C:
            raise ValueError(f"num_heads={attention.heads} not divisible by channel size {C}")
        layer = DistributedAttention(
            attention.in_dim, attention.embed_dim, attention.out_dim, attention.heads, c, device, spatial, channel,
            dropout_p=attention.dropout_p, qk_norm=attention.qk_norm, ring=ring, ulysses=ulysses,
            ulysses_intra_size=ulysses_intra_size, ulysses_inter_save_scope=ulysses_inter_save_scope,
            ulysses_inter_overlap=ulysses_inter_overlap, ulysses_inter_offload=ulysses_inter_offload,
            attn_backend=attn_backend, dtype=attention.qkv.weight.dtype, config=config,        # the weights' dtype: the module may have been cast after it was built
            out_bias=attention.head_concat.bias is not None,
        )
        with torch.no_grad():
            w = attention.qkv.weight.data.view(3, attention.heads, attention.head_dim, attention.in_dim)
            w = w.view(3, C, attention.heads // C, attention.head_dim, attention.in_dim).transpose(0, 1)
            w = w.reshape(3 * attention.embed_dim, attention.in_dim)
            cin = attention.in_dim // C
            layer.qkv.weight.data.copy_(w[:, c * cin : (c + 1) * cin] if C > 1 else w)
            ce = attention.embed_dim // C
            hw = attention.head_concat.weight.data
            layer.head_concat.weight.data.copy_(hw[:, c * ce : (c + 1) * ce] if C > 1 else hw)
            if attention.head_concat.bias is not None:
                co = attention.out_dim // C
                layer.head_concat.bias.data.copy_(attention.head_concat.bias.data[c * co : (c + 1) * co])
            if attention.qk_norm:
                layer.q_norm.load_state_dict(attention.q_norm.state_dict())
                layer.k_norm.load_state_dict(attention.k_norm.state_dict())
            if spatial.size() > 1:
                for p in layer.parameters():
                    dist.broadcast(p.data, group_src=0, group=spatial)
        return layer


class DistributedAttention(torch.nn.Module):
    def __init__(
        self, in_dim: int, embed_dim: int, out_dim: int, heads: int, local_rank: int | None, device: torch.device | str,
        spatial_group: dist.ProcessGroup, channel_group: dist.ProcessGroup, dropout_p: float = 0.0, qk_norm: bool = False,
        ring: bool = False, ulysses: bool = False, ulysses_intra_size: int = 0,
        ulysses_inter_save_scope: SaveScope | str = SaveScope.LOCAL, ulysses_inter_overlap: bool = False,
        ulysses_inter_offload: Offload | str = Offload.DISABLED, attn_backend: AttnBackend | str = AttnBackend.SDPA,
        dtype: torch.dtype = torch.float32, config: RingAttentionConfig | None = None, out_bias: bool = True,
    ) -> None:
        super().__init__()
        self.local_rank, self.device = local_rank, torch.device(device)
        self.spatial_group, self.channel_group = spatial_group, channel_group
        self.in_dim, self.embed_dim, self.out_dim = in_dim, embed_dim, out_dim
        self.qk_norm, self.dtype, self.dropout_p = qk_norm, dtype, dropout_p
        self.ring, self.ulysses = ring, ulysses
        self.ulysses_intra_size = ulysses_intra_size if ulysses else 0
        self.ulysses_inter_save_scope = coerce_enum(SaveScope, ulysses_inter_save_scope, "ulysses_inter_save_scope")
        self.ulysses_inter_overlap = bool(ulysses_inter_overlap)
        self.ulysses_inter_offload = coerce_enum(Offload, ulysses_inter_offload, "ulysses_inter_offload")
        if self.ulysses_inter_overlap and self.ulysses_intra_size and self.ulysses_inter_save_scope is SaveScope.GLOBAL:
            import warnings

            warnings.warn(
                "ulysses_inter_overlap with ulysses_inter_save_scope=GLOBAL only overlaps the forward pass of the outer "
                "K/V ring: GLOBAL keeps every chunk that arrived, so the backward pass fetches nothing that an overlap "
                "could hide.  Use ulysses_inter_save_scope=LOCAL to overlap the backward pass as well.", stacklevel=2)
        if ring and ulysses:
            raise ValueError("ring and ulysses are mutually exclusive")
        self.attn_backend = coerce_enum(AttnBackend, attn_backend, "attn_backend")
        self.attn_backend = resolve_backend(self.attn_backend)
        C, P = channel_group.size(), spatial_group.size()
        if heads % C:
            raise ValueError("heads is not divisible by channel group size")
        if embed_dim % heads:
            raise ValueError("embed_dim is not divisible by heads")
        self.heads = heads // C
        self.head_dim = embed_dim // heads
        self.scale = self.head_dim**-0.5
        self.config = self._ring_config(config)
        if ring and P == 1:
            raise ValueError("Cannot perform ring attention if spatial size is 1.")
        if ulysses:
            if P == 1:
                raise ValueError("Cannot perform ulysses attention if spatial size is 1.")
            a = self.ulysses_intra_size
            if a:
                if P % a or P // a < 2:
                    raise ValueError(
                        f"hierarchical ulysses needs spatial ({P}) to split into all-to-all intra groups of {a} "
                        "and an outer ring of >= 2; use ulysses_intra_size=0 for the flat scheme"
                    )
                if self.heads % a:
                    raise ValueError(
                        f"hierarchical ulysses scatters heads over the intra group: heads // channel ({self.heads}) "
                        f"must be divisible by ulysses_intra_size ({a})"
                    )
                self._intra, self._inter = hybrid_subgroups(spatial_group, a)
                self._inter_cfg = RingAttentionConfig(
                    device=self.device, send_in_forward=SendForward.KV, save_for_backward=SaveBackward.KV,
                    save_scope=self.ulysses_inter_save_scope, attn_backend=self.attn_backend,
                    overlap_comm=self.ulysses_inter_overlap, offload=self.ulysses_inter_offload,
                )
            elif self.heads % P:
                raise ValueError(
                    f"ulysses attention needs heads // channel ({self.heads}) divisible by spatial group size ({P})"
                )
        if C == 1:
            self.qkv = torch.nn.Linear(in_dim, 3 * embed_dim, bias=False, device=self.device, dtype=dtype)
            self.head_concat = torch.nn.Linear(embed_dim, out_dim, bias=out_bias, device=self.device, dtype=dtype)
        else:
            self.qkv = DistributedLinear(in_dim, 3 * embed_dim, self.device, channel_group, spatial_group, channel_group,
                                         bias=False, dtype=dtype)
            self.head_concat = DistributedLinear(embed_dim, out_dim, self.device, channel_group, spatial_group,
                                                 channel_group, bias=out_bias, dtype=dtype)
        if qk_norm:
            self.q_norm = torch.nn.LayerNorm(self.head_dim, device=self.device, dtype=dtype)
            self.k_norm = torch.nn.LayerNorm(self.head_dim, device=self.device, dtype=dtype)
            both = [g for g in (spatial_group, channel_group) if g.size() > 1]
            for norm in (self.q_norm, self.k_norm):
                for p in norm.parameters():
                    parallel.mark_replicated(p, both)
        for p in self.parameters():
            if not parallel.replica_groups(p):
                parallel.mark_replicated(p, spatial_group)
        parallel.broadcast_replicas(self)

    def _ring_config(self, config: RingAttentionConfig | None) -> RingAttentionConfig | None:
        if not self.ring:
            return config
        needs_kv = self.channel_group.size() > 1 or self.qk_norm
        if config is None:
            kw: dict = dict(device=self.device, attn_backend=self.attn_backend)
            if needs_kv:
                kw.update(send_in_forward=SendForward.KV, save_for_backward=SaveBackward.KV)
            return RingAttentionConfig(**kw)
        if needs_kv and (config.send_in_forward is not SendForward.KV or config.save_for_backward is not SaveBackward.KV):
            raise ValueError(
                "ring attention with channel/tensor parallelism or qk_norm "
                f"(channel_group.size()={self.channel_group.size()}, qk_norm={self.qk_norm}) needs "
                "send_in_forward=KV and save_for_backward=KV: the qkv projection is sharded across the channel "
                "group and/or the normalized keys only exist after the local projection, so the ring cannot "
                f"recompute K/V from a circulated x chunk. Got send_in_forward={config.send_in_forward.name}, "
                f"save_for_backward={config.save_for_backward.name}."
            )
        return config

    # ------------------------------------------------------------------ forward
    def forward(self, x: torch.Tensor, attn_mask: torch.Tensor | None = None) -> torch.Tensor:
        routed = parallel.synced_parameters(self)
        if routed:
            return torch.func.functional_call(self, routed, (x,), {"attn_mask": attn_mask})
        if attn_mask is not None and (self.ring or self.ulysses):
            kind = "ring" if self.ring else "ulysses"
            raise ValueError(f"{kind} attention does not support attn_mask: a mask over the whole sequence cannot be "
                             "applied to one chunk at a time; use ring=False, ulysses=False for masked (window) attention")
        core = attn_core_dtype(x)
        p = self.dropout_p if self.training else 0.0
        if self.ulysses and not self.ulysses_intra_size and not self.qk_norm and x.is_cuda and type(self.qkv) is torch.nn.Linear:
            from ...ops import ulysses_fused

            # projection with the sequence -> head exchange inside its epilogue: (3, b, s, h / P, d)
            full = ulysses_fused.maybe_fused_ulysses_qkv(x, self.qkv.weight, self.spatial_group, self.heads, self.head_dim)
            if full is not None:
                return self._ulysses_core(full.to(core), x, p)
        qkv = _split_heads(self.qkv(x), self.heads, bshd=self.ulysses)
        if self.qk_norm:
            q, k, v = qkv.unbind(0)
            q, k, v = self.q_norm(q).to(core), self.k_norm(k).to(core), v.to(core)
            qkv = torch.stack((q, k, v))
        else:
            qkv = qkv.to(core)
        if self.ring:
            q, k, v = qkv.unbind(0)             # head-transposed views; the ring makes the copies it needs
            send_x = self.config.send_in_forward is SendForward.X and isinstance(self.qkv, torch.nn.Linear)
            out = ring_attention(
                q, k, v, self.scale, self.spatial_group, self.config, p,
                x=x.to(core) if send_x else None, w_qkv=self.qkv.weight if send_x else None,
            ).transpose(-3, -2)
        elif self.ulysses and self.ulysses_intra_size:
            out = hierarchical_ulysses_attention(qkv, self._intra, self._inter, self.scale, self._inter_cfg, p)
        elif self.ulysses:
            return self._ulysses_core(seq_to_heads(qkv, self.spatial_group), x, p)
        else:
            q, k, v = qkv.unbind(0)
            if attn_mask is not None and attn_mask.dtype != torch.bool:
                attn_mask = attn_mask.to(core)
            out = _dense_attention(q, k, v, self.scale, p, self.attn_backend, attn_mask, True).transpose(-3, -2)
        out = out.reshape(*x.shape[:-1], self.heads * self.head_dim).to(x.dtype)
        return self.head_concat(out)

    def _ulysses_core(self, full: torch.Tensor, x: torch.Tensor, p: float) -> torch.Tensor:
        """Dense attention on the head shard ``full`` ``(3, ..., s, h / P, d)``, the head -> sequence
        exchange and the output projection (one GEMM whose operand loads do the exchange, when that applies)."""
        q, k, v = (t.transpose(-3, -2) for t in full.unbind(0))
        out = _dense_attention(q, k, v, self.scale, p, self.attn_backend, None, True).transpose(-3, -2)
        if out.is_cuda and type(self.head_concat) is torch.nn.Linear:
            from ...ops import ulysses_fused

            y = ulysses_fused.maybe_fused_ulysses_out(out, self.head_concat.weight, self.head_concat.bias, self.spatial_group)
            if y is not None:
                return y
        out = heads_to_seq(out.contiguous(), self.spatial_group)
        out = out.reshape(*x.shape[:-1], self.heads * self.head_dim).to(x.dtype)
        return self.head_concat(out)

    # ------------------------------------------------------------------ conversion
    def convert_to_torch(self, process_mesh_dict: dict, row_kw: str = "row", col_kw: str = "col", model_kw: str = "model") -> Attention:
        """Merge the shards into a serial ``Attention`` (collective over the channel group)."""
        channel = process_mesh_dict[col_kw]
        C = channel.size()
        heads = self.heads * C
        out = Attention(self.in_dim, self.embed_dim, self.out_dim, heads, self.device, self.dropout_p, self.qk_norm,
                        self.qkv.weight.dtype, self.head_concat.bias is not None)
        with torch.no_grad():
            w = gather_dim(self.qkv.weight.data, channel, 1) if C > 1 else self.qkv.weight.data
            w = w.view(C, 3, self.heads, self.head_dim, self.in_dim).transpose(0, 1).reshape(3 * self.embed_dim, self.in_dim)
            out.qkv.weight.data.copy_(w)
            hw = gather_dim(self.head_concat.weight.data, channel, 1) if C > 1 else self.head_concat.weight.data
            out.head_concat.weight.data.copy_(hw)
            if self.head_concat.bias is not None:
                hb = gather_dim(self.head_concat.bias.data, channel, 0) if C > 1 else self.head_concat.bias.data
                out.head_concat.bias.data.copy_(hb)
            if self.qk_norm:
                out.q_norm.load_state_dict(self.q_norm.state_dict())
                out.k_norm.load_state_dict(self.k_norm.state_dict())
        return out

    def reshard_parameters(self, from_process_mesh_dict: dict, to_process_mesh_dict: dict, row_kw: str = "row",
                           col_kw: str = "col", model_kw: str = "model") -> None:
        """Move this layer from one mesh to another (collective on both meshes).  The weights travel through
        the serial layout, because the row order of the qkv projection depends on the channel split; the
        layer then adopts the state of a layer built for the new mesh, so heads per rank, groups and the
        sequence-parallel scheme all follow.  On a mesh whose spatial group has one rank the layer runs
        dense attention and returns to ring / Ulysses when a later mesh splits the sequence again.  If the
        new mesh does not divide the layer, the error comes before anything is changed.

        Reference parity: none (the reference reshards attention through ``convert_to_torch`` and
        ``convert_to_jigsaw`` by hand, examples/reshard.py:78-107)."""
        want_ring, want_ulysses, ring_cfg = getattr(self, "_requested_sequence_parallel", (self.ring, self.ulysses, self.config))
        serial = self.convert_to_torch(from_process_mesh_dict, row_kw, col_kw, model_kw)
        split = to_process_mesh_dict[row_kw].size() > 1
        new = Attention.convert_to_jigsaw(
            serial, to_process_mesh_dict, self.device, row_kw, col_kw, model_kw, ring=want_ring and split,
            ulysses=want_ulysses and split, ulysses_intra_size=self.ulysses_intra_size if split else 0,
            ulysses_inter_save_scope=self.ulysses_inter_save_scope, ulysses_inter_overlap=self.ulysses_inter_overlap,
            ulysses_inter_offload=self.ulysses_inter_offload, attn_backend=self.attn_backend,
            config=ring_cfg if want_ring and split else None,
        )
        new.train(self.training)
        new._requested_sequence_parallel = (want_ring, want_ulysses, ring_cfg)
        self.__dict__ = new.__dict__

    def row_order_tags(self) -> dict[str, str]:
        """The qkv rows are stored channel-rank-major (``C, 3, heads / C, head_dim``), which
        depends on the channel split; a checkpoint records the split so that another mesh can
        reorder the rows (:meth:`reorder_rows`)."""
        return {"qkv.weight": f"qkv:{self.channel_group.size()}:{self.heads * self.channel_group.size()}:{self.head_dim}"}

    @staticmethod
    def reorder_rows(tensor: torch.Tensor, from_tag: str, to_tag: str) -> torch.Tensor:
        """Global qkv weight written under one channel split, reordered for another."""
        _, c_from, heads, hd = from_tag.split(":")
        _, c_to, heads_to, hd_to = to_tag.split(":")
        if (heads, hd) != (heads_to, hd_to):
            raise ValueError(f"attention shapes differ: {from_tag} vs {to_tag}")
        c_from, c_to, heads, hd = int(c_from), int(c_to), int(heads), int(hd)
        rest = tensor.shape[1:]
        t = tensor.view(c_from, 3, heads // c_from, hd, *rest).transpose(0, 1).reshape(3, heads, hd, *rest)
        t = t.view(3, c_to, heads // c_to, hd, *rest).transpose(0, 1)
        return t.reshape(3 * heads * hd, *rest).contiguous()

    def get_parameter_count(self) -> int:
        """Parameters this module answers for: the q/k norms, and the projections where they are plain
        ``torch.nn.Linear`` (channel group of one rank); distributed projections report their own."""
        plain = sum(p.numel() for proj in (self.qkv, self.head_concat) if isinstance(proj, torch.nn.Linear)
                    for p in proj.parameters())
        return plain + (4 * self.head_dim if self.qk_norm else 0)

    def extra_repr(self) -> str:
        return (
            f"in_dim={self.in_dim}, embed_dim={self.embed_dim}, out_dim={self.out_dim}, "
            f"heads={self.heads * self.channel_group.size()}, dropout_p={self.dropout_p}, qk_norm={self.qk_norm}, "
            f"ring={self.ring}, " + ("ulysses=True, " if self.ulysses else "")
            + shard_repr(spatial=self.spatial_group, channel=self.channel_group)
        )
