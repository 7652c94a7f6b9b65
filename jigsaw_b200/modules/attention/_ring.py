"""Ring attention: every rank keeps its queries and visits all key/value chunks of the
sequence-parallel group, merging per-chunk results with the online-softmax rule.

Schedule.  ``chunk_owner(send_op, p, s)`` names the rank whose chunk position ``p`` works
on at step ``s``; every policy visits each chunk exactly once.  The transport is one
sparse exchange per step in which owners send their chunk to whoever needs it: on an
NVSwitch fabric every peer is equally near, so a chunk always comes straight from its
owner instead of being relayed hop by hop.  With ``overlap_comm`` the exchange for step
``s + 1`` is started before the core of step ``s`` runs.

Backward.  Each chunk's gradient is computed against the final (merged) output and
log-sum-exp, which makes it exact.  ``save_scope=GLOBAL`` keeps the arrived chunks
(optionally offloaded to pinned host memory), ``LOCAL`` fetches them again, so memory per
rank does not grow with the ring.  dK/dV go back to the owner every step (``SEND_DKV``) or
are accumulated per owner and reduced once at the end (``GATHER_DKV``).  When the layer
input ``x`` circulates instead of K/V (``send_in_forward=X``, only without channel
sharding and q/k norms), K/V are re-projected from the arriving chunk and the projection
weight receives its gradient share on the visiting rank.

Reference parity: jigsaw/modules/attention/_functional/ring.py:16-37 (seeds), :99-242
(hybrid topology), :264-445 (Function); forward.py:102-200; backward.py:109-312, :318-735;
forward_chunk_provider.py:30-740; backward_chunk_provider.py:25-1021; _comm_overlap.py:21-140.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from ..._core.comm import sparse_exchange
from ..._core.vmap import to_front
from ._config import Offload, RingAttentionConfig, SaveScope, SendBackward, SendForward, SendOp
from ._cores import chunk_seed, merge_chunks, select_core


def chunk_owner(send_op: SendOp, p: int, s: int, P: int, A: int) -> int:
    """Ring position whose chunk position ``p`` processes at step ``s``."""
    if send_op is SendOp.RING:
        return (p + s) % P
    if send_op is SendOp.BROADCAST:
        return s % P
    A = max(1, min(A, P))
    if P % A:
        raise ValueError(f"ring size {P} is not divisible by intra_size {A}")
    n = P // A
    g, local = divmod(p, A)
    og = (g + s // A) % n
    if send_op is SendOp.HYBRID:
        return og * A + (local + s % A) % A
    return og * A + s % A


class _Fetcher:
    """Moves chunk payloads from their owners to the ranks that need them at a step."""

    def __init__(self, payload: torch.Tensor, group: dist.ProcessGroup, cfg: RingAttentionConfig) -> None:
        self.payload = payload.contiguous()
        self.group, self.cfg = group, cfg
        self.P, self.me = group.size(), group.rank()
        self._pending: dict[int, tuple[torch.Tensor, Any]] = {}

    def owner(self, p: int, s: int) -> int:
        return chunk_owner(self.cfg.send_op, p, s, self.P, self.cfg.intra_size)

    def _peer(self):
        """Peer-memory transport (CUDA): the payload is published once in symmetric memory and every
        chunk is pulled from its owner by a copy kernel on a side stream."""
        if getattr(self, "_peer_chunks", None) is None:
            self._peer_chunks = False
            if self.payload.is_cuda:
                from ...ops import exchange_fused

                if exchange_fused.PeerChunks.usable(self.payload, self.group):
                    self._peer_chunks = exchange_fused.PeerChunks(self.payload, self.group)
        return self._peer_chunks

    def _start(self, s: int) -> None:
        o = self.owner(self.me, s)
        peer = self._peer()
        if peer:
            buf, ready = peer.start(o)
            self._pending[s] = (buf, ready)
            return
        sends = {p: self.payload for p in range(self.P) if p != self.me and self.owner(p, s) == self.me}
        if o == self.me:
            buf, recvs = self.payload, {}
        else:
            buf = torch.empty_like(self.payload)
            recvs = {o: buf}
        work = sparse_exchange(sends, recvs, self.group, self.cfg.comm, async_op=True)
        self._pending[s] = (buf, work)

    def get(self, s: int) -> torch.Tensor:
        if s not in self._pending:
            self._start(s)
        if self.cfg.overlap_comm and s + 1 < self.P and (s + 1) not in self._pending:
            self._start(s + 1)
        buf, work = self._pending.pop(s)
        if work is not None:
            if isinstance(work, torch.cuda.Event):
                torch.cuda.current_stream(buf.device).wait_event(work)
            else:
                work.wait()
        return buf


def _return_to_owner(contrib: torch.Tensor, s: int, fetch: _Fetcher, acc: torch.Tensor) -> None:
    """Send ``contrib`` (gradient of the chunk visited at step ``s``) to its owner and add what
    other ranks computed for OUR chunk at this step into ``acc``."""
    me, P = fetch.me, fetch.P
    o = fetch.owner(me, s)
    senders = [p for p in range(P) if p != me and fetch.owner(p, s) == me]
    recvs = {p: torch.empty_like(acc) for p in senders}
    sends = {} if o == me else {o: contrib.contiguous()}
    if o == me:
        acc.add_(contrib)
    sparse_exchange(sends, recvs, fetch.group, fetch.cfg.comm)
    for buf in recvs.values():
        acc.add_(buf)


def _project_kv(x: torch.Tensor, w_qkv: torch.Tensor, heads: int) -> tuple[torch.Tensor, torch.Tensor]:
    """K and V ``(..., heads, seq, d)`` of a circulated input chunk ``(..., seq, in_dim)``."""
    e = w_qkv.shape[0] // 3
    kv = torch.matmul(x, w_qkv[e:].to(x.dtype).t())
    k, v = kv[..., :e], kv[..., e:]
    split = lambda t: t.reshape(*t.shape[:-1], heads, e // heads).transpose(-3, -2)  # noqa: E731
    return split(k), split(v)


class _RingAttention(torch.autograd.Function):
    """``forward`` leaves what the backward pass needs besides inputs and output (the circulated payload, the
    log-sum-exp, the kept chunks, the dropout states) in ``stash``, a dict that the caller passes in empty;
    ``setup_context`` moves it onto ``ctx``.  ``vmap`` puts the ensemble axis in front of the batch axes and
    applies the Function once to the whole stack: the schedule only looks at the last three axes."""

    @staticmethod
    def forward(
        q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, x: torch.Tensor | None, w_qkv: torch.Tensor | None,
        scale: float, dropout_p: float, group: dist.ProcessGroup, cfg: RingAttentionConfig, save_chunks: bool, stash: dict,
    ) -> torch.Tensor:
        core = select_core(cfg.attn_backend)
        send_x = cfg.send_in_forward is SendForward.X and x is not None and w_qkv is not None
        heads = q.shape[-3]
        payload = x.contiguous() if send_x else torch.stack((k, v)).contiguous()
        fetch = _Fetcher(payload, group, cfg)
        P, me = fetch.P, fetch.me
        base_seed = int(torch.randint(0, 2**31 - 1, (1,)).item()) if dropout_p > 0.0 else 0
        acc = torch.promote_types(q.dtype, torch.float32)
        out = torch.zeros(q.shape, dtype=acc, device=q.device)
        lse = torch.full(q.shape[:-1], float("-inf"), dtype=acc, device=q.device)
        saved: list[Any] = []
        rng: list[Any] = []
        keep_all = save_chunks and cfg.save_scope is SaveScope.GLOBAL
        for s in range(P):
            chunk = fetch.get(s)
            if send_x:
                kj, vj = _project_kv(chunk, w_qkv, heads)
                kj, vj = kj.to(q.dtype), vj.to(q.dtype)
            else:
                kj, vj = chunk[0], chunk[1]
            seed = chunk_seed(base_seed, me, fetch.owner(me, s))
            out_j, lse_j, state = core.forward(q, kj, vj, scale, dropout_p, seed)
            out, lse = merge_chunks(out, lse, out_j, lse_j.to(acc))
            rng.append(state)
            if keep_all:
                if cfg.offload is Offload.CPU and fetch.owner(me, s) != me:
                    saved.append(cfg.offloader.offload(chunk))
                else:
                    saved.append(chunk)
        if cfg.offload is Offload.CPU:
            cfg.wait_offloads()
        result = out.to(q.dtype)
        if save_chunks:
            stash.update(payload=payload, lse=lse, saved_chunks=saved if keep_all else None, rng=rng, send_x=send_x, heads=heads)
        return result

    @staticmethod
    def setup_context(ctx: Any, inputs: tuple, output: torch.Tensor) -> None:
        q, _, _, _, w_qkv, scale, dropout_p, group, cfg, _, stash = inputs
        if not stash:                                   # forward ran without grad mode: nothing was kept
            return
        ctx.save_for_backward(q, output, w_qkv if stash["send_x"] else None)
        ctx.payload, ctx.lse, ctx.saved_chunks, ctx.rng = stash["payload"], stash["lse"], stash["saved_chunks"], stash["rng"]
        ctx.send_x, ctx.heads = stash["send_x"], stash["heads"]
        ctx.scale, ctx.dropout_p, ctx.group, ctx.cfg = scale, dropout_p, group, cfg
        stash.clear()

    @staticmethod
    def vmap(info: Any, in_dims: tuple, q, k, v, x, w_qkv, scale, dropout_p, group, cfg, save_chunks, stash) -> tuple:
        n = info.batch_size
        if in_dims[4] is not None:
            # one projection weight per member: K and V were projected per member by the caller and carry the
            # gradient to ``x`` and the weights, so they circulate instead of the layer input
            x = w_qkv = None
        q, k, v = (to_front(t, d, n).contiguous() for t, d in zip((q, k, v), in_dims[:3]))
        x = None if x is None else to_front(x, in_dims[3], n).contiguous()
        out = _RingAttention.apply(q, k, v, x, w_qkv, scale, dropout_p, group, cfg, save_chunks, {})
        return out, 0

    @staticmethod
    def backward(ctx: Any, dout: torch.Tensor) -> tuple:
        q, out, w_qkv = ctx.saved_tensors
        payload, lse = ctx.payload, ctx.lse
        cfg, group = ctx.cfg, ctx.group
        core = select_core(cfg.attn_backend)
        fetch = _Fetcher(payload, group, cfg)
        P, me = fetch.P, fetch.me
        dout = dout.contiguous()
        acc = torch.promote_types(q.dtype, torch.float32)
        dq = torch.zeros(q.shape, dtype=acc, device=q.device)
        d_own = torch.zeros(payload.shape, dtype=acc, device=q.device)
        gathered = (
            torch.zeros((P, *payload.shape), dtype=acc, device=q.device)
            if cfg.send_backward is SendBackward.GATHER_DKV
            else None
        )
        dw = torch.zeros_like(w_qkv, dtype=acc) if ctx.send_x else None
        nxt = None
        for s in range(P):
            if ctx.saved_chunks is not None:
                chunk = ctx.saved_chunks[s]
                if chunk.device != q.device:  # offloaded: prefetch the next one while this one computes
                    dev, ev = nxt if nxt is not None else cfg.offloader.prefetch(chunk)
                    chunk = cfg.offloader.consume(dev, ev)
                    nxt = None
                    if s + 1 < P and ctx.saved_chunks[s + 1].device != q.device:
                        nxt = cfg.offloader.prefetch(ctx.saved_chunks[s + 1])
            else:
                chunk = fetch.get(s)
            if ctx.send_x:
                kj, vj = _project_kv(chunk, w_qkv, ctx.heads)
                kj, vj = kj.to(q.dtype), vj.to(q.dtype)
            else:
                kj, vj = chunk[0], chunk[1]
            dq_j, dk_j, dv_j = core.backward(dout, q, kj, vj, out, lse, ctx.scale, ctx.dropout_p, ctx.rng[s])
            dq += dq_j.to(acc)
            if ctx.send_x:
                e = w_qkv.shape[0] // 3
                merge = lambda t: t.to(acc).transpose(-3, -2).reshape(*chunk.shape[:-1], e)  # noqa: E731
                dkv = torch.cat((merge(dk_j), merge(dv_j)), dim=-1)                    # (..., s, 2E)
                contrib = torch.matmul(dkv, w_qkv[e:].to(acc))                            # (..., s, in)
                flat_dkv = dkv.reshape(-1, 2 * e)
                dw[e:] += torch.matmul(flat_dkv.t(), chunk.to(acc).reshape(-1, chunk.shape[-1]))
            else:
                contrib = torch.stack((dk_j, dv_j)).to(acc)
            if gathered is not None:
                gathered[fetch.owner(me, s)] += contrib
            else:
                _return_to_owner(contrib, s, fetch, d_own)
        if gathered is not None:
            dist.all_reduce(gathered, op=dist.ReduceOp.SUM, group=group)
            d_own = gathered[me]
        if ctx.send_x:
            return dq.to(q.dtype), None, None, d_own.to(payload.dtype), dw.to(w_qkv.dtype), None, None, None, None, None, None
        return dq.to(q.dtype), d_own[0].to(payload.dtype), d_own[1].to(payload.dtype), None, None, None, None, None, None, None, None


def _under_vmap(t: torch.Tensor) -> bool:
    try:
        return bool(torch._C._functorch.is_batchedtensor(t))
    except AttributeError:                       # a torch without that probe: let the fused path decide
        return False


def ring_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, group: dist.ProcessGroup, cfg: RingAttentionConfig,
    dropout_p: float = 0.0, x: torch.Tensor | None = None, w_qkv: torch.Tensor | None = None,
) -> torch.Tensor:
    """Attention of local queries against the keys / values of the whole group.
    ``q, k, v``: ``(..., heads, seq_local, d)``.  Grad mode is sampled here because it is
    always off inside ``Function.forward``.

    On CUDA with bf16 operands of head dimension 64 and no dropout the whole ring is one fused forward
    launch (``ops/attention_fused.py``): every send policy of ``cfg`` describes the same sum, the fused
    kernels pull each part from its owner, and circulating ``x`` instead of K / V is a transport
    choice that changes nothing in the result (K and V are differentiable outputs of the local
    projection), so ``cfg`` only matters to the chunked schedule below."""
    if q.is_cuda and not _under_vmap(q):         # the fused launch has no batching rule: vmapped calls take the chunked schedule
        from ...ops import attention_fused

        out = attention_fused.maybe_fused_ring_attention(q, k, v, scale, group, dropout_p)
        if out is not None:
            return out
    return _RingAttention.apply(q, k, v, x, w_qkv, scale, dropout_p, group, cfg, torch.is_grad_enabled(), {})


_subgroup_cache: dict[tuple, tuple[dist.ProcessGroup, dist.ProcessGroup]] = {}


def hybrid_subgroups(group: dist.ProcessGroup, intra_size: int) -> tuple[dist.ProcessGroup, dist.ProcessGroup]:
    """``(intra, inter)`` sub-groups of a sequence-parallel group: ``intra_size`` consecutive
    positions, and the positions with the same offset across the intra groups.  Created once
    per (group, size) with local synchronisation (only member ranks take part)."""
    ranks = tuple(dist.get_process_group_ranks(group))
    key = (ranks, intra_size)
    if key not in _subgroup_cache:
        P = len(ranks)
        if intra_size < 1 or P % intra_size:
            raise ValueError(f"group of {P} ranks does not split into intra groups of {intra_size}")
        me = group.rank()
        intra = inter = None
        for g0 in range(0, P, intra_size):
            members = [ranks[g0 + i] for i in range(intra_size)]
            if g0 <= me < g0 + intra_size:
                intra = dist.new_group(members, use_local_synchronization=True)
        for off in range(intra_size):
            members = [ranks[off + i] for i in range(0, P, intra_size)]
            if me % intra_size == off:
                inter = dist.new_group(members, use_local_synchronization=True)
        _subgroup_cache[key] = (intra, inter)
    return _subgroup_cache[key]
