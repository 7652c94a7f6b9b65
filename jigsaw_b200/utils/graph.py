"""Capture a whole training step (forward, backward, optimizer) in one CUDA graph.

A domain-parallel step on small per-rank tiles is bound by the host: dozens of kernel
launches, autograd bookkeeping and collectives' launch paths per step.  Replaying the step
as one graph removes that.  Two things make a captured step different from an eager one:

* Inputs are *static* tensors: copy each batch into ``graphed.inputs`` (``copy_`` from pinned
  host memory is enough) and call ``graphed.replay()``.
* The fused kernels signal halo arrival with per-buffer epochs that must grow from step to
  step although a graph's launch arguments are frozen.  During capture the halo descriptors
  therefore point at a device counter that the graph itself increments once per replay; a
  launch captured with epoch ``e`` uses ``e + replays * EPOCH_STRIDE``.  The host-side epoch
  bookkeeping advances by the same stride per replay, so eager launches may follow replays
  (up to ``EPOCH_STRIDE`` productions of one buffer slot between two replays).
* Staging blocks that peers write into are used in rings of two; a step that uses such a ring an odd number
  of times would end and begin on the same block, so the capture then appends a one-element all-reduce
  over all ranks that separates consecutive replays.

The optimizer must be capturable (``jigsaw_b200.optim.FusedAdam``, or ``torch.optim.Adam(...,
capturable=True)``; ``fused=True`` is fine).  A learning rate given as a float is frozen into the
graph; for a schedule give the optimizer a one-element device tensor and overwrite it in place
between replays.  NCCL collectives inside the step are captured by PyTorch's process group.

Reference parity: none - the reference has no graph capture.
"""

from __future__ import annotations

from collections.abc import Callable, Sequence

import torch

from ..ops import _lib, symm


EPOCH_STRIDE = 4096


class GraphedStep:
    """``step_fn(*inputs) -> tensor | tuple of tensors`` (e.g. the loss), captured after
    ``warmup`` eager runs.  ``step_fn`` must do everything the step needs, including
    ``zero_grad(set_to_none=True)`` *before* the forward pass and ``optimizer.step()``."""

    def __init__(self, step_fn: Callable, inputs: Sequence[torch.Tensor], warmup: int = 3) -> None:
        self.inputs = tuple(inputs)
        device = self.inputs[0].device
        if device.type != "cuda":
            raise ValueError("GraphedStep needs CUDA tensors")
        self._arena = symm.arena(device)
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                step_fn(*self.inputs)
            launches = _lib.LAUNCHES
            self._arena.start_ring_count()
            step_fn(*self.inputs)
            self.launches_per_step = _lib.LAUNCHES - launches    # kernels of this package per replay
            fenced = self._arena.some_ring_used_an_odd_number_of_times()
            if fenced:
                self._fence(device)                              # its staging block comes into being outside the capture
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self._graph = torch.cuda.CUDAGraph()
        self._slots = (set(), [])
        self._arena.begin_capture(EPOCH_STRIDE)
        try:
            with torch.cuda.graph(self._graph):
                self._arena.replay.add_(1)
                self.outputs = step_fn(*self.inputs)
                if fenced:
                    self._fence(device)
        finally:
            self._slots = self._arena.end_capture()
        # Capturing advanced the host epochs of the produced slots without running anything;
        # replay n (counter = n) publishes captured + n * stride, which is what the host holds
        # after n calls of advance().

    @staticmethod
    def _fence(device: torch.device) -> None:
        """A one-element sum over all ranks at the end of the captured step: a rank leaves it only after every
        rank has entered it, i.e. after every rank's kernels of this replay are complete in stream order, so
        the first operation of the next replay may overwrite a staging block the last one of this replay used."""
        import torch.distributed as dist

        if not dist.is_initialized() or dist.get_world_size() < 2:
            return
        from ..ops import reduce_fused

        token = torch.zeros(4, dtype=torch.float32, device=device)
        ranks = list(range(dist.get_world_size()))
        if reduce_fused.usable([token], ranks):
            reduce_fused._launch([token], ranks, 1.0, "fence")
        else:
            dist.all_reduce(token)

    def close(self) -> None:
        """Destroy the graph.  Call this before ``dist.destroy_process_group()``: a live graph
        that holds captured NCCL collectives keeps their communicator busy and the teardown of
        the process group waits for it."""
        if self._graph is not None:
            self._graph.reset()
            self._graph = None

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    def replay(self):
        """Run the captured step on the current contents of ``inputs``; returns the static outputs."""
        if self._graph is None:
            raise RuntimeError("this GraphedStep was closed")
        self._graph.replay()
        self._arena.advance(self._slots, EPOCH_STRIDE)
        return self.outputs
