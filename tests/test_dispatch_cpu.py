"""The dispatcher around the fused entry points (``ops/_lib.py``), as far as it can be exercised without a GPU:
what counts as a fused call, what a decline records, strict dispatch, and stepping aside under ``torch.vmap``.
"""

import pytest
import torch

from jigsaw_b200.ops import _lib


@pytest.fixture
def clean_counts():
    saved = dict(_lib.DISPATCH)
    _lib.DISPATCH.clear()
    previous = _lib.set_strict(False)
    yield
    _lib.set_strict(previous)
    _lib.DISPATCH.clear()
    _lib.DISPATCH.update(saved)


def test_counts_reasons_and_strict_dispatch(clean_counts):
    calls = []

    @_lib.audited("probe_op")
    def maybe(x, accept=True):
        calls.append(x.shape)
        return x + 1 if accept else _lib.decline("the probe was told to refuse")

    x = torch.zeros(3)
    assert torch.equal(maybe(x), torch.ones(3)) and _lib.dispatch_counts()["probe_op"] == {"fused": 1, "fallback": 0}
    assert maybe(x, accept=False) is None and _lib._last_reason == "the probe was told to refuse"
    # a decline on CPU tensors is the ordinary CPU path: not counted, and not an error under strict dispatch
    assert _lib.dispatch_counts()["probe_op"] == {"fused": 1, "fallback": 0}
    with _lib.strict_fused():
        assert maybe(x, accept=False) is None
    # record() is what turns a declined CUDA call into an error under strict dispatch
    _lib.decline("outside the kernel's sizes")
    _lib.record("probe_op", False)
    assert _lib.dispatch_counts()["probe_op"]["fallback"] == 1
    with _lib.strict_fused():
        with pytest.raises(_lib.FusedPathDeclined, match="probe_op declined CUDA inputs: outside the kernel's sizes"):
            _lib.record("probe_op", False)
    assert _lib.dispatch_counts(reset=True)["probe_op"]["fallback"] == 2 and not _lib.dispatch_counts()


def test_fused_entry_points_step_aside_under_vmap(clean_counts):
    calls = []

    @_lib.audited("probe_op")
    def maybe(x, w):
        calls.append(1)
        return x @ w

    w = torch.ones(4, 2)
    seen = []

    def member(x):
        out = maybe(x, w)
        seen.append((out is None, _lib._last_reason))
        return x @ w if out is None else out

    got = torch.vmap(member)(torch.ones(3, 5, 4))
    assert seen == [(True, "called under torch.vmap")] and not calls and tuple(got.shape) == (3, 5, 2)
    # the weight alone being batched (stacked member weights) counts as well
    seen.clear()
    torch.vmap(lambda wi: (seen.append(maybe(torch.ones(5, 4), wi) is None), wi)[1])(torch.ones(3, 4, 2))
    assert seen == [True] and not calls
    assert maybe(torch.ones(5, 4), w) is not None and calls == [1]              # outside vmap nothing changes
    assert not _lib._any_batched((torch.ones(2), None, 3, "x"))
