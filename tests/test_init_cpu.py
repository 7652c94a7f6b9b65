"""``jigsaw_b200.init``: the initialisers of ``torch.nn.init`` with the fans of the undivided parameter.

Without ``global_shape`` / ``fan_in`` / ``fan_out`` each function must give the bits of its torch namesake for the
same generator; with them, the scale must come from the shape that is named and not from the piece being filled,
so that a piece of a weight is drawn from the distribution of the whole weight.

Reference behaviours covered: tests/test_init.py (drop-in equivalence, re-exported helpers, global shape and
explicit fans, empty pieces, mode names).
"""

import math

import pytest
import torch

from jigsaw_b200 import init

FAN_BASED = {
    "kaiming_uniform_": {"a": math.sqrt(5)},
    "kaiming_normal_": {"mode": "fan_out", "nonlinearity": "relu"},
    "xavier_uniform_": {"gain": 1.5},
    "xavier_normal_": {},
}


def _draw(fn, shape, seed=0, **kw):
    return fn(torch.empty(shape), generator=torch.Generator().manual_seed(seed), **kw)


@pytest.mark.parametrize("name", list(FAN_BASED))
@pytest.mark.parametrize("shape", [(8, 5), (8, 5, 3), (12, 6, 3, 3)])
def test_same_bits_as_torch_when_no_global_shape_is_given(name, shape):
    kw = FAN_BASED[name]
    assert torch.equal(_draw(getattr(init, name), shape, **kw), _draw(getattr(torch.nn.init, name), shape, **kw))


def test_elementwise_initialisers_are_torchs_own_objects():
    for name in ("uniform_", "normal_", "constant_", "ones_", "zeros_", "trunc_normal_", "calculate_gain"):
        assert getattr(init, name) is getattr(torch.nn.init, name), name
    assert sorted(init.__all__) == sorted([*FAN_BASED, "uniform_", "normal_", "constant_", "ones_", "zeros_", "trunc_normal_",
                                           "calculate_gain"])


def test_uniform_bounds_come_from_the_named_shape():
    # (4, 6) of a (4, 60) weight: bound 1 / sqrt(60), far tighter than the piece's own 1 / sqrt(6)
    piece = _draw(init.kaiming_uniform_, (4, 6), a=math.sqrt(5), global_shape=(4, 60))
    assert float(piece.abs().max()) <= 1 / math.sqrt(60) + 1e-6
    piece = _draw(init.xavier_uniform_, (4, 6), global_shape=(4, 60))
    assert float(piece.abs().max()) <= math.sqrt(6 / (60 + 4)) + 1e-6
    # a convolution weight: the receptive field of the named shape counts
    piece = _draw(init.kaiming_uniform_, (2, 3, 3, 3), a=math.sqrt(5), global_shape=(8, 12, 3, 3))
    assert float(piece.abs().max()) <= 1 / math.sqrt(12 * 9) + 1e-6


def test_explicit_fans_win_over_the_named_shape():
    piece = _draw(init.kaiming_uniform_, (1, 1000), a=math.sqrt(5), global_shape=(1, 5), fan_in=1000)
    assert float(piece.abs().max()) <= 1 / math.sqrt(1000) + 1e-6
    piece = _draw(init.xavier_uniform_, (1, 1000), global_shape=(5, 5), fan_out=1000)      # fan_in still from the shape
    assert float(piece.abs().max()) <= math.sqrt(6 / (5 + 1000)) + 1e-6
    got = _draw(init.kaiming_normal_, (8, 5), fan_in=100)
    want = _draw(torch.nn.init.normal_, (8, 5), std=math.sqrt(2 / 100))
    assert torch.allclose(got, want)
    got = _draw(init.xavier_normal_, (8, 5), fan_in=30, fan_out=70)
    want = _draw(torch.nn.init.normal_, (8, 5), std=math.sqrt(2 / 100))
    assert torch.allclose(got, want)
    # both fans given: a 1-D piece (a bias treated as a row) can be filled
    init.xavier_uniform_(torch.empty(7), fan_in=3, fan_out=4)


def test_pieces_are_drawn_from_the_distribution_of_the_whole():
    whole_shape, bound = (4, 4000), 1 / math.sqrt(4000)
    whole = _draw(torch.nn.init.kaiming_uniform_, whole_shape, a=math.sqrt(5))
    halves = [_draw(init.kaiming_uniform_, (4, 2000), seed=s, a=math.sqrt(5), global_shape=whole_shape) for s in (0, 1)]
    for part in (whole, *halves):
        assert 0.85 * bound < float(part.abs().max()) <= bound + 1e-6                  # same bound, and it is reached
    # standard deviation of the normal variants likewise
    piece = _draw(init.xavier_normal_, (64, 512), global_shape=(1024, 512))
    assert abs(float(piece.std()) / math.sqrt(2 / (1024 + 512)) - 1) < 0.05


@pytest.mark.parametrize("name", list(FAN_BASED))
def test_empty_piece_is_left_alone(name):
    for shape, whole in (((0, 4), (8, 4)), ((4, 0), (4, 8))):
        out = getattr(init, name)(torch.empty(shape), global_shape=whole)
        assert out.numel() == 0 and tuple(out.shape) == shape


def test_modes_and_shapes_that_are_refused():
    for fn in (init.kaiming_uniform_, init.kaiming_normal_):
        with pytest.raises(ValueError, match="Mode fan_avg not supported"):
            fn(torch.empty(4, 4), mode="fan_avg")
        with pytest.raises(ValueError, match="fewer than 2 dimensions"):
            fn(torch.empty(6))
        with pytest.raises(ValueError, match="fewer than 2 dimensions"):
            fn(torch.empty(6, 2), global_shape=(6,))
    assert torch.equal(_draw(init.kaiming_normal_, (8, 5), mode="FAN_OUT"), _draw(init.kaiming_normal_, (8, 5), mode="fan_out"))


def test_fill_happens_outside_autograd():
    w = torch.nn.Parameter(torch.empty(4, 4))
    for name in FAN_BASED:
        out = getattr(init, name)(w)
        assert out is w and w.grad_fn is None and w.requires_grad
