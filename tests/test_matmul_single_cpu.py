"""The block products in a single process, without a process group (``model_group=None``): they are then the
plain products, differentiable, usable under ``vmap``, free of parameters, and convertible from the plain modules.

Reference behaviours covered: tests/modules/linear/test_matmul_single.py.
"""

import warnings

import pytest
import torch

import jigsaw_b200 as jb

M = jb.modules
KINDS = {
    "xw": (M.DistributedMatMulXW, M.MatMulXW, (2, 4, 5), (2, 5, 3), lambda x, w: x @ w),
    "xwt": (M.DistributedMatMulXWT, M.MatMulXWT, (2, 4, 5), (2, 3, 5), lambda x, w: x @ w.mT),
    "xtw": (M.DistributedMatMulXTW, M.MatMulXTW, (2, 5, 4), (2, 5, 3), lambda x, w: x.mT @ w),
}


def _operands(kind, lead=()):
    gen = torch.Generator().manual_seed(len(kind))
    _, _, xs, ws, _ = KINDS[kind]
    return (torch.randn(*lead, *xs, dtype=torch.float64, generator=gen, requires_grad=True),
            torch.randn(*lead, *ws, dtype=torch.float64, generator=gen, requires_grad=True))


@pytest.mark.parametrize("kind", list(KINDS))
def test_product_and_gradients_are_torchs(kind):
    cls, plain_cls, _, _, product = KINDS[kind]
    x, w = _operands(kind)
    out, plain, want = cls("cpu", None)(x, w), plain_cls()(x, w), product(x, w)
    assert torch.allclose(out, want) and torch.equal(plain, want)
    seed = torch.randn(want.shape, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    for g, g_want in zip(torch.autograd.grad(out, (x, w), seed), torch.autograd.grad(want, (x, w), seed)):
        assert torch.allclose(g, g_want)


@pytest.mark.parametrize("kind", list(KINDS))
def test_vmap_over_a_leading_axis(kind):
    cls, _, _, _, product = KINDS[kind]
    x, w = _operands(kind, lead=(3,))
    got = torch.vmap(cls("cpu", None))(x, w)
    assert torch.allclose(got, torch.stack([product(x[i], w[i]) for i in range(3)]))
    got = torch.vmap(cls("cpu", None), in_dims=(0, None))(x, w[0])                 # one operand shared by the members
    assert torch.allclose(got, torch.stack([product(x[i], w[0]) for i in range(3)]))


@pytest.mark.parametrize("kind", list(KINDS))
def test_no_parameters_conversion_and_the_retired_argument(kind):
    cls, plain_cls, _, _, product = KINDS[kind]
    layer = cls("cpu", None)
    assert layer.get_parameter_count() == 0 and plain_cls().get_parameter_count() == 0 and not list(layer.parameters())
    assert "model=1" in repr(layer)

    class OneRank:                                     # what the converter needs of a group
        def rank(self):
            return 0

        def size(self):
            return 1

    group = OneRank()
    converted = cls.convert_to_jigsaw(plain_cls(), {"model": group}, "cpu")
    assert isinstance(converted, cls) and converted.model_group is group
    assert isinstance(converted.convert_to_torch({"model": group}), plain_cls)
    with warnings.catch_warnings(record=True) as seen:
        warnings.simplefilter("always")
        old = cls("cpu", None, local_rank=3)
    assert any(issubclass(w.category, DeprecationWarning) and "local_rank" in str(w.message) for w in seen)
    x, w = _operands(kind)
    assert torch.allclose(old(x, w), product(x, w))


def test_configuration_of_another_group_size_is_refused():
    from jigsaw_b200.modules.linear import LinearConfig

    config = LinearConfig(None, linear_layer=False, device="cpu")
    assert config.model_size == 1
    M.DistributedMatMulXW("cpu", None, config)
    with pytest.raises(ValueError, match="different layer"):
        M.DistributedMatMulXW("cpu", None, LinearConfig(None, linear_layer=True, device="cpu"))
