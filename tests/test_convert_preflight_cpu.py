"""The converter's report about what it leaves as plain torch, as one table of cases.

Each case is ``(model, options, outcome)``.  Outcomes: ``silent`` (no warning, the model comes back as it was),
``("warns", pattern)``, ``("raises", pattern)``.  A refused conversion must leave the module tree untouched.  No
case contains a layer that would be converted, so an empty mesh and no process group are enough.

Behaviour of the reference these cases follow: jigsaw/convert.py:174-209 (report lines with qualified names),
:282-315 (``on_unrecognized``, ``non_safe``); its suite for them is tests/test_convert_unrecognized.py.
"""

import re
import warnings

import pytest
import torch
from torch import nn

from jigsaw_b200 import convert


class BareScale(nn.Module):
    """Owns a parameter directly: nothing says how it would be sharded."""

    def __init__(self):
        super().__init__()
        self.gain = nn.Parameter(torch.ones(3))
        self.inner = nn.Tanh()


class Mystery(nn.Module):
    """A leaf that neither table of the converter knows."""

    def forward(self, x):
        return x + 1


def _tree(model):
    return [(name, type(m)) for name, m in model.named_modules()]


CASES = {
    # elementwise layers and dropout act per element: nothing to report
    "elementwise stack": (lambda: nn.Sequential(nn.SiLU(), nn.Dropout(0.1), nn.Sigmoid(), nn.Identity()), {}, "silent"),
    "layer norm left alone on request": (lambda: nn.LayerNorm(6), {"convert_layer_norm": False}, "silent"),
    "unknown leaf, told to ignore": (lambda: nn.Sequential(Mystery()), {"on_unrecognized": "ignore"}, "silent"),
    # unknown things are named with their path inside the model
    "unknown leaf two levels down": (lambda: nn.Sequential(nn.ELU(), nn.Sequential(nn.ReLU(), Mystery())), {},
                                     ("warns", r"1\.1: unrecognized leaf module Mystery")),
    "root owns a parameter": (lambda: BareScale(), {}, ("warns", r"<root>: BareScale owns parameters")),
    "nested owner of a parameter": (lambda: nn.Sequential(nn.ReLU(), BareScale()), {}, ("warns", r"1: BareScale owns parameters")),
    "unknown leaf, told to raise": (lambda: nn.Sequential(Mystery()), {"on_unrecognized": "raise"},
                                    ("raises", r"0: unrecognized leaf module Mystery")),
    "bad mode": (lambda: nn.ReLU(), {"on_unrecognized": "shout"}, ("raises", r"on_unrecognized")),
    # layers that mix values along a dimension that may be sharded: refused, with the way out named
    "pooling": (lambda: nn.Sequential(nn.ReLU(), nn.AdaptiveAvgPool2d(1)), {},
                ("raises", r"non_safe=True(.|\n)*\n  1: non-elementwise module AdaptiveAvgPool2d")),
    "instance norm": (lambda: nn.Sequential(nn.InstanceNorm1d(4)), {}, ("raises", r"0: non-elementwise module InstanceNorm1d")),
    "recurrent": (lambda: nn.Sequential(nn.Tanh(), nn.GRU(4, 4)), {}, ("raises", r"1: non-elementwise module GRU")),
    "pixel shuffle": (lambda: nn.Sequential(nn.PixelShuffle(2)), {}, ("raises", r"0: non-elementwise module PixelShuffle")),
    "embedding bag": (lambda: nn.Sequential(nn.EmbeddingBag(10, 4)), {}, ("raises", r"0: non-elementwise module EmbeddingBag")),
    "softmin": (lambda: nn.Softmin(dim=-1), {}, ("raises", r"<root>: non-elementwise module Softmin")),
    "refused whatever the unrecognized mode": (lambda: nn.Sequential(nn.LocalResponseNorm(2)), {"on_unrecognized": "ignore"},
                                               ("raises", r"non-elementwise module LocalResponseNorm")),
    # non_safe=True hands such layers to the unrecognized mode instead
    "non_safe warns": (lambda: nn.Sequential(nn.MaxPool1d(2)), {"non_safe": True}, ("warns", r"0: non-elementwise module MaxPool1d")),
    "non_safe and ignore": (lambda: nn.ReflectionPad2d(1), {"non_safe": True, "on_unrecognized": "ignore"}, "silent"),
    "non_safe and raise": (lambda: nn.Sequential(nn.ChannelShuffle(2)), {"non_safe": True, "on_unrecognized": "raise"},
                           ("raises", r"0: non-elementwise module ChannelShuffle")),
}


@pytest.mark.parametrize("case", CASES, ids=list(CASES))
def test_report(case):
    build, options, outcome = CASES[case]
    model = build()
    before = _tree(model)
    if outcome == "silent":
        with warnings.catch_warnings():
            warnings.simplefilter("error")
            assert convert.convert_to_jigsaw(model, {}, "cpu", **options) is model
    elif outcome[0] == "warns":
        with pytest.warns(UserWarning, match=outcome[1]):
            assert convert.convert_to_jigsaw(model, {}, "cpu", **options) is model
    else:
        with pytest.raises(ValueError) as info:
            convert.convert_to_jigsaw(model, {}, "cpu", **options)
        assert re.search(outcome[1], str(info.value)), str(info.value)
    assert _tree(model) == before, "the module tree changed"


def test_a_refused_container_is_reported_once_not_per_child():
    block = nn.TransformerDecoderLayer(8, 2, dim_feedforward=16)
    model = nn.Sequential(nn.GELU(), block)
    with pytest.raises(ValueError) as info:
        convert.convert_to_jigsaw(model, {}, "cpu")
    findings = [line for line in str(info.value).splitlines() if line.startswith("  ")]
    assert findings == ["  1: non-elementwise module TransformerDecoderLayer"]


def test_the_plan_lists_every_finding_before_anything_is_changed():
    model = nn.Sequential(Mystery(), nn.BatchNorm2d(3), BareScale(), nn.ReLU())
    plan = convert.ConversionPlan(model)
    assert plan.findings("block") == [("1", "non-elementwise module BatchNorm2d")]
    reported = dict(plan.findings("report"))
    assert set(reported) == {"0", "2"} and "Mystery" in reported["0"] and "owns parameters" in reported["2"]
    assert plan.findings("replace") == [] and [s.path for s in plan.steps if s.action == "keep"] == ["2.inner", "3"]
