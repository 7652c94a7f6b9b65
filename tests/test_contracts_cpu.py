"""Contracts of constructors, ``convert_to_jigsaw`` and ``reshard_parameters``: a mesh axis that does not
divide a parameter is refused on every rank before the first collective (the job fails instead of hanging);
options of the converter; meshes keyed with other names; multi-hop re-sharding; dtypes.

Reference behaviours covered: tests/test_reshard_convert_coverage.py:47-105 (converter divisibility), :109-170
(constructor divisibility), :173-216 (LayerNorm rejections and the ``convert_layer_norm`` flag), :219-302 (reshard
divisibility), :305-342 (alias-keyed meshes), :345-376 (container recursion), :378-447 (multi-hop), :449-477 and
:572-593 (dtypes).
"""

import copy

import pytest
import torch

from dist_utils import all_ok, assert_close, run_distributed, split


def _meshes():
    import jigsaw_b200 as jb

    return (jb.make_process_mesh({"row": 2, "col": 2}), jb.make_process_mesh({"row": 1, "col": 4}),
            jb.make_process_mesh({"row": 4, "col": 1}))


def _worker_divisibility(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200 import convert
    from jigsaw_b200.modules.attention import Attention

    m22, m14, m41 = _meshes()
    M = jb.modules
    # converter: every rank raises alike
    for build, kind in ((lambda: torch.nn.Linear(3, 4), ValueError), (lambda: torch.nn.Linear(4, 3), ValueError),
                        (lambda: torch.nn.Conv2d(3, 4, 2), ValueError), (lambda: torch.nn.ConvTranspose2d(4, 3, 2), ValueError),
                        (lambda: torch.nn.LayerNorm(3), ValueError), (lambda: torch.nn.LayerNorm([4, 4]), NotImplementedError)):
        with pytest.raises(kind):
            convert.convert_to_jigsaw(build(), m22, "cpu")
    with pytest.raises(ValueError, match="channel group size"):
        convert.convert_to_jigsaw(torch.nn.Conv2d(3, 4, 2), m22, "cpu")
    with pytest.raises(ValueError):
        Attention.convert_to_jigsaw(Attention(12, 12, 12, 3, "cpu"), m14, "cpu")            # 3 heads over 4 channel ranks
    # constructors check the same contracts
    with pytest.raises(ValueError, match="in_dim=3"):
        M.DistributedLinear(3, 4, "cpu", m22["model"], m22["row"], m22["col"])
    with pytest.raises(ValueError, match="bias"):
        M.DistributedLinear(4, 2, "cpu", m14["model"], m14["row"], m14["col"])             # 2 outputs over 4 column ranks
    with pytest.raises(ValueError, match="normalized_dim=3"):
        M.DistributedLayerNorm(3, m22["model"].rank(), "cpu", m22["row"], m22["col"])
    with pytest.raises(ValueError, match="num_groups=3"):
        M.DistributedGroupNorm(3, 6, "cpu", channel_group=m22["col"])
    # reshard: a target mesh that cannot hold the global parameter is refused before anything is gathered
    lin = convert.convert_to_jigsaw(torch.nn.Linear(2, 2), m22, "cpu")
    with pytest.raises(ValueError):
        lin.reshard_parameters(m22, m41)
    for layer in (torch.nn.Conv2d(2, 2, 2), torch.nn.ConvTranspose2d(2, 2, 2)):
        conv = convert.convert_to_jigsaw(layer, m22, "cpu")
        with pytest.raises(ValueError, match="channel group size"):
            conv.reshard_parameters(m22, m14)
    ln = M.DistributedLayerNorm(6, m22["model"].rank(), "cpu", m22["row"], m22["col"])
    with pytest.raises(ValueError):
        ln.reshard_parameters(m22, m14)
    gn = M.DistributedGroupNorm(2, 6, "cpu", channel_group=m22["col"])
    with pytest.raises(ValueError):
        gn.reshard_parameters(m22, m14)
    assert all_ok(True)


def test_divisibility_is_checked_before_any_collective():
    run_distributed(_worker_divisibility, 4, timeout=300)


def _worker_converter_options(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200 import convert

    m22, m14, m41 = _meshes()
    M = jb.modules
    # convert_layer_norm=False leaves nn.LayerNorm alone; the default converts it
    model = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.LayerNorm(4))
    keep = model[1]
    out = convert.convert_to_jigsaw(model, m22, "cpu", convert_layer_norm=False)
    assert out[1] is keep and isinstance(out[0], M.DistributedLinear)
    out = convert.convert_to_jigsaw(torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.LayerNorm(4)), m22, "cpu")
    assert isinstance(out[1], M.DistributedLayerNorm)
    # containers: leaves are swapped in place, a module without mapped leaves comes back unchanged
    seq = torch.nn.Sequential(torch.nn.Linear(4, 8), torch.nn.GELU(), torch.nn.Sequential(torch.nn.Linear(8, 4), torch.nn.Tanh()))
    act = seq[1]
    out = convert.convert_to_jigsaw(seq, m22, "cpu")
    assert out is seq and out[1] is act and isinstance(out[0], M.DistributedLinear) and isinstance(out[2][0], M.DistributedLinear)
    plain = torch.nn.Sequential(torch.nn.GELU(), torch.nn.Tanh())
    assert convert.convert_to_jigsaw(plain, m22, "cpu") is plain
    # a mesh keyed with other names: convert, merge, reshard onto itself, convert back
    alias = {"tok": m22["row"], "chan": m22["col"], "mp": m22["model"]}
    for bias in (True, False):
        torch.manual_seed(1234)
        ref = torch.nn.Linear(24, 16, bias=bias)
        jm = convert.convert_to_jigsaw(copy.deepcopy(ref), alias, "cpu", row_kw="tok", col_kw="chan", model_kw="mp")
        w, b = jm.merge_weights(alias, "tok", "chan", "mp")
        assert_close(w, ref.weight.data, "alias mesh: merged weight", 0, 0)
        assert (b is None) == (not bias)
        jm.reshard_parameters(alias, alias, "tok", "chan", "mp")
        back = jm.convert_to_torch(alias, "tok", "chan", "mp")
        assert_close(back.weight.data, ref.weight.data, "alias mesh: weight after the round trip", 0, 0)
        assert (back.bias is None) == (not bias)
        if bias:
            assert_close(back.bias.data, ref.bias.data, "alias mesh: bias after the round trip", 0, 0)


def test_converter_options_containers_and_alias_keys():
    run_distributed(_worker_converter_options, 4, timeout=300)


def _worker_multi_hop(rank, world):
    """2x2 -> 1x4 -> 4x1 -> 2x2: after every hop the merged parameters equal the original, and the layer
    computes the undivided layer's output on the mesh it lives on; float64 stays float64."""
    import jigsaw_b200 as jb
    from jigsaw_b200 import convert

    meshes = _meshes()
    torch.manual_seed(7)
    ref = torch.nn.Linear(8, 16).double()
    x = torch.randn(3, 8, 8, dtype=torch.float64)
    jm = convert.convert_to_jigsaw(copy.deepcopy(ref), meshes[0], "cpu")
    assert jm.weight.dtype == torch.float64
    order = [0, 1, 2, 0]
    for a, b in zip(order, order[1:]):
        jm.reshard_parameters(meshes[a], meshes[b])
        w, bias = jm.merge_weights(meshes[b])
        assert_close(w, ref.weight.data, f"linear hop {a}->{b}: weight", 0, 0)
        assert_close(bias, ref.bias.data, f"linear hop {a}->{b}: bias", 0, 0)
        cuts = {1: meshes[b]["row"], 2: meshes[b]["col"]}
        assert_close(jm(split(x, cuts)), split(ref(x).detach(), cuts), f"linear hop {a}->{b}: output", 1e-12, 1e-12)
    refc = torch.nn.Conv2d(4, 8, 3, padding=1).double()
    img = torch.randn(2, 4, 8, 8, dtype=torch.float64)
    jc = convert.convert_to_jigsaw(copy.deepcopy(refc), meshes[0], "cpu")
    assert jc.weight.dtype == torch.float64
    for a, b in zip(order, order[1:]):
        jc.reshard_parameters(meshes[a], meshes[b])
        back = jc.convert_to_torch(meshes[b])
        assert back.weight.dtype == torch.float64
        assert_close(back.weight.data, refc.weight.data, f"conv hop {a}->{b}: weight", 0, 0)
        cuts = {1: meshes[b]["col"], 3: meshes[b]["row"]}
        assert_close(jc(split(img, cuts)), split(refc(img).detach(), cuts), f"conv hop {a}->{b}: output", 1e-12, 1e-12)
    # constructor dtypes
    layer = jb.modules.DistributedConv2d(4, 4, 3, "cpu", meshes[0]["row"], meshes[0]["col"], padding=1, dtype=torch.bfloat16)
    assert all(p.dtype == torch.bfloat16 for p in layer.parameters())
    att = jb.modules.attention.Attention(8, 8, 8, 2, "cpu", dtype=torch.float64)
    assert all(p.dtype == torch.float64 for p in att.parameters())


def test_multi_hop_reshard_and_dtypes():
    run_distributed(_worker_multi_hop, 4, timeout=300)
