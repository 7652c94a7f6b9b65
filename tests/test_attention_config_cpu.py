"""Attention configuration rules: the ring policy a layer builds for itself when its projection is sharded over the
channel group or when q / k are normalised (K/V must travel, they cannot be rebuilt from a circulated input),
refusal of explicit policies that contradict that, output-bias handling, backend resolution, the dtype the attention
core runs in, enum coercion.

Reference behaviours covered: tests/modules/attention/test_attention_convert.py:65-120 (output bias), :203-277
(automatic K/V policy, refused policies), tests/modules/attention/test_attention_module.py:392-403 (q/k norm),
:434-448 (backend fall-back, core dtype), tests/modules/attention/test_attention_config.py:262-296 (enum names).
"""

import pytest
import torch

from dist_utils import assert_close, run_distributed, split


def test_single_process_rules():
    from jigsaw_b200.modules import attention as A
    from jigsaw_b200.modules.attention import Attention, RingAttentionConfig

    # output bias: on by default, off on request, and the parameter count follows
    with_bias, without = Attention(8, 16, 8, 4, "cpu"), Attention(8, 16, 8, 4, "cpu", out_bias=False)
    assert with_bias.head_concat.bias is not None and without.head_concat.bias is None
    assert with_bias.get_parameter_count() - without.get_parameter_count() == 8
    assert with_bias.qkv.bias is None                                       # the fused projection never has one
    # enum names in any case, members pass through, unknown names list the valid ones
    cfg = RingAttentionConfig(device="cpu", send_in_forward="KV", send_op="Hybrid", save_scope="LOCAL", send_backward="gather_dkv",
                              offload="disabled", attn_backend="Math")
    assert cfg.send_in_forward is A.SendForward.KV and cfg.send_op is A.SendOp.HYBRID and cfg.save_scope is A.SaveScope.LOCAL
    assert cfg.send_backward is A.SendBackward.GATHER_DKV and cfg.offload is A.Offload.DISABLED and cfg.attn_backend is A.AttnBackend.MATH
    assert RingAttentionConfig(device="cpu", send_op=A.SendOp.BROADCAST).send_op is A.SendOp.BROADCAST
    with pytest.raises(ValueError, match="RING"):
        RingAttentionConfig(device="cpu", send_op="carrier_pigeon")          # the message names the valid values
    with pytest.raises(ValueError):
        RingAttentionConfig(device="cpu", intra_size=0)
    assert "send_op" in repr(cfg) and cfg.wait_offloads() is None
    # the core runs in the input dtype, or in the autocast dtype
    x = torch.zeros(2, dtype=torch.float64)
    from jigsaw_b200.modules.attention._attention import attn_core_dtype

    assert attn_core_dtype(x) == torch.float64
    with torch.autocast("cpu", dtype=torch.bfloat16):
        assert attn_core_dtype(x) == torch.bfloat16
    # TransformerEngine is optional: without it the backend resolves to the default core
    assert A.JIGSAW_TE_AVAILABLE in (True, False)
    if not A.JIGSAW_TE_AVAILABLE:
        import warnings

        from jigsaw_b200.modules.attention import RingAttentionConfig

        for build in (lambda: Attention(8, 16, 8, 4, "cpu", attn_backend="te"), lambda: RingAttentionConfig(device="cpu", attn_backend="TE")):
            with warnings.catch_warnings(record=True) as seen:
                warnings.simplefilter("always")
                assert build().attn_backend is A.AttnBackend.SDPA
            assert any(issubclass(w.category, UserWarning) and "falling back to 'sdpa'" in str(w.message) for w in seen)
        with warnings.catch_warnings(record=True) as seen:                 # the other backends say nothing
            warnings.simplefilter("always")
            assert Attention(8, 16, 8, 4, "cpu", attn_backend="math").attn_backend is A.AttnBackend.MATH
        assert not seen


def _worker_policies(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules import attention as A
    from jigsaw_b200.modules.attention import Attention, RingAttentionConfig

    m22 = jb.make_process_mesh({"row": 2, "col": 2})
    m41 = jb.make_process_mesh({"row": 4, "col": 1})
    torch.manual_seed(0)
    serial = Attention(8, 16, 8, 4, "cpu", dtype=torch.float64, out_bias=False, attn_backend="math")
    # a channel split selects the K/V policy without being told, through the converter and the constructor
    layer = Attention.convert_to_jigsaw(serial, m22, "cpu", ring=True, attn_backend="math")
    assert layer.ring and layer.config.send_in_forward is A.SendForward.KV and layer.config.save_for_backward is A.SaveBackward.KV
    built = jb.modules.DistributedAttention(8, 16, 8, 4, m22["col"].rank(), "cpu", m22["row"], m22["col"], ring=True, attn_backend="math")
    assert built.config.send_in_forward is A.SendForward.KV and built.config.save_for_backward is A.SaveBackward.KV
    # explicit policies: K/V is accepted, rebuilding K/V from x (sent or saved) is refused
    for send, save, accepted in (("kv", "kv", True), ("x", "kv", False), ("kv", "x", False)):
        def build():
            cfg = RingAttentionConfig(device="cpu", send_in_forward=send, save_for_backward=save, attn_backend="math")
            return jb.modules.DistributedAttention(8, 16, 8, 4, m22["col"].rank(), "cpu", m22["row"], m22["col"], ring=True,
                                                   attn_backend="math", config=cfg)
        if accepted:
            assert build().ring
        else:
            with pytest.raises(ValueError, match="channel/tensor parallelism"):
                build()
    # q / k normalisation does the same on a mesh without a channel split
    normed = Attention(8, 16, 8, 4, "cpu", dtype=torch.float64, qk_norm=True, attn_backend="math")
    layer = Attention.convert_to_jigsaw(normed, m41, "cpu", ring=True, attn_backend="math")
    assert layer.config.send_in_forward is A.SendForward.KV and layer.config.save_for_backward is A.SaveBackward.KV
    x = torch.randn(2, 8, 8, dtype=torch.float64)
    y = layer(split(x, {1: m41["row"]}))
    assert_close(y, split(normed(x).detach(), {1: m41["row"]}), "ring with q/k norm", 1e-10, 1e-10)
    # without a split and without a norm the input may circulate (the default policy)
    plain = Attention.convert_to_jigsaw(serial, m41, "cpu", ring=True, attn_backend="math")
    assert plain.config.send_in_forward is A.SendForward.X
    # the converted layer keeps the serial layer's output-bias choice; the weights of row replicas come from row 0
    assert layer.head_concat.bias is not None and Attention.convert_to_jigsaw(serial, m22, "cpu", ring=False, attn_backend="math").head_concat.bias is None
    back = Attention.convert_to_jigsaw(serial, m22, "cpu", ring=True, attn_backend="math").convert_to_torch(m22)
    assert back.head_concat.bias is None
    assert_close(back.qkv.weight.data, serial.qkv.weight.data, "round trip of the qkv rows", 0, 0)


def test_ring_policies_follow_the_layout():
    run_distributed(_worker_policies, 4, timeout=300)


def _worker_outer_ring_overlap_warning(rank, world):
    import warnings

    import jigsaw_b200 as jb

    mesh = jb.make_process_mesh({"row": 4, "col": 1})

    def build(**kw):
        with warnings.catch_warnings(record=True) as seen:
            warnings.simplefilter("always")
            jb.modules.DistributedAttention(8, 16, 8, 4, 0, "cpu", mesh["row"], mesh["col"], ulysses=True, ulysses_intra_size=2,
                                            attn_backend="math", **kw)
        return [str(w.message) for w in seen if issubclass(w.category, UserWarning)]

    said = build(ulysses_inter_overlap=True, ulysses_inter_save_scope="global")
    assert len(said) == 1 and "only overlaps the forward pass" in said[0] and "LOCAL" in said[0]
    assert not build(ulysses_inter_overlap=True, ulysses_inter_save_scope="local")
    assert not build(ulysses_inter_overlap=False, ulysses_inter_save_scope="global")


def test_overlap_of_the_outer_ring_with_kept_chunks_says_what_it_overlaps():
    from dist_utils import run_distributed

    run_distributed(_worker_outer_ring_overlap_warning, 4, timeout=120)
