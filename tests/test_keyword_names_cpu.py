"""Keyword names of the public constructors, methods and functions.

A user of the reference who calls ``layer.reshard_parameters(from_process_mesh=a, to_process_mesh=b)`` or
``loss(logits=x, target=y)`` must be able to keep that call.  The table below lists, for the main classes and
functions, the parameter names of the reference's signatures (read from its sources: jigsaw/modules/**,
jigsaw/parallel/*, jigsaw/convert.py, jigsaw/mesh.py, jigsaw/gather.py, jigsaw/debug.py, jigsaw/launch.py,
jigsaw/log.py); every one of them must be a named parameter here, or be swallowed by a ``**kwargs`` of the
same callable.  Extra parameters here are allowed.
"""

import inspect

import pytest

import jigsaw_b200 as jb

CLASSES = {'Attention': {'__init__': ['in_dim', 'embed_dim', 'out_dim', 'heads', 'device', 'dropout_p', 'qk_norm', 'dtype', 'out_bias',
                            'attn_backend'],
               'convert_to_jigsaw': ['attention', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw', 'ring',
                                     'ulysses', 'ulysses_intra_size', 'ulysses_inter_save_scope', 'ulysses_inter_overlap',
                                     'ulysses_inter_offload', 'attn_backend', 'config'],
               'forward': ['x', 'attn_mask']},
 'ConvNdConfig': {'__init__': ['channel_group', 'bias', 'kernel_size', 'stride', 'device', 'channel_comm', 'groups']},
 'ConvTransposeNdConfig': {'__init__': ['channel_group', 'bias', 'kernel_size', 'stride', 'device', 'channel_comm',
                                        'groups']},
 'DistributedAttention': {'__init__': ['in_dim', 'embed_dim', 'out_dim', 'heads', 'local_rank', 'device', 'spatial_group',
                                       'channel_group', 'dropout_p', 'qk_norm', 'ring', 'ulysses', 'ulysses_intra_size',
                                       'ulysses_inter_save_scope', 'ulysses_inter_overlap', 'ulysses_inter_offload',
                                       'attn_backend', 'dtype', 'config', 'out_bias'],
                          'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                          'forward': ['x', 'attn_mask']},
 'DistributedBCELoss': {'__init__': ['reduce_groups', 'weight', 'reduction'], 'forward': ['probs', 'target']},
 'DistributedBCEWithLogitsLoss': {'__init__': ['reduce_groups', 'weight', 'pos_weight', 'reduction'],
                                  'forward': ['logits', 'target']},
 'DistributedConv1d': {'__init__': ['in_channels', 'out_channels', 'kernel_size', 'device', 'spatial_group', 'channel_group',
                                    'stride', 'padding', 'dilation', 'groups', 'bias', 'dtype', 'channel_comm', 'config'],
                       'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw'],
                       'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                       'forward': ['x'],
                       'merge_weights': ['process_mesh_dict', 'col_kw'],
                       'reshard_parameters': ['from_process_mesh_dict', 'to_process_mesh_dict', 'pm_row_key', 'pm_col_key',
                                              'pm_model_key']},
 'DistributedConv2d': {'__init__': ['in_channels', 'out_channels', 'kernel_size', 'device', 'spatial_group', 'channel_group',
                                    'stride', 'padding', 'dilation', 'groups', 'bias', 'dtype', 'channel_comm', 'config'],
                       'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw'],
                       'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                       'forward': ['x'],
                       'merge_weights': ['process_mesh_dict', 'col_kw'],
                       'reshard_parameters': ['from_process_mesh_dict', 'to_process_mesh_dict', 'pm_row_key', 'pm_col_key',
                                              'pm_model_key']},
 'DistributedConv3d': {'__init__': ['in_channels', 'out_channels', 'kernel_size', 'device', 'spatial_group', 'channel_group',
                                    'stride', 'padding', 'dilation', 'groups', 'bias', 'dtype', 'channel_comm', 'config'],
                       'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw'],
                       'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                       'forward': ['x'],
                       'merge_weights': ['process_mesh_dict', 'col_kw'],
                       'reshard_parameters': ['from_process_mesh_dict', 'to_process_mesh_dict', 'pm_row_key', 'pm_col_key',
                                              'pm_model_key']},
 'DistributedConvTranspose1d': {'__init__': ['in_channels', 'out_channels', 'kernel_size', 'device', 'spatial_group',
                                             'channel_group', 'stride', 'padding', 'dilation', 'groups', 'bias', 'dtype',
                                             'channel_comm', 'config'],
                                'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw',
                                                      'model_kw'],
                                'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                                'forward': ['x'],
                                'merge_weights': ['process_mesh_dict', 'col_kw'],
                                'reshard_parameters': ['from_process_mesh_dict', 'to_process_mesh_dict', 'pm_row_key',
                                                       'pm_col_key', 'pm_model_key']},
 'DistributedConvTranspose2d': {'__init__': ['in_channels', 'out_channels', 'kernel_size', 'device', 'spatial_group',
                                             'channel_group', 'stride', 'padding', 'dilation', 'groups', 'bias', 'dtype',
                                             'channel_comm', 'config'],
                                'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw',
                                                      'model_kw'],
                                'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                                'forward': ['x'],
                                'merge_weights': ['process_mesh_dict', 'col_kw'],
                                'reshard_parameters': ['from_process_mesh_dict', 'to_process_mesh_dict', 'pm_row_key',
                                                       'pm_col_key', 'pm_model_key']},
 'DistributedConvTranspose3d': {'__init__': ['in_channels', 'out_channels', 'kernel_size', 'device', 'spatial_group',
                                             'channel_group', 'stride', 'padding', 'dilation', 'groups', 'bias', 'dtype',
                                             'channel_comm', 'config'],
                                'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw',
                                                      'model_kw'],
                                'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                                'forward': ['x'],
                                'merge_weights': ['process_mesh_dict', 'col_kw'],
                                'reshard_parameters': ['from_process_mesh_dict', 'to_process_mesh_dict', 'pm_row_key',
                                                       'pm_col_key', 'pm_model_key']},
 'DistributedCrossEntropyLoss': {'__init__': ['channel_group', 'reduce_groups', 'weight', 'ignore_index', 'reduction',
                                              'label_smoothing', 'dim'],
                                 'forward': ['logits', 'target']},
 'DistributedGroupNorm': {'__init__': ['num_groups', 'num_channels', 'device', 'channel_group', 'eps', 'affine', 'bias',
                                       'dtype', 'spatial_group'],
                          'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw'],
                          'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                          'forward': ['x'],
                          'merge_weights': ['from_process_mesh', 'row_kw', 'col_kw', 'model_kw'],
                          'reshard_parameters': ['from_process_mesh', 'to_process_mesh', 'pm_row_key', 'pm_col_key']},
 'DistributedL1Loss': {'__init__': ['reduce_groups', 'reduction'], 'forward': ['input', 'target']},
 'DistributedLayerNorm': {'__init__': ['normalized_dim', 'local_rank', 'device', 'row_group', 'col_group', 'eps',
                                       'elementwise_affine', 'bias', 'dtype'],
                          'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw'],
                          'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                          'forward': ['x'],
                          'merge_weights': ['from_process_mesh', 'row_kw', 'col_kw', 'model_kw'],
                          'reshard_parameters': ['from_process_mesh', 'to_process_mesh', 'pm_row_key', 'pm_col_key']},
 'DistributedLinear': {'__init__': ['in_dim', 'out_dim', 'device', 'model_group', 'row_group', 'col_group', 'bias', 'config',
                                    'dtype', 'local_rank'],
                       'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw', 'comm'],
                       'convert_to_torch': ['process_mesh_dict', 'row_kw', 'col_kw', 'model_kw'],
                       'forward': ['x'],
                       'merge_weights': ['from_process_mesh', 'row_kw', 'col_kw', 'model_kw'],
                       'reshard_parameters': ['from_process_mesh', 'to_process_mesh', 'pm_row_key', 'pm_col_key',
                                              'pm_model_key']},
 'DistributedMSELoss': {'__init__': ['reduce_groups', 'reduction'], 'forward': ['input', 'target']},
 'DistributedMatMulXW': {'__init__': ['device', 'model_group', 'config', 'local_rank'],
                         'convert_to_jigsaw': ['module', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw',
                                               'comm'],
                         'forward': ['x', 'w']},
 'DistributedNLLLoss': {'__init__': ['channel_group', 'reduce_groups', 'weight', 'ignore_index', 'reduction', 'dim'],
                        'forward': ['log_probs', 'target']},
 'DistributedRoll': {'__init__': ['shifts', 'dims', 'distributed_dims', 'spatial_groups', 'device', 'dtype', 'config'],
                     'convert_to_jigsaw': ['roll', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw',
                                           'dim_to_mesh_axis'],
                     'forward': ['x'],
                     'reshard': ['distributed_dims', 'spatial_groups']},
 'DistributedSegmentationMetrics': {'__init__': ['num_classes', 'channel_group', 'reduce_groups', 'ignore_index', 'dim',
                                                 'exclude'],
                                    'update': ['pred', 'target']},
 'DistributedSmoothL1Loss': {'__init__': ['reduce_groups', 'beta', 'reduction'], 'forward': ['input', 'target']},
 'DistributedSoftmax': {'__init__': ['group', 'dim'],
                        'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw'],
                        'forward': ['x']},
 'LinearConfig': {'__init__': ['model_group', 'linear_layer', 'device', 'comm']},
 'RingAttentionConfig': {'__init__': ['device', 'send_in_forward', 'send_op', 'save_for_backward', 'save_scope',
                                      'send_backward', 'offload', 'intra_size', 'attn_backend', 'overlap_comm', 'comm',
                                      'outer_comm']},
 'Roll': {'__init__': ['shifts', 'dims', 'dtype'], 'forward': ['x']},
 'RollConfig': {'__init__': ['device', 'comm']}}

FUNCTIONS = {'assert_replica_consistency': ['model', 'mesh', 'dp_key', 'atol', 'unmarked'],
 'average_weights': ['params', 'spatial_group'],
 'average_weights_module': ['model', 'spatial_group', 'bias_only'],
 'broadcast_replicas': ['module', 'src'],
 'check_ddp': ['ddp'],
 'clip_grad_norm_': ['parameters', 'max_norm', 'group', 'norm_type', 'error_if_nonfinite'],
 'configure_logging': ['level', 'rank', 'log_dir', 'as_json', 'colour', 'capture_warnings', 'install_excepthook',
                       'enable_faulthandler', 'force'],
 'confusion_to_metrics': ['confusion', 'exclude'],
 'convert_to_jigsaw': ['model', 'process_mesh_dict', 'device', 'row_kw', 'col_kw', 'model_kw', 'convert_layer_norm',
                       'on_unrecognized', 'non_safe'],
 'count_parameters': ['model', 'mesh', 'model_key'],
 'distributed_argmax': ['x', 'dim', 'group'],
 'distributed_binary_cross_entropy': ['probs', 'target', 'weight', 'reduction', 'reduce_groups'],
 'distributed_binary_cross_entropy_with_logits': ['logits', 'target', 'weight', 'pos_weight', 'reduction', 'reduce_groups'],
 'distributed_confusion_matrix': ['pred', 'target', 'num_classes', 'ignore_index', 'dim', 'channel_group', 'reduce_groups',
                                  'pred_is_logits'],
 'distributed_cross_entropy': ['logits', 'target', 'weight', 'ignore_index', 'reduction', 'label_smoothing', 'dim',
                               'channel_group', 'reduce_groups'],
 'distributed_l1_loss': ['input', 'target', 'reduction', 'reduce_groups'],
 'distributed_log_softmax': ['x', 'dim', 'group'],
 'distributed_mse_loss': ['input', 'target', 'reduction', 'reduce_groups'],
 'distributed_nll_loss': ['log_probs', 'target', 'weight', 'ignore_index', 'reduction', 'dim', 'channel_group',
                          'reduce_groups'],
 'distributed_permute': ['x', 'dims', 'row_dim', 'col_dim', 'local_rank', 'device', 'mesh', 'comm'],
 'distributed_smooth_l1_loss': ['input', 'target', 'beta', 'reduction', 'reduce_groups'],
 'gather_1d_results': ['x', 'process_mesh_dict', 'dim', 'pm_key'],
 'gather_results': ['x', 'process_mesh_dict', 'pm_key_row', 'pm_key_col', 'pm_key_model'],
 'make_process_mesh': ['axes', 'device_type', 'model_parallel_axes', 'model_key'],
 'mark_replicated': ['param', 'groups', 'extend'],
 'redundant_all_reduce': ['x', 'groups'],
 'register_joint_comm_hook': ['ddp', 'wrapper'],
 'resolve_launch_env': ['strict'],
 'set_all_seeds': ['seed'],
 'sync_grad': [],
 'synced_call': ['module'],
 'wrap_ddp': ['module', 'mesh', 'dp_key', 'joint_hook']}


def _accepts(callable_, names):
    parameters = inspect.signature(callable_).parameters
    if any(p.kind is p.VAR_KEYWORD for p in parameters.values()):
        return []
    return [n for n in names if n not in parameters and n not in ("args", "kwargs")]


def _find(name):
    for module in (jb.modules, jb.modules.functional, jb.modules.activation, jb.modules.linear, jb.modules.convolution,
                   jb.modules.attention, jb.modules.roll, jb.parallel, jb.convert, jb.mesh, jb.gather, jb.debug, jb.launch, jb.log):
        if hasattr(module, name):
            return getattr(module, name)
    raise AssertionError(f"{name} is not a public name")


@pytest.mark.parametrize("cls_name", sorted(CLASSES))
def test_methods_take_the_reference_keywords(cls_name):
    cls = _find(cls_name)
    missing = {}
    for method, names in CLASSES[cls_name].items():
        assert hasattr(cls, method), f"{cls_name}.{method} does not exist"
        lost = _accepts(getattr(cls, method), names)
        if lost:
            missing[method] = lost
    assert not missing, f"{cls_name}: keywords of the reference that are not accepted: {missing}"


@pytest.mark.parametrize("fn_name", sorted(FUNCTIONS))
def test_functions_take_the_reference_keywords(fn_name):
    lost = _accepts(_find(fn_name), FUNCTIONS[fn_name])
    assert not lost, f"{fn_name}: keywords of the reference that are not accepted: {lost}"


def _worker_attribute_names(rank, world):
    """Attributes of the reference's layers that describe the cut (read by user code that sizes buffers or logs)."""
    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    M, row, col = jb.modules, mesh["row"], mesh["col"]
    ln = M.DistributedLayerNorm(8, mesh["model"].rank(), "cpu", row, col)
    assert ln.local_dim == 4 and ln.spatial_group is row and ln.channel_group is col and ln.local_rank == mesh["model"].rank()
    gn = M.DistributedGroupNorm(4, 8, "cpu", channel_group=col, spatial_group=row)
    assert (gn.num_local_groups, gn.num_local_channels) == (2, 4)
    lin = M.DistributedLinear(8, 12, "cpu", mesh["model"], row, col)
    assert lin.global_weight_shape == (12, 8) and lin.global_bias_shape == (12,)
    assert M.DistributedLinear(8, 12, "cpu", mesh["model"], row, col, bias=False).global_bias_shape is None


def test_attributes_that_describe_the_cut():
    import os
    import sys

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_utils import run_distributed

    run_distributed(_worker_attribute_names, 4, timeout=120)
