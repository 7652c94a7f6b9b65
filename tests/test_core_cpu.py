"""Runtime layer on CPU: public API surface, mesh, launch environment, logging, init, gather,
converter."""

import importlib
import io
import json
import logging
import os

import pytest
import torch

from dist_utils import assert_close, run_distributed, split

EXPECTED = {
    "jigsaw_b200": {"ProcessMesh", "make_process_mesh", "checkpoint", "convert", "data", "models", "optim", "utils", "debug", "gather", "init", "launch", "log", "modules",
                    "parallel"},
    "jigsaw_b200.parallel": {"JointCommHookState", "OverlappedGradSync", "broadcast_replicas", "check_ddp", "clip_grad_norm_", "joint_comm_hook",
                             "mark_replicated", "no_grad_sync", "overlapped_sum_plan", "reduce_replica_grads", "register_joint_comm_hook",
                             "replica_groups", "sync_grad", "synced_call", "synced_parameters", "wrap_ddp"},
    "jigsaw_b200.modules.functional": {"confusion_to_metrics", "distributed_argmax", "distributed_binary_cross_entropy",
                                       "distributed_binary_cross_entropy_with_logits", "distributed_confusion_matrix",
                                       "distributed_cross_entropy", "distributed_l1_loss", "distributed_log_softmax",
                                       "distributed_mse_loss", "distributed_nll_loss", "distributed_permute",
                                       "distributed_smooth_l1_loss", "redundant_all_reduce"},
    "jigsaw_b200.modules.attention": {"Attention", "AttnBackend", "DistributedAttention", "JIGSAW_TE_AVAILABLE", "Offload",
                                      "RingAttentionConfig", "SaveBackward", "SaveScope", "SendBackward", "SendForward",
                                      "SendOp"},
    "jigsaw_b200.modules.convolution": {"ConvNdConfig", "ConvTransposeNdConfig", "DistributedConv1d", "DistributedConv2d",
                                        "DistributedConv3d", "DistributedConvTranspose1d", "DistributedConvTranspose2d",
                                        "DistributedConvTranspose3d"},
    "jigsaw_b200.modules.linear": {"DistributedLinear", "DistributedMatMulXTW", "DistributedMatMulXW", "DistributedMatMulXWT",
                                   "LinearConfig", "MatMulXTW", "MatMulXW", "MatMulXWT"},
    "jigsaw_b200.modules.normalization": {"DistributedGroupNorm", "DistributedLayerNorm"},
    "jigsaw_b200.modules.roll": {"DistributedRoll", "Roll", "RollConfig"},
    "jigsaw_b200.modules.permute": {"distributed_permute"},
    "jigsaw_b200.modules.metrics": {"DistributedSegmentationMetrics", "confusion_to_metrics", "distributed_confusion_matrix"},
    "jigsaw_b200.modules.activation": {"DistributedSoftmax", "distributed_argmax", "distributed_log_softmax"},
}


def test_public_api_is_pinned():
    for name, expected in EXPECTED.items():
        mod = importlib.import_module(name)
        assert set(mod.__all__) == expected, name
        for n in mod.__all__:
            assert hasattr(mod, n), (name, n)
    import jigsaw_b200.modules as M

    assert len(M.__all__) == 44
    assert M.DistributedConv2d.__module__.startswith("jigsaw_b200.modules")
    for loss in ("DistributedMSELoss", "DistributedCrossEntropyLoss", "DistributedBCEWithLogitsLoss", "DistributedNLLLoss",
                 "DistributedBCELoss", "DistributedL1Loss", "DistributedSmoothL1Loss"):
        assert loss in M.__all__


def test_launch_env_resolution(monkeypatch):
    from jigsaw_b200 import launch

    for k in ("SLURM_PROCID", "SLURM_NTASKS", "SLURM_LOCALID", "RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR",
              "MASTER_PORT", "SLURM_JOB_NODELIST"):
        monkeypatch.delenv(k, raising=False)
    env = launch.resolve_launch_env()
    assert (env.source, env.rank, env.world_size, env.master_addr, env.master_port) == ("single", 0, 1, "localhost", "29500")
    with pytest.raises(RuntimeError):
        launch.resolve_launch_env(strict=True)
    monkeypatch.setenv("RANK", "3")
    monkeypatch.setenv("WORLD_SIZE", "8")
    monkeypatch.setenv("LOCAL_RANK", "1")
    monkeypatch.setenv("MASTER_ADDR", "127.0.0.1")
    env = launch.resolve_launch_env()
    assert (env.source, env.rank, env.world_size, env.local_rank, env.master_addr) == ("torchrun", 3, 8, 1, "127.0.0.1")
    monkeypatch.setenv("SLURM_PROCID", "5")
    monkeypatch.setenv("SLURM_NTASKS", "16")
    monkeypatch.setenv("SLURM_LOCALID", "2")
    env = launch.resolve_launch_env()      # SLURM wins over torchrun
    assert (env.source, env.rank, env.world_size, env.local_rank) == ("slurm", 5, 16, 2)
    launch.set_all_seeds(7)
    a = torch.rand(3)
    launch.set_all_seeds(7)
    assert torch.equal(a, torch.rand(3))
    launch.setup_precision(False)
    assert torch.backends.cuda.matmul.allow_tf32 is False


def test_logging_rank_filter_json_and_once(tmp_path, monkeypatch):
    from jigsaw_b200 import log

    monkeypatch.setenv("RANK", "2")
    monkeypatch.setenv("WORLD_SIZE", "4")
    logger = log.configure_logging("DEBUG", rank=2, log_dir=tmp_path, as_json=True, install_excepthook=False,
                                   enable_faulthandler=False, force=True)
    stream = io.StringIO()
    logger.handlers[0].stream = stream
    log.info("hello %d", 1)
    log.at(0).info("not for me")
    log.info_all("everyone")
    for _ in range(3):
        log.log_once("only once")
    with log.only_rank(1):
        log.info("scoped away")
    with log.timed("block"):
        pass
    lines = [json.loads(row) for row in stream.getvalue().splitlines()]
    msgs = [rec["msg"] for rec in lines]
    assert msgs[:3] == ["hello 1", "everyone", "only once"] and msgs.count("only once") == 1
    assert "not for me" not in msgs and "scoped away" not in msgs and any("block took" in m for m in msgs)
    assert all(rec["rank"] == 2 and rec["world"] == 4 for rec in lines)
    assert (tmp_path / "rank_0002.log").exists()
    with pytest.raises(ValueError):
        log.at("some")
    assert log.assert_all_agree("x", 1) is True     # no process group: trivially true
    log.configure_logging(force=True, install_excepthook=False, enable_faulthandler=False)
    logging.getLogger("jigsaw").handlers[0].stream = io.StringIO()


def test_init_uses_global_fans():
    from jigsaw_b200 import init

    torch.manual_seed(0)
    shard = torch.empty(64, 128)
    init.kaiming_uniform_(shard, a=5 ** 0.5, global_shape=(256, 512))
    assert shard.abs().max() <= 1 / 512 ** 0.5 + 1e-7 and shard.abs().max() > 0.95 / 512 ** 0.5
    full = torch.empty(256, 512)
    torch.nn.init.kaiming_uniform_(full, a=5 ** 0.5)
    assert abs(float(full.std()) - float(shard.std())) < 0.05 * float(full.std())
    x = torch.empty(32, 64)
    init.xavier_normal_(x, global_shape=(128, 256))
    assert abs(float(x.std()) - (2.0 / (128 + 256)) ** 0.5) < 0.1 * (2.0 / 384) ** 0.5
    init.xavier_uniform_(x, fan_in=10, fan_out=20)
    assert x.abs().max() <= (6.0 / 30) ** 0.5 + 1e-6
    init.kaiming_normal_(x, mode="fan_out", nonlinearity="relu", global_shape=(128, 256))
    with pytest.raises(ValueError):
        init.kaiming_uniform_(torch.empty(4))
    with pytest.raises(ValueError):
        init.kaiming_uniform_(x, mode="sideways")


def _worker_mesh_gather_convert(rank, world):
    import jigsaw_b200 as jb
    from jigsaw_b200.modules.attention import Attention

    with pytest.raises(ValueError):
        jb.make_process_mesh({"a": 3, "b": 2})
    with pytest.raises(ValueError):
        jb.make_process_mesh({"a": -1, "b": -1})
    with pytest.raises(ValueError):
        jb.make_process_mesh({"dp": 2, "row": 2}, model_parallel_axes=("dp",))
    with pytest.raises(ValueError):
        jb.make_process_mesh({"model": 4})
    mesh = jb.make_process_mesh({"dp": -1, "row": 2, "col": 1}, model_parallel_axes=("row", "col"))
    assert mesh.axis_sizes == {"dp": 2, "row": 2, "col": 1} and mesh["model"].size() == 2
    assert mesh.device_mesh["dp"].size() == 2 and mesh.coordinate()["dp"] == rank // 2
    mesh = jb.make_process_mesh({"row": 2, "col": 2})
    # gather helpers
    full = torch.arange(2 * 6 * 8, dtype=torch.float32).view(2, 6, 8)
    local = split(full, {1: mesh["row"], 2: mesh["col"]})
    assert_close(jb.gather.gather_results(local, mesh), full, "gather_results", 0, 0)
    assert_close(jb.gather.gather_1d_results(split(full, {2: mesh["model"]}), mesh, dim=-1), full, "gather_1d", 0, 0)
    assert len(jb.gather.gather_results_as_list(local, mesh)) == 4
    t = torch.full((3,), float(rank))
    jb.gather.average_weights([t, None], mesh["model"])
    assert_close(t, torch.full((3,), 1.5), "average_weights", 0, 0)
    # converter: pre-flight, unsafe modules, containers, round trip
    torch.manual_seed(0)

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.norm = torch.nn.LayerNorm(8)
            self.att = Attention(8, 16, 8, 4, "cpu", attn_backend="math")
            self.fc = torch.nn.Linear(8, 8)
            self.act = torch.nn.GELU()

        def forward(self, x):
            return self.act(self.fc(self.att(self.norm(x))))

    serial = Block()
    x = torch.randn(2, 8, 8)
    y_ref = serial(x)
    import copy

    model = jb.convert.convert_to_jigsaw(copy.deepcopy(serial), mesh, "cpu", attn_backend="math", on_unrecognized="raise")
    assert isinstance(model.fc, jb.modules.DistributedLinear) and isinstance(model.norm, jb.modules.DistributedLayerNorm)
    assert isinstance(model.att, jb.modules.DistributedAttention) and model.att.ring
    y = model(split(x, {1: mesh["row"], 2: mesh["col"]}))
    assert_close(y, split(y_ref.detach(), {1: mesh["row"], 2: mesh["col"]}), "converted block output", 1e-4, 1e-5)
    assert jb.debug.count_parameters(model, mesh) == sum(p.numel() for p in serial.parameters())
    keep = jb.convert.convert_to_jigsaw(copy.deepcopy(serial), mesh, "cpu", convert_layer_norm=False, attn_backend="math",
                                        on_unrecognized="ignore")
    assert isinstance(keep.norm, torch.nn.LayerNorm)
    unsafe = torch.nn.Sequential(torch.nn.Linear(4, 4), torch.nn.BatchNorm1d(4))
    before = [type(m) for m in unsafe]
    with pytest.raises(ValueError, match="non-elementwise"):
        jb.convert.convert_to_jigsaw(unsafe, mesh, "cpu")
    assert [type(m) for m in unsafe] == before            # nothing was touched
    jb.convert.convert_to_jigsaw(unsafe, mesh, "cpu", non_safe=True, on_unrecognized="ignore")
    assert isinstance(unsafe[0], jb.modules.DistributedLinear)

    class Odd(torch.nn.Module):
        def forward(self, x):
            return x

    with pytest.warns(UserWarning):
        jb.convert.convert_to_jigsaw(torch.nn.Sequential(Odd()), mesh, "cpu")
    with pytest.raises(ValueError):
        jb.convert.convert_to_jigsaw(torch.nn.Sequential(Odd()), mesh, "cpu", on_unrecognized="raise")
    # reshard a linear layer from 2x2 to 1x4 and back
    lin = jb.modules.DistributedLinear(8, 8, "cpu", mesh["model"], mesh["row"], mesh["col"])
    w0, b0 = lin.merge_weights(mesh)
    mesh2 = jb.make_process_mesh({"row": 1, "col": 4})
    lin.reshard_parameters(mesh, mesh2)
    assert lin.weight.shape == (8, 2)
    w1, b1 = lin.merge_weights(mesh2)
    assert_close(w1, w0, "reshard keeps the global weight", 0, 0)
    lin.reshard_parameters(mesh2, mesh)
    assert lin.weight.shape == (4, 4)
    assert_close(lin.merge_weights(mesh)[1], b0, "reshard round trip bias", 0, 0)


def test_mesh_gather_convert_reshard():
    run_distributed(_worker_mesh_gather_convert, 4)


def _worker_log_collectives(rank, world):
    """The collective parts of the logger on real ranks: a disagreement is seen by every rank, and
    ``log_ranks`` prints one line per rank in rank order from rank 0."""
    from jigsaw_b200 import log

    os.environ["RANK"], os.environ["WORLD_SIZE"] = str(rank), str(world)
    logger = log.configure_logging("DEBUG", as_json=True, install_excepthook=False, enable_faulthandler=False, force=True)
    stream = io.StringIO()
    logger.handlers[0].stream = stream
    assert log.assert_all_agree("depth", 12) is True
    assert log.assert_all_agree("seed", rank, fatal=False) is False          # every rank learns of it
    log.log_ranks("tile %d", rank, level=logging.INFO)
    lines = [json.loads(row) for row in stream.getvalue().splitlines()]
    if rank == 0:
        assert any("ranks disagree on seed" in rec["msg"] and "r2=2" in rec["msg"] for rec in lines)
        dump = [rec["msg"] for rec in lines if rec["msg"].startswith("rank dump")][0]
        assert dump.index("[0] tile 0") < dump.index("[1] tile 1") < dump.index("[2] tile 2")
    else:
        assert not any(rec["msg"].startswith("rank dump") for rec in lines)


def test_logging_collectives_on_ranks():
    run_distributed(_worker_log_collectives, 3)
