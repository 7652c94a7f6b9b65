"""jigsaw_b200: domain- and tensor-parallel training for PyTorch, native to NVIDIA B200.

Swap layers for the distributed layers of :mod:`jigsaw_b200.modules`, give them a process
mesh from :func:`make_process_mesh`, and train as usual: each rank holds its tile of the
data and its shard of the weights.  Every distributed layer gives the same result as the
undivided torch layer, including its initialisation.  On CUDA the communication-bound hot
paths run as hand-written sm_100a kernels (:mod:`jigsaw_b200.ops`) that read and write
peer memory over NVLink; on CPU (gloo) the same layers run on ``torch.distributed``.

Reference parity: jigsaw/__init__.py:3-17.
"""

from . import checkpoint, convert, data, debug, gather, init, launch, log, models, modules, optim, parallel, utils
from ._core.public import set_module
from .mesh import ProcessMesh, make_process_mesh

__all__ = [
    "ProcessMesh",
    "make_process_mesh",
    "checkpoint",
    "convert",
    "data",
    "debug",
    "gather",
    "init",
    "launch",
    "log",
    "models",
    "modules",
    "optim",
    "parallel",
    "utils",
]

set_module(globals(), __all__)
__version__ = "0.1.0"
