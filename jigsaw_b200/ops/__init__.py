"""Hand-written sm_100a kernels and their PyTorch bindings.

``csrc/`` holds the CUDA sources (one translation unit, C ABI), ``_build.py`` compiles them
in-tree with nvcc, ``_lib.py`` loads the shared object with ctypes.  The ``*_fused`` modules
expose ``maybe_fused_*`` entry points used by the layers: they return ``None`` when the
shape / dtype / device is outside what the kernels cover (the caller then takes the
``torch.distributed`` path) and raise if a CUDA device is present but the library is not.
"""
