"""B200-native (sm_100a) lane-verify kernels behind TensorFold's lane-engine interface.

The kernels live in ``libtensorfold_b200.so`` (C ABI, ``include/tensorfold_b200.h``), built ahead of
time by ``python -m tensorfold_b200.build``. There is no CPU or PyTorch fallback.
"""

__version__ = "0.1.0"
