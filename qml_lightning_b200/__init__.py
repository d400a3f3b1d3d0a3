"""B200-native rebuild of the qml-lightning inference / training hot path.

Public classes keep the upstream names and signatures:
``FCHLCuda`` (representations/FCHL.py), ``HadamardFeaturesModel`` (models/hadamard_features.py) and
``RandomFourrierFeaturesModel`` (models/random_features.py).  All arithmetic runs in hand-written sm_100a kernels
behind the C ABI of ``lib/libqmlb200.so``; ``lib/libqmlb200_torch.so`` registers the TorchScript operators.
Both are built in-tree by ``python qml_lightning_b200/build.py``; nothing falls back to the CPU or to PyTorch ops.
"""
import os

import torch

from . import _lib

_HERE = os.path.dirname(os.path.abspath(__file__))
TORCH_OPS_LIB = os.environ.get('QML_LIGHTNING_TORCHSCRIPT_LIB_B200', os.path.join(_HERE, 'lib', 'libqmlb200_torch.so'))
_ops_loaded = False


def load_torch_ops():
    """Register the TorchScript operators (idempotent); raises if the shim has not been built."""
    global _ops_loaded
    if not _ops_loaded:
        if not os.path.exists(TORCH_OPS_LIB):
            raise RuntimeError(f"{TORCH_OPS_LIB} not found: build it with `python qml_lightning_b200/build.py`")
        _lib.load()  # libqmlb200.so must be resolvable first
        torch.ops.load_library(TORCH_OPS_LIB)
        _ops_loaded = True


load_torch_ops()

from .representations.FCHL import FCHLCuda  # noqa: E402
from .models.hadamard_features import HadamardFeaturesModel  # noqa: E402
from .models.random_features import RandomFourrierFeaturesModel  # noqa: E402

__all__ = ['FCHLCuda', 'HadamardFeaturesModel', 'RandomFourrierFeaturesModel', 'load_torch_ops']
