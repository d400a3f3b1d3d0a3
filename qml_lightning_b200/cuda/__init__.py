"""Function-level mirror of the upstream extension modules ``qml_lightning.cuda.{pairlist_gpu, fchl_gpu, sorf_gpu,
rff_gpu, utils_gpu}``: same function names, argument orders and in-place accumulation rules, implemented over the C
ABI of ``libqmlb200.so``.  Scripts that call these modules directly (the upstream training path does) can switch their
import to ``qml_lightning_b200.cuda``.  Neighbour lists and element types are accepted where upstream takes them and
ignored: the FCHL19 kernels find neighbours themselves."""
from . import fchl_gpu, pairlist_gpu, rff_gpu, sorf_gpu, utils_gpu  # noqa: F401
