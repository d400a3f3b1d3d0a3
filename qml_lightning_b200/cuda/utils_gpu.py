"""``utils_gpu.matmul_and_reduce`` of the upstream project (cuda/utils_cuda.cpp:26-33, 68)."""
from .. import cabi


def matmul_and_reduce(A, B, C):
    """``C f64[M,N] += A f32[M,K] @ B f32[K,N]`` in place: a float32-accurate product accumulated in float64
    (kernel cuda/utils_kernel.cu:70-129).  build_Z_components calls it with ``A = Ztrain.float().T`` and
    ``B = Ztrain.float()`` (models/kernel.py:176-188); ``A`` may be any strided view."""
    cabi.matmul_and_reduce(A, B, C)
