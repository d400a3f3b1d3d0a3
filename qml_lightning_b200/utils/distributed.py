"""Process-group plumbing of the sharded normal equations (one process per GPU).

Every rank accumulates the upper triangle of its own ``Z^T Z`` and its own ``Z^T y``; the ranks then exchange the
packed triangle (``F (F + 1) / 2`` float64 values, half the bytes of the square matrix) with ONE all-reduce, mirror it
locally, and rank 0 alone factorises and broadcasts the weights.  Upstream trains on a single device
(models/kernel.py:46-247), so this module has no upstream counterpart.

Failure detection: every process group created here carries a timeout, so a rank that raised, exited or never joined
ends the next collective of the others with an exception instead of a hang.
"""
import datetime
import os

import torch
import torch.distributed as dist

DEFAULT_TIMEOUT_S = float(os.environ.get('QMLB200_DIST_TIMEOUT_S', 180))


def init_process_group(backend, timeout_s=None, device=None, **kwargs):
    """``dist.init_process_group`` with a finite ``timeout`` (seconds; default 180, or QMLB200_DIST_TIMEOUT_S)."""
    timeout = datetime.timedelta(seconds=float(DEFAULT_TIMEOUT_S if timeout_s is None else timeout_s))
    if device is not None and backend == 'nccl':
        kwargs.setdefault('device_id', device)
    dist.init_process_group(backend, timeout=timeout, **kwargs)


def is_distributed():
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def _pack(ZTZ):
    if ZTZ.is_cuda:
        from .. import cabi
        return cabi.pack_upper(ZTZ)
    # host-resident matrix (the cpu_solve option keeps Z^T Z in host memory, models/kernel.py:189-190)
    iu = torch.triu_indices(ZTZ.shape[0], ZTZ.shape[0])
    return ZTZ[iu[0], iu[1]].contiguous()


def _unpack(packed, ZTZ):
    if ZTZ.is_cuda:
        from .. import cabi
        return cabi.unpack_upper(packed, ZTZ)
    iu = torch.triu_indices(ZTZ.shape[0], ZTZ.shape[0])
    ZTZ[iu[0], iu[1]] = packed
    ZTZ[iu[1], iu[0]] = packed
    return ZTZ


def allreduce_normal_equations(ZTZ, ZtrainY):
    """Sum the per-rank partial normal equations in place and leave ``ZTZ`` symmetric.

    ``ZTZ`` needs only its upper triangle on entry.  With a single rank (or no process group) the triangle is just
    mirrored.  A rank that fails before this call makes the collective raise on the others after the group's timeout
    (NCCL: ``torch.distributed.DistBackendError``; gloo: ``RuntimeError``)."""
    packed = _pack(ZTZ)
    if is_distributed():
        dist.all_reduce(packed, op=dist.ReduceOp.SUM)
        dist.all_reduce(ZtrainY, op=dist.ReduceOp.SUM)
    _unpack(packed, ZTZ)
    del packed
    return ZTZ, ZtrainY


def solve_on_rank0_and_broadcast(solve, ZTZ, ZtrainY, nfeatures, device):
    """``alpha f64[nfeatures]`` on every rank: rank 0 runs ``solve(ZTZ, ZtrainY)``, the others receive the result
    (8 bytes per feature) instead of repeating the factorisation."""
    if not is_distributed():
        return solve(ZTZ, ZtrainY)
    alpha = torch.empty(nfeatures, dtype=torch.float64, device=device)
    if dist.get_rank() == 0:
        alpha.copy_(solve(ZTZ, ZtrainY))
    dist.broadcast(alpha, src=0)
    return alpha
