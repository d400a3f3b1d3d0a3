"""Failure detection on the device without a fault: a bounded wait that runs out.

The tensor-core projection kernel waits on mbarriers with an iteration limit.  This test builds a second copy of the
library in which ONLY the first wait of the MMA-issuing warp is granted no polls at all (compile-time macro
``QMLB_TEST_FIRST_WAIT_POLLS`` = 0; a single ``mbarrier.try_wait`` may itself block for a while, so any positive number
could still succeed); every other wait keeps the production limit.  That first wait then gives up before
anything was issued to the tensor cores, the other warps run into their own (full-length) limits, the block drains its
bulk copies, releases its tensor memory and returns.  Checked: the event is counted, the output tile carries NaN instead
of stale data, and the production library computes correct results on the same context right afterwards.
"""
import ctypes
import glob
import os
import subprocess

import pytest
import torch

from qml_lightning_b200 import _lib

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, 'qml_lightning_b200')


def _build_test_library(tmpdir):
    nvcc = '/usr/local/cuda/bin/nvcc' if os.path.exists('/usr/local/cuda/bin/nvcc') else 'nvcc'
    flags = ['-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-std=c++17', '--expt-relaxed-constexpr', '-Xcompiler', '-fPIC',
             '-I', os.path.join(ROOT, 'include'), '-I', os.path.join(PKG, 'csrc')]
    obj = os.path.join(tmpdir, 'pca_tc2_firstwait.o')
    subprocess.run([nvcc] + flags + ['-DQMLB_TEST_FIRST_WAIT_POLLS=0', '-c', os.path.join(PKG, 'csrc', 'pca_tc2.cu'), '-o', obj], check=True)
    others = [o for o in sorted(glob.glob(os.path.join(PKG, 'build', '*.o'))) if os.path.basename(o) != 'pca_tc2.o']
    assert others, 'the product library has to be built first (python qml_lightning_b200/build.py)'
    so = os.path.join(tmpdir, 'libqmlb200_firstwait.so')
    subprocess.run([nvcc, '-shared', '-gencode', 'arch=compute_100a,code=sm_100a', '-o', so, obj] + others + ['-lcudart', '-lcublas'],
                   check=True)
    lib = ctypes.CDLL(so)
    for name in ('qmlb_pca_pack_bytes', 'qmlb_pca_pack', 'qmlb_pca_project_packed', 'qmlb_tc_timeouts', 'qmlb_last_error'):
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = _lib.SIGNATURES[name]
    return lib


def _project(lib, x, red, group_start, out):
    nel, repsize, npcas = red.shape
    nbytes = lib.qmlb_pca_pack_bytes(nel, repsize, npcas, 0)
    packed = torch.empty(nbytes, dtype=torch.uint8, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.qmlb_pca_pack(red.data_ptr(), nel, repsize, npcas, 0, packed.data_ptr(), nbytes, stream) == 0
    rc = lib.qmlb_pca_project_packed(x.data_ptr(), packed.data_ptr(), group_start.data_ptr(), nel, x.shape[0], repsize, npcas, 0,
                                     out.data_ptr(), stream)
    assert rc == 0, lib.qmlb_last_error()
    torch.cuda.synchronize()


def test_first_wait_runs_out_and_the_context_survives(tmp_path):
    product = _lib.load()
    gen = torch.Generator().manual_seed(0)
    rows, repsize, npcas = 128, 336, 128                       # one row tile, one column tile: a single block
    x = torch.randn(rows, repsize, generator=gen).to(DEV)
    red = torch.randn(1, repsize, npcas, generator=gen).to(DEV)
    gs = torch.tensor([0, rows], dtype=torch.int32, device=DEV)
    ref = x.double() @ red[0].double()

    test_lib = _build_test_library(str(tmp_path))
    assert test_lib.qmlb_tc_timeouts() == 0
    out = torch.full((rows, npcas), 7.0, device=DEV)
    _project(test_lib, x, red, gs, out)                        # returns: the waits are bounded
    assert test_lib.qmlb_tc_timeouts() == 1                    # the give-up was recorded (host reads a status, no fault)
    assert bool(torch.isnan(out).all())                        # results withheld and marked, nothing stale or partial

    before = product.qmlb_tc_timeouts()
    good = torch.empty(rows, npcas, device=DEV)
    _project(product, x, red, gs, good)                        # same context, production limits
    assert product.qmlb_tc_timeouts() == before
    assert float((good.double() - ref).abs().max()) <= 3e-6 * float(ref.abs().max())
