"""The tensor-core kernels (csrc/pca_tc2.cu, csrc/rff_tc.cu) build tcgen05.mma shared-memory descriptors by hand.  This test
compiles a small stand-alone program (tests/native/mma_operand_layouts.cu) that runs single-block accumulation chains with
operands in the no-swizzle K-major, SWIZZLE_128B K-major and SWIZZLE_128B MN-major layouts and checks the tensor-memory
result against a host product; it also prints the measured cycles per instruction for several shapes (run with ``-s`` to
see them; they are the figures quoted in the design notes on operand layouts)."""
import os
import re
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_operand_layouts_give_exact_products(tmp_path):
    nvcc = shutil.which('nvcc') or '/usr/local/cuda/bin/nvcc'
    if not os.path.exists(nvcc):
        pytest.skip('nvcc not available on this machine')
    exe = str(tmp_path / 'mma_operand_layouts')
    subprocess.run([nvcc, '-gencode', 'arch=compute_100a,code=sm_100a', '-O3', '-o', exe,
                    os.path.join(HERE, 'native', 'mma_operand_layouts.cu')], check=True)
    out = subprocess.run([exe], check=True, capture_output=True, text=True, timeout=300).stdout
    print(out)
    checked = re.findall(r'^mode (\d) N +(\d+) K (\d+): max \|err\| (\S+) status (\d)', out, flags=re.M)
    assert len(checked) == 8, out
    for mode, n, k, err, status in checked:
        assert float(err) == 0.0 and status == '0', (mode, n, k, err, status)
    assert 'status 1' not in out
    # an N = 256 instruction with both operands in shared memory runs at its math time (128 cycles) in either layout
    cycles = {(m, int(n)): float(c) for m, n, c in re.findall(r'^mode (\d) N +(\d+) K \d+: .*?, (\S+) cycles per MMA', out, flags=re.M)}
    assert cycles[('0', 256)] < 140 and cycles[('1', 256)] < 140
