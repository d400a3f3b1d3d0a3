"""In-tree build of the qmlb200 shared libraries for sm_100a.

``build_native()`` compiles every ``csrc/*.cu`` into ``qml_lightning_b200/lib/libqmlb200.so`` with nvcc (no torch
headers, a few seconds per file); ``build_torch_ops()`` compiles the TorchScript operator shim
``csrc/torch_ops.cpp`` with g++ against the installed torch and links it to that library.  Objects are cached by
source modification time.  Run as ``python qml_lightning_b200/build.py`` (a plain script, so that it works before the
libraries exist; importing the package loads them).
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, 'csrc')
LIBDIR = os.path.join(HERE, 'lib')
OBJDIR = os.path.join(HERE, 'build')
NATIVE_LIB = os.path.join(LIBDIR, 'libqmlb200.so')
TORCH_LIB = os.path.join(LIBDIR, 'libqmlb200_torch.so')

NVCC_FLAGS = ['-gencode', 'arch=compute_100a,code=sm_100a', '-lineinfo', '-O3', '-std=c++17', '--expt-relaxed-constexpr',
              '-Xcompiler', '-fPIC', '-I', os.path.join(ROOT, 'include'), '-I', CSRC]


def _nvcc():
    for cand in (os.environ.get('NVCC'), '/usr/local/cuda/bin/nvcc', 'nvcc'):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError('nvcc not found')


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def _run(cmd, verbose):
    if verbose:
        print(' '.join(cmd), flush=True)
    subprocess.run(cmd, check=True)


def build_native(verbose=False, ptxas_info=False):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, '*.cuh')) + glob.glob(os.path.join(ROOT, 'include', '*.h'))
    objs = []
    for src in sorted(glob.glob(os.path.join(CSRC, '*.cu'))):
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + '.o')
        if _newer([src] + headers, obj):
            cmd = [_nvcc()] + NVCC_FLAGS + (['-Xptxas', '-v'] if ptxas_info else []) + ['-c', src, '-o', obj]
            _run(cmd, verbose)
        objs.append(obj)
    if _newer(objs, NATIVE_LIB):
        _run([_nvcc(), '-shared', '-gencode', 'arch=compute_100a,code=sm_100a', '-o', NATIVE_LIB] + objs + ['-lcudart', '-lcublas'], verbose)
    return NATIVE_LIB


def build_torch_ops(verbose=False):
    import torch
    from torch.utils import cpp_extension
    build_native(verbose)
    src = os.path.join(CSRC, 'torch_ops.cpp')
    if not os.path.exists(src):
        return None
    if _newer([src, os.path.join(ROOT, 'include', 'qmlb200.h')], TORCH_LIB):
        inc = []
        for p in cpp_extension.include_paths() + ['/usr/local/cuda/include', os.path.join(ROOT, 'include')]:
            inc += ['-I', p]
        tlib = os.path.join(os.path.dirname(torch.__file__), 'lib')
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        cmd = ['g++', '-O2', '-std=c++17', '-fPIC', '-shared', f'-D_GLIBCXX_USE_CXX11_ABI={abi}', src, '-o', TORCH_LIB] + inc + [
            '-L', LIBDIR, '-lqmlb200', '-L', tlib, '-ltorch', '-ltorch_cpu', '-lc10', '-ltorch_cuda', '-lc10_cuda',
            '-L', '/usr/local/cuda/lib64', '-lcudart', f'-Wl,-rpath,$ORIGIN', f'-Wl,-rpath,{tlib}']
        _run(cmd, verbose)
    return TORCH_LIB


if __name__ == '__main__':
    v = '-q' not in sys.argv
    build_native(verbose=v, ptxas_info='--ptxas' in sys.argv)
    if '--no-torch' not in sys.argv:
        build_torch_ops(verbose=v)
    print('built', NATIVE_LIB)
