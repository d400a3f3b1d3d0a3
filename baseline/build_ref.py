"""Builds the two TorchScript operator libraries of the upstream project for sm_100a into ``baseline/_ref/``.

    python baseline/build_ref.py [path of an upstream qml-lightning checkout]

They serve one purpose: ``baseline/ref_cuda_bench.py`` runs upstream's own CUDA operators next to this repository's
on the same inputs.  The upstream sources are compiled from a scratch copy outside the repository (nothing of them is
stored here; ``baseline/_ref/`` is git-ignored) with the flags of upstream's setup.py (``-O2``) plus the sm_100a target.

ONE change is applied to the scratch copy, and every number obtained with these libraries is labelled "reference +
72-byte allocation fix": the launcher of the FCHL19 backward kernel requests ``nRs2 + nRs3 + 8 * max_neighbours`` floats
of dynamic shared memory (cuda/fchl_cuda_kernel.cu:1900) while the kernel carves ``8 * max_neighbours + nRs2 + nRs3 + 18``
floats out of it (:1347-1361), so the unpatched kernel writes 72 bytes past its allocation.  The fix adds the 18 floats
to the request; the kernel itself is unchanged.
"""
import os
import shutil
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, '_ref')

LIBS = {
    'ref_torchscript_fchl19': ['qml_lightning/cuda/torchscript/FCHL19.cpp', 'qml_lightning/cuda/fchl_cuda_kernel.cu',
                               'qml_lightning/cuda/pairlist_kernel.cu'],
    'ref_torchscript_sorf': ['qml_lightning/cuda/torchscript/SORF.cpp', 'qml_lightning/cuda/hadamard_kernel.cu'],
}
OLD = 'int shared_mem_size = nRs2 + nRs3 + 8 * max_neighbours;'
NEW = 'int shared_mem_size = nRs2 + nRs3 + 8 * max_neighbours + 18;'


def patch_backward_launcher(text):
    start = text.index('void FCHLBackwardsCuda(')
    pos = text.index(OLD, start)
    end = text.index('\nvoid ', start + 10)
    assert pos < end, 'the allocation to fix is not inside FCHLBackwardsCuda'
    return text[:pos] + NEW + text[pos + len(OLD):]


def main(upstream):
    os.environ.setdefault('TORCH_CUDA_ARCH_LIST', '10.0')
    from torch.utils import cpp_extension
    os.makedirs(OUT, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix='qml_ref_build_') as tmp:
        for name, sources in LIBS.items():
            local = []
            for rel in sources:
                dst = os.path.join(tmp, name + '_' + os.path.basename(rel))
                with open(os.path.join(upstream, rel)) as fh:
                    text = fh.read()
                if rel.endswith('fchl_cuda_kernel.cu'):
                    text = patch_backward_launcher(text)
                with open(dst, 'w') as fh:
                    fh.write(text)
                local.append(dst)
            build = os.path.join(tmp, 'build_' + name)
            os.makedirs(build)
            cpp_extension.load(name=name, sources=local, extra_cflags=['-O2'],
                               extra_cuda_cflags=['-O2', '-gencode', 'arch=compute_100a,code=sm_100a'], build_directory=build,
                               is_python_module=False, verbose=True)
            shutil.copyfile(os.path.join(build, name + '.so'), os.path.join(OUT, 'lib' + name + '.so'))
            print('built', os.path.join(OUT, 'lib' + name + '.so'))


if __name__ == '__main__':
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get('QML_LIGHTNING_UPSTREAM', os.path.join(os.path.dirname(os.path.dirname(HERE)), 'reference')))
