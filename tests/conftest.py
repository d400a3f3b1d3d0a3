import importlib.util
import os
import shutil
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# a checkout of the upstream project, when there is one: QML_LIGHTNING_UPSTREAM, else a `reference` directory beside this repository
UPSTREAM = os.environ.get('QML_LIGHTNING_UPSTREAM', os.path.join(os.path.dirname(ROOT), 'reference'))


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on the B200 box)')


def _ensure_built():
    """Build the shared libraries when a compiler is at hand and they are missing or stale (cached by mtime)."""
    if shutil.which('nvcc') is None and not os.path.exists('/usr/local/cuda/bin/nvcc'):
        return
    spec = importlib.util.spec_from_file_location('qmlb200_build', os.path.join(ROOT, 'qml_lightning_b200', 'build.py'))
    b = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(b)
    b.build_native(verbose=False)
    b.build_torch_ops(verbose=False)


_ensure_built()


@pytest.fixture(scope='session')
def upstream_dir():
    """Path of an upstream qml-lightning checkout, or skip when there is none."""
    if not os.path.isdir(os.path.join(UPSTREAM, 'unit_tests')):
        pytest.skip('no upstream checkout available')
    return UPSTREAM
