import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

UPSTREAM = os.environ.get('QML_LIGHTNING_UPSTREAM', '/root/reference')


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run on the B200 box)')


@pytest.fixture(scope='session')
def upstream_dir():
    """Path of an upstream qml-lightning checkout, or skip when there is none."""
    if not os.path.isdir(os.path.join(UPSTREAM, 'unit_tests')):
        pytest.skip('no upstream checkout available')
    return UPSTREAM
