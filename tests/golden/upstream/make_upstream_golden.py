"""Copies the upstream project's known-answer test into ``tests/golden/upstream/`` (test infrastructure).

    python tests/golden/upstream/make_upstream_golden.py [path of an upstream qml-lightning checkout]

Sources, both inside the upstream tree:

* ``unit_tests/models/saved_models/model_sorf.pt`` -- the TorchScript archive the upstream test loads; copied
  byte for byte to ``model_sorf.pt`` (it is loaded by ``torch.jit.load`` in the GPU tests, so it has to stay an
  archive).
* ``unit_tests/models/unit_test_sorf.py:11-80`` -- geometry, charges, expected total energy and expected forces as
  Python literals; parsed from the script's syntax tree (nothing is executed) and written to ``kat_literals.npz``.

The acceptance criteria of that script (``unit_test_sorf.py:100-101``) are restated in the tests that read these
files: ``np.isclose`` with default tolerances for the total energy, ``rtol = atol = 1e-4`` for every force component.
"""
import os
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, ROOT)

from oracle.kat_fixture import parse_unit_test  # noqa: E402


def main(upstream):
    shutil.copyfile(os.path.join(upstream, 'unit_tests/models/saved_models/model_sorf.pt'), os.path.join(HERE, 'model_sorf.pt'))
    u = parse_unit_test(os.path.join(upstream, 'unit_tests/models/unit_test_sorf.py'))
    np.savez(os.path.join(HERE, 'kat_literals.npz'), coordinates=np.asarray(u['coordinates'], dtype=np.float64),
             charges=np.asarray(u['charges'], dtype=np.int64), ref_energy=np.float64(u['ref_energy']),
             ref_forces=np.asarray(u['ref_forces'], dtype=np.float64))
    print('wrote', os.path.join(HERE, 'model_sorf.pt'), 'and', os.path.join(HERE, 'kat_literals.npz'))


if __name__ == '__main__':
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get('QML_LIGHTNING_UPSTREAM', os.path.join(os.path.dirname(ROOT), 'reference')))
