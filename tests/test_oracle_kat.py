"""Pins the CPU oracle against the upstream project's own known-answer test.

The model tensors come from upstream's TorchScript fixture and the geometry, charges and expected values from the
literals of upstream's script (unit_tests/models/unit_test_sorf.py:11-80), both committed under
tests/golden/upstream/ by tests/golden/upstream/make_upstream_golden.py; the acceptance criteria are the script's own
(unit_test_sorf.py:100-101).  Where an upstream checkout is present the committed copies are compared with it.
"""
import filecmp
import os

import numpy as np
import torch

from oracle import FCHLParams, energy_and_forces
from oracle.kat_fixture import load_torchscript_tensors, parse_unit_test

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'upstream')
ARCHIVE = os.path.join(GOLDEN, 'model_sorf.pt')


def load_kat():
    t = load_torchscript_tensors(ARCHIVE)
    u = dict(np.load(os.path.join(GOLDEN, 'kat_literals.npz')))
    p = FCHLParams(species=[int(s) for s in t['rep.species']], rcut=float(t['rep.rcut']), nRs2=int(t['rep.nRs2']),
                   nRs3=int(t['rep.nRs3']), eta2=float(t['rep.eta2']), eta3=float(t['rep.eta3']),
                   two_body_decay=float(t['rep.two_body_decay']), three_body_decay=float(t['rep.three_body_decay']),
                   scaled_three_body_weight=float(t['rep.three_body_weight']), Rs2=t['rep.Rs2'], Rs3=t['rep.Rs3'])
    model = dict(kind='sorf', elements=[int(e) for e in t['elements']], reductors=t['reductors'], Dmat=t['Dmat'],
                 bias=t['bias'], alpha=t['alpha'], sigma=float(t['sigma']), ntransforms=int(t['ntransforms']))
    X = torch.tensor(u['coordinates'], dtype=torch.float32)[None]
    Z = torch.tensor(u['charges'], dtype=torch.float32)[None]
    counts = torch.tensor([X.shape[1]], dtype=torch.int32)
    return t, u, p, model, X, Z, counts


def test_committed_fixture_is_upstreams(upstream_dir):
    """The committed copies are what an upstream checkout holds (skipped where there is none)."""
    assert filecmp.cmp(ARCHIVE, os.path.join(upstream_dir, 'unit_tests/models/saved_models/model_sorf.pt'), shallow=False)
    lit = parse_unit_test(os.path.join(upstream_dir, 'unit_tests/models/unit_test_sorf.py'))
    u = np.load(os.path.join(GOLDEN, 'kat_literals.npz'))
    for k in ('coordinates', 'charges', 'ref_forces'):
        assert np.array_equal(np.asarray(lit[k]), u[k])
    assert float(lit['ref_energy']) == float(u['ref_energy'])


def test_fixture_shapes():
    t, u, p, model, X, Z, counts = load_kat()
    assert p.repsize == 336 == int(t['rep.fp_size'])
    assert tuple(t['reductors'].shape) == (3, 336, 128)
    assert tuple(t['Dmat'].shape) == (3, 1, 128, 128)
    assert set(torch.unique(t['Dmat']).tolist()) == {-1.0, 1.0}
    assert X.shape == (1, 21, 3)


def test_oracle_reproduces_upstream_known_answer():
    t, u, p, model, X, Z, counts = load_kat()
    E, F = energy_and_forces(X, Z, counts, p, model, dtype=torch.float64)
    total = E.item() + t['self_energy'][Z.long()].sum().item()
    # unit_test_sorf.py:100 -- np.isclose with default rtol/atol
    assert np.isclose(u['ref_energy'], total)
    # unit_test_sorf.py:101
    assert np.isclose(u['ref_forces'], F[0].numpy(), rtol=1e-4, atol=1e-4).all()
