"""Generates the committed golden vectors from the float64 CPU oracle.

    python tests/golden/make_golden.py

Writes ``tests/golden/sorf_small.npz``: seeded inputs (a 9-atom conformer batch and a mixed 4-12 atom batch, small
model) and the oracle's representation, energies and forces; and ``tests/golden/rff_small.npz``: a 9-atom batch with
an RFF model, its energies, forces and float64 training rows.  The oracle itself is pinned to the upstream project's
known-answer fixture by tests/test_oracle_kat.py; these vectors make that pin travel to machines without an upstream
checkout.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import energy_and_forces, fchl19_representation, training_rows  # noqa: E402
from tests import helpers as H  # noqa: E402


def case(name, X, Z, c, species, npcas, nstacks, T):
    p = H.fchl_params(species)
    model = H.sorf_model(X, Z, c, p, species, npcas, nstacks, T)
    rep = fchl19_representation(X.double(), Z, c, p)
    E, F = energy_and_forces(X, Z, c, p, model, dtype=torch.float64)
    out = {'X': X.numpy(), 'Z': Z.numpy(), 'counts': c.numpy(), 'species': np.array(species), 'npcas': npcas,
           'nstacks': nstacks, 'ntransforms': T, 'sigma': model['sigma'], 'reductors': model['reductors'].numpy(),
           'Dmat': model['Dmat'].numpy(), 'bias': model['bias'].numpy(), 'alpha': model['alpha'].numpy(),
           'rep': rep.numpy().astype(np.float64), 'E': E.numpy(), 'F': F.numpy()}
    return {f'{name}_{k}': v for k, v in out.items()}


def rff_case(name, X, Z, c, species, npcas, nfeatures):
    """RFF model: energies, forces and the float64 training rows (Z and G = -dZ/dr)."""
    p = H.fchl_params(species)
    model = H.rff_model(X, Z, c, p, species, npcas, nfeatures)
    E, F = energy_and_forces(X, Z, c, p, model, dtype=torch.float64)
    Zrows, Grows = training_rows(X, Z, c, p, model)
    out = {'X': X.numpy(), 'Z': Z.numpy(), 'counts': c.numpy(), 'species': np.array(species), 'npcas': npcas,
           'nfeatures': nfeatures, 'reductors': model['reductors'].numpy(), 'W': model['W'].numpy(), 'b': model['b'].numpy(),
           'alpha': model['alpha'].numpy(), 'E': E.numpy(), 'F': F.numpy(), 'Zrows': Zrows.numpy(), 'Grows': Grows.numpy()}
    return {f'{name}_{k}': v for k, v in out.items()}


def main():
    X, Z, c, species = H.batch_c0(5, seed=4244)
    rff = rff_case('c0', X, Z, c, species, 32, 96)
    path = os.path.join(ROOT, 'tests', 'golden', 'rff_small.npz')
    np.savez_compressed(path, **rff)
    print('wrote', path, os.path.getsize(path), 'bytes')
    data = {}
    X, Z, c, species = H.batch_c0(6, seed=4242)
    data.update(case('c0', X, Z, c, species, 32, 4, 1))
    X, Z, c, species = H.batch_mixed(6, seed=4243, max_atoms=12)
    data.update(case('mixed', X, Z, c, species, 16, 4, 2))
    path = os.path.join(ROOT, 'tests', 'golden', 'sorf_small.npz')
    np.savez_compressed(path, **data)
    print('wrote', path, os.path.getsize(path), 'bytes')


if __name__ == '__main__':
    main()
