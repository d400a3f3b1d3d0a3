"""Shared builders for the parity tests: seeded inputs, oracle models and their CUDA twins."""
import math

import numpy as np
import torch

from oracle import FCHLParams, fchl19_representation
from qml_lightning_b200.utils import synthetic as syn


def fchl_params(species, **over):
    kw = dict(syn.FCHL_DEFAULTS)
    kw.update(over)
    return FCHLParams(species=list(species), **kw)


def kernel_params(p, device):
    """CUDA-side twin of an oracle FCHLParams."""
    from qml_lightning_b200.cabi import FchlKernelParams
    return FchlKernelParams(torch.tensor(p.species, dtype=torch.float32, device=device), p.Rs2.to(device), p.Rs3.to(device),
                            p.eta2, p.eta3, p.two_body_decay, p.w3, p.three_body_decay, p.rcut)


def batch_c0(nconf, seed=1000):
    X, Z, c = syn.conformers(seed, syn.C0_CHARGES, nconf)
    return torch.from_numpy(X), torch.from_numpy(Z), torch.from_numpy(c), [1, 6, 8]


def batch_c1(nconf, seed=1001):
    X, Z, c = syn.conformers(seed, syn.C1_CHARGES, nconf)
    return torch.from_numpy(X), torch.from_numpy(Z), torch.from_numpy(c), [1, 6, 8]


def batch_mixed(nmol, seed=1002, max_atoms=29):
    X, Z, c = syn.mixed_molecules(seed, nmol, max_atoms=max_atoms)
    return torch.from_numpy(X), torch.from_numpy(Z), torch.from_numpy(c), [1, 6, 7, 8, 9]


def sorf_model(X, Z, counts, p, elements, npcas, nstacks, ntransforms=1, sigma=2.0, seed=7):
    """Oracle-side model dict with SVD reductors computed from the oracle representation of the batch."""
    rep = fchl19_representation(X.double(), Z, counts, p).numpy()
    red = syn.svd_reductors(rep, Z.numpy(), counts.numpy(), elements, npcas, seed)
    D, bias, alpha = syn.sorf_parameters(seed + 1, len(elements), npcas, nstacks, ntransforms)
    return dict(kind='sorf', elements=list(elements), reductors=torch.from_numpy(red), Dmat=torch.from_numpy(D),
                bias=torch.from_numpy(bias), alpha=torch.from_numpy(alpha), sigma=sigma, ntransforms=ntransforms)


def rff_model(X, Z, counts, p, elements, npcas, nfeatures, sigma=2.0, seed=9):
    rep = fchl19_representation(X.double(), Z, counts, p).numpy()
    red = syn.svd_reductors(rep, Z.numpy(), counts.numpy(), elements, npcas, seed)
    W, b, alpha = syn.rff_parameters(seed + 1, len(elements), npcas, nfeatures, sigma)
    return dict(kind='rff', elements=list(elements), reductors=torch.from_numpy(red), W=torch.from_numpy(W),
                b=torch.from_numpy(b), alpha=torch.from_numpy(alpha))


def energy_tolerance(E_ref):
    """1e-5 relative, with the batch RMS as the floor for molecules whose energy is near zero."""
    rms = float(torch.sqrt(torch.mean(E_ref.double() ** 2)))
    return 1e-5 * torch.clamp(E_ref.double().abs(), min=rms)
