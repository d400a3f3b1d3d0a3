"""Seeded synthetic molecules and model parameters with the shapes of the benchmark configurations.

The upstream examples train on MD17 / QM9 / 3BPA, which are not available offline; these generators stand in for them:
random connected clusters with 1.0-1.6 Angstrom nearest-neighbour spacing, conformers as equilibrium plus Gaussian
jitter, Rademacher SORF diagonals, uniform phases and normal weights.  Everything is a pure function of the seed
(numpy ``default_rng``) so that every implementation reads identical inputs.
"""
import numpy as np

FCHL_DEFAULTS = dict(rcut=6.0, nRs2=24, nRs3=22, eta2=0.32, eta3=2.7, two_body_decay=1.8, three_body_decay=0.57,
                     three_body_weight=13.4)


def random_cluster(rng, natoms, dmin=1.0, dmax=1.5, min_sep=1.0):
    """Atom k sits at U(dmin,dmax) from a random earlier atom; rejected if closer than ``min_sep`` to any atom."""
    pos = np.zeros((natoms, 3))
    k = 1
    while k < natoms:
        parent = rng.integers(0, k)
        v = rng.normal(size=3)
        v /= np.linalg.norm(v)
        cand = pos[parent] + v * rng.uniform(dmin, dmax)
        if np.min(np.linalg.norm(pos[:k] - cand, axis=1)) >= min_sep:
            pos[k] = cand
            k += 1
    return pos


def conformers(seed, charges, nconf, jitter=0.05, dmax=1.5):
    """``nconf`` jittered copies of one seeded equilibrium geometry: X f32[nconf,A,3], Z f32[nconf,A], counts i32."""
    rng = np.random.default_rng(seed)
    charges = np.asarray(charges)
    eq = random_cluster(rng, len(charges), 1.0, dmax)
    X = eq[None] + rng.normal(0.0, jitter, size=(nconf, len(charges), 3))
    Z = np.tile(charges[None].astype(np.float32), (nconf, 1))
    counts = np.full(nconf, len(charges), dtype=np.int32)
    return X.astype(np.float32), Z, counts


def mixed_molecules(seed, nmol, min_atoms=4, max_atoms=29, species=(1, 6, 7, 8, 9), probs=(0.5, 0.3, 0.1, 0.08, 0.02)):
    """Zero-padded batch of random clusters with atom counts uniform in [min_atoms, max_atoms].

    Same construction as ``random_cluster`` (atom k at U(1.0,1.6) from a random earlier atom, rejected below 1.0 from
    any atom), vectorised over the molecules so that 200,000 molecules take seconds.
    """
    rng = np.random.default_rng(seed)
    counts = rng.integers(min_atoms, max_atoms + 1, size=nmol).astype(np.int32)
    X = np.zeros((nmol, max_atoms, 3), dtype=np.float64)
    Z = np.zeros((nmol, max_atoms), dtype=np.float32)
    for k in range(1, max_atoms):
        todo = np.where(counts > k)[0]
        while todo.size:
            parent = (rng.random(todo.size) * k).astype(np.int64)
            v = rng.normal(size=(todo.size, 3))
            v /= np.linalg.norm(v, axis=1, keepdims=True)
            cand = X[todo, parent] + v * rng.uniform(1.0, 1.6, size=(todo.size, 1))
            d = np.linalg.norm(X[todo, :k] - cand[:, None, :], axis=2).min(axis=1)
            ok = d >= 1.0
            X[todo[ok], k] = cand[ok]
            todo = todo[~ok]
    real = np.arange(max_atoms)[None, :] < counts[:, None]
    Z[real] = rng.choice(np.asarray(species, dtype=np.float32), size=int(real.sum()), p=probs)
    return X.astype(np.float32), Z, counts


def sorf_parameters(seed, nelements, npcas, nstacks, ntransforms=1):
    """Dmat f32[nel,T,S,N] (+-1), bias f32[nel,S*N] ~ U(0,2pi), alpha f32[S*N] ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    D = rng.integers(0, 2, size=(nelements, ntransforms, nstacks, npcas)).astype(np.float32) * 2.0 - 1.0
    bias = rng.uniform(0.0, 2.0 * np.pi, size=(nelements, nstacks * npcas)).astype(np.float32)
    alpha = rng.normal(size=nstacks * npcas).astype(np.float32)
    return D, bias, alpha


def rff_parameters(seed, nelements, npcas, nfeatures, sigma):
    """W f32[nel,npcas,D] ~ N(0, 1/sigma^2), b f32[nel,D] ~ U(0,2pi), alpha f32[D] ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    W = (rng.normal(size=(nelements, npcas, nfeatures)) / sigma).astype(np.float32)
    b = rng.uniform(0.0, 2.0 * np.pi, size=(nelements, nfeatures)).astype(np.float32)
    alpha = rng.normal(size=nfeatures).astype(np.float32)
    return W, b, alpha


def random_orthonormal_reductors(seed, nelements, repsize, npcas):
    """Orthonormal columns per element (stand-in for SVD reductors when no representation is at hand)."""
    rng = np.random.default_rng(seed)
    out = np.zeros((nelements, repsize, npcas), dtype=np.float32)
    for e in range(nelements):
        q, _ = np.linalg.qr(rng.normal(size=(repsize, npcas)))
        out[e] = q.astype(np.float32)
    return out


def svd_reductors(rep, Z, counts, elements, npcas, seed, nsample=512):
    """Per element: SVD of up to ``nsample`` random atom representations, first ``npcas`` left singular vectors
    (the rule of upstream representations/dimensionality_reduction.py:27-36).  ``rep`` f[nb,A,repsize] numpy."""
    rng = np.random.default_rng(seed)
    nb, A, repsize = rep.shape
    real = np.arange(A)[None, :] < counts[:, None]
    out = np.zeros((len(elements), repsize, npcas), dtype=np.float32)
    for ei, e in enumerate(elements):
        rows = rep[(Z == e) & real]
        if rows.shape[0] == 0:
            continue
        idx = rng.permutation(rows.shape[0])[:nsample]
        u, s, vt = np.linalg.svd(rows[idx].T.astype(np.float64), full_matrices=False)
        k = min(npcas, u.shape[1])
        out[ei, :, :k] = u[:, :k].astype(np.float32)
    return out


# Benchmark configurations (atom lists; conformer counts are arguments of the callers).
C0_CHARGES = [6, 6, 8, 1, 1, 1, 1, 1, 1]
C1_CHARGES = [6] * 9 + [1] * 8 + [8] * 4   # C9H8O4 composition
