"""Torch-CPU restatement of the upstream CUDA arithmetic (test infrastructure).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this module.  Every function works on CPU tensors, is
differentiable with respect to the coordinates (forces come from
``torch.autograd.grad``) and runs in the dtype of the coordinates it is given
(float64 for parity checks, float32 for the timed CPU baseline).

Upstream files restated here (paths inside the upstream project):
  qml_lightning/representations/FCHL.py:18-46        grids, three-body weight scaling
  qml_lightning/cuda/fchl_cuda_kernel.cu:1716-1742   element index = position in ``species``
  qml_lightning/cuda/pairlist_kernel.cu:372-390      neighbour rule 0 < r^2 < rcut^2
  qml_lightning/cuda/fchl_cuda_kernel.cu:476-674     two-body and three-body terms
  qml_lightning/cuda/fchl_cuda_kernel.cu:16-49 and
  qml_lightning/cuda/pairlist_kernel.cu:6-39         minimum-image convention of periodic cells
  qml_lightning/representations/dimensionality_reduction.py:47-58   PCA projection
  qml_lightning/cuda/hadamard_kernel.cu:5-102        [HD]^T transform, 2^(-log2N/2) per H
  qml_lightning/cuda/hadamard_kernel.cu:778-800      cos features, sqrt(2/F), per-molecule sum
  qml_lightning/models/hadamard_features.py:82-123   SORF model forward (assembly, E = Z.alpha)
  qml_lightning/models/random_features.py:69-102     RFF model forward
  qml_lightning/cuda/hadamard_kernel.cu:565-717 and
  qml_lightning/models/kernel.py:119-124,164-170     training rows: G = -dZ/dr
  qml_lightning/cuda/utils_kernel.cu:70-129 and
  qml_lightning/models/kernel.py:176-188             float32 Kahan product accumulated in float64
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch


@dataclass
class FCHLParams:
    """Constructor-level FCHL19 hyper-parameters (FCHL.py:18-19)."""

    species: Sequence[int] = (1, 6, 7, 8)
    rcut: float = 6.0
    nRs2: int = 24
    nRs3: int = 20
    eta2: float = 0.32
    eta3: float = 2.7
    two_body_decay: float = 1.8
    three_body_weight: float = 13.4
    three_body_decay: float = 0.57
    # When set, used verbatim as the kernel-level weight (a saved model stores
    # the already scaled value); otherwise FCHL.py:35 scaling is applied.
    scaled_three_body_weight: Optional[float] = None
    Rs2: Optional[torch.Tensor] = field(default=None, repr=False)
    Rs3: Optional[torch.Tensor] = field(default=None, repr=False)

    def __post_init__(self):
        # FCHL.py:39-40 -- float32 linspace without the first (zero) point.
        if self.Rs2 is None:
            self.Rs2 = torch.linspace(0.0, float(self.rcut), self.nRs2 + 1, dtype=torch.float32)[1:]
        if self.Rs3 is None:
            self.Rs3 = torch.linspace(0.0, float(self.rcut), self.nRs3 + 1, dtype=torch.float32)[1:]

    @property
    def nspecies(self) -> int:
        return len(self.species)

    @property
    def repsize(self) -> int:
        n = self.nspecies
        return n * self.nRs2 + n * (n + 1) * self.nRs3  # FCHL.py:42

    @property
    def w3(self) -> float:
        if self.scaled_three_body_weight is not None:
            return float(self.scaled_three_body_weight)
        return math.sqrt(self.eta3 / math.pi) * self.three_body_weight  # FCHL.py:35


def element_types(Z: torch.Tensor, species: Sequence[int]) -> torch.Tensor:
    """Index of each charge in ``species`` (-1 if absent); fchl_cuda_kernel.cu:1716-1742."""
    et = torch.full(Z.shape, -1, dtype=torch.long)
    for idx, s in enumerate(species):
        et = torch.where(Z.round().long() == int(s), torch.full_like(et, idx), et)
    return et


def minimum_image(d, cell, inv_cell):
    """get_pbc_drij (fchl_cuda_kernel.cu:16-49, pairlist_kernel.cu:6-39): ``s = inv_cell . d``, ``s -= round(s)``,
    ``d = cell . s`` with the row-major 3x3 matrices of each molecule; ``d [nb, ..., 3]``, ``cell [nb,3,3]``."""
    shape = d.shape
    flat = d.reshape(shape[0], -1, 3)
    s = torch.einsum('bmk,bnk->bnm', inv_cell.to(d.dtype), flat)
    s = s - torch.round(s)
    return torch.einsum('bmk,bnk->bnm', cell.to(d.dtype), s).reshape(shape)


def _fchl_chunk(X, Z, counts, p: FCHLParams, cell=None, inv_cell=None):
    nb, A, _ = X.shape
    dt = X.dtype
    nel = p.nspecies
    nRs2, nRs3 = p.nRs2, p.nRs3
    Rs2 = p.Rs2.to(dt)
    Rs3 = p.Rs3.to(dt)
    pi = math.pi

    ar = torch.arange(A)
    real = ar[None, :] < counts[:, None].long()                    # [nb,A]
    et = element_types(Z, p.species)
    known = real & (et >= 0)

    d = X[:, :, None, :] - X[:, None, :, :]                         # d[b,a,c] = r_a - r_c
    if cell is not None:
        d = minimum_image(d, cell, inv_cell)                        # :375-377, :414-416 (every r_i - r_j, r_i - r_k)
    r2 = (d * d).sum(-1)
    offdiag = ar[:, None] != ar[None, :]
    pair_ok = known[:, :, None] & known[:, None, :] & offdiag[None]
    # neighbour rule of pairlist_kernel.cu:386: 0 < r^2 < rcut^2
    nbr = pair_ok & (r2 > 0) & (r2 < p.rcut * p.rcut)
    r2s = torch.where(pair_ok, r2, torch.ones_like(r2))             # safe for sqrt / division
    r = torch.sqrt(r2s)

    fc = 0.5 * (torch.cos(pi * r / p.rcut) + 1.0)                   # get_cutoff, :57

    # ---- two-body, fchl_cuda_kernel.cu:586-603
    scaling = r ** (-p.two_body_decay)
    sig2 = torch.log(1.0 + p.eta2 / r2s)
    mu = torch.log(r / torch.sqrt(1.0 + p.eta2 / r2s))
    sig = torch.sqrt(sig2)
    radial2 = (1.0 / (sig[..., None] * math.sqrt(2.0 * pi) * Rs2)
               * torch.exp(-(torch.log(Rs2) - mu[..., None]) ** 2 / (2.0 * sig2[..., None]))
               * (scaling * fc)[..., None])
    radial2 = torch.where(nbr[..., None], radial2, torch.zeros_like(radial2))
    onehot = (et[:, :, None] == torch.arange(nel)[None, None, :]).to(dt)      # [nb,A,nel] (neighbour j)
    rep2 = torch.einsum('bje,bijz->biez', onehot, radial2).reshape(nb, A, nel * nRs2)

    # ---- three-body, fchl_cuda_kernel.cu:605-672 (pairs j<k of the neighbour list of i)
    tri = nbr[:, :, :, None] & nbr[:, :, None, :] & (ar[:, None] < ar[None, :])[None, None]
    # the third side of a triplet is the difference of the two (minimum-image) vectors from the centre atom,
    # drjk = drik - drij = r_j - r_k (:617-619); without a cell this is r[b,j,k]
    vjk = d[:, :, None, :, :] - d[:, :, :, None, :]                 # [b,i,j,k,:]
    rjk2 = (vjk * vjk).sum(-1)
    rjk = torch.sqrt(torch.where(tri, rjk2, torch.ones_like(rjk2)))
    dots_i = torch.einsum('bijx,bikx->bijk', d, d)                  # (ri-rj).(ri-rk)
    dots_j = -torch.einsum('bijx,bijkx->bijk', d, vjk)              # (ri-rj).(rk-rj): angle at j (:649)
    dots_k = torch.einsum('bikx,bijkx->bijk', d, vjk)               # (ri-rk).(rj-rk): angle at k (:647)
    rij = r[:, :, :, None]
    rik = r[:, :, None, :]
    one = torch.ones_like(dots_i)
    zero = torch.zeros_like(dots_i)
    cos_i = torch.where(tri, dots_i / (rij * rik), zero)
    cos_j = torch.where(tri, dots_j / (rij * rjk), zero)
    cos_k = torch.where(tri, dots_k / (rik * rjk), zero)
    theta = torch.acos(torch.clamp(cos_i, -1.0, 1.0))               # calc_angle_abcb, :251-262
    rprod = torch.where(tri, rij * rik * rjk, one)
    ksi3 = p.w3 * (1.0 + 3.0 * cos_i * cos_j * cos_k) / rprod ** p.three_body_decay
    zeta2 = 2.0 * math.exp(-pi * pi * 0.5)
    amp = ksi3 * fc[:, :, :, None] * fc[:, :, None, :]
    amp = torch.where(tri, amp, zero)
    a_cos = zeta2 * torch.cos(theta) * amp
    a_sin = zeta2 * torch.sin(theta) * amp
    rbar = 0.5 * (rij + rik)
    radial3 = torch.exp(-p.eta3 * (rbar[..., None] - Rs3) ** 2)      # [nb,A,A,A,nRs3]
    etj = et[:, :, None].clamp(min=0)
    etk = et[:, None, :].clamp(min=0)
    pp = torch.minimum(etj, etk)
    qq = torch.maximum(etj, etk)
    ptype = qq + nel * pp - (pp * (pp + 1)) // 2                     # :661
    npt = nel * (nel + 1) // 2
    pt_onehot = (ptype[..., None] == torch.arange(npt)).to(dt)       # [nb,A(j),A(k),npt]
    rc = torch.einsum('bjkp,bijk,bijkl->bipl', pt_onehot, a_cos, radial3)
    rs = torch.einsum('bjkp,bijk,bijkl->bipl', pt_onehot, a_sin, radial3)
    rep3 = torch.stack((rc, rs), dim=-1).reshape(nb, A, npt * nRs3 * 2)

    rep = torch.cat((rep2, rep3), dim=-1)
    return torch.where(known[..., None], rep, torch.zeros_like(rep))


def fchl19_representation(X: torch.Tensor, Z: torch.Tensor, atom_counts: torch.Tensor, p: FCHLParams,
                          chunk: Optional[int] = None, cell: Optional[torch.Tensor] = None,
                          inv_cell: Optional[torch.Tensor] = None) -> torch.Tensor:
    """FCHL19 representation ``[nb, A, repsize]``; padded atoms are zero rows.

    Restates fchl19_representation_cuda (fchl_cuda_kernel.cu:476-674) with the
    neighbour rule of pairlist_kernel.cu:372-390.  ``cell`` / ``inv_cell``
    ``[nb,3,3]`` switch on the minimum-image convention (an atom sees at most one
    image of every other atom and never its own images, as upstream).
    """
    nb, A, _ = X.shape
    if cell is not None and cell.numel() == 0:
        cell = inv_cell = None
    if chunk is None:
        per_mol = max(1, A * A * A * p.nRs3 * 6)
        chunk = max(1, int(6e7 // per_mol))
    out = []
    for s in range(0, nb, chunk):
        out.append(_fchl_chunk(X[s:s + chunk], Z[s:s + chunk], atom_counts[s:s + chunk], p,
                               None if cell is None else cell[s:s + chunk],
                               None if cell is None else inv_cell[s:s + chunk]))
    return torch.cat(out, dim=0) if out else X.new_zeros((0, A, p.repsize))


def neighbour_lists(X, atom_counts, rcut, cell=None, inv_cell=None):
    """``(counts i64[nb,A], lists: nb x A python lists)``: neighbours j != i with 0 < r^2 < rcut^2 in ascending j
    (pairlist_kernel.cu:145-224, 326-391), minimum image when a cell is given."""
    nb, A, _ = X.shape
    d = X[:, :, None, :] - X[:, None, :, :]
    if cell is not None and cell.numel():
        d = minimum_image(d, cell, inv_cell)
    r2 = (d * d).sum(-1)
    ar = torch.arange(A)
    real = ar[None, :] < atom_counts[:, None].long()
    ok = real[:, :, None] & real[:, None, :] & (ar[:, None] != ar[None, :])[None] & (r2 > 0) & (r2 < rcut * rcut)
    lists = [[torch.where(ok[b, i])[0].tolist() for i in range(A)] for b in range(nb)]
    return ok.sum(-1), lists


def fwht(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Walsh-Hadamard transform (Sylvester order) of the last axis.

    Any butterfly order yields the same matrix as hadamard_kernel.cu:32-83.
    """
    N = x.shape[-1]
    assert N & (N - 1) == 0 and N > 0, "length must be a power of two"
    lead = x.shape[:-1]
    h = 1
    while h < N:
        x = x.reshape(*lead, N // (2 * h), 2, h)
        a = x[..., 0, :]
        b = x[..., 1, :]
        x = torch.stack((a + b, a - b), dim=-2)
        h *= 2
    return x.reshape(*lead, N)


def sorf_coefficients(x: torch.Tensor, D: torch.Tensor, coeff_normalisation: float, ntransforms: int) -> torch.Tensor:
    """``[n,N] , [T,S,N] -> [n,S,N]``; hadamard_kernel.cu:5-102."""
    n, N = x.shape
    S = D.shape[1]
    normh = 1.0 / math.sqrt(N)
    u = x[:, None, :].expand(n, S, N)
    for m in range(ntransforms):
        u = fwht(u * D[m][None].to(x.dtype)) * normh
    return coeff_normalisation * u


def _element_masks(Z, counts, elements):
    A = Z.shape[1]
    real = torch.arange(A)[None, :] < counts[:, None].long()
    for ei, e in enumerate(elements):
        mask = (Z.round().long() == int(e)) & real
        yield ei, mask


def sorf_energy(rep, Z, counts, elements, reductors, Dmat, bias, alpha, sigma, ntransforms):
    """Model energies ``[nb]`` from a representation; hadamard_features.py:82-123."""
    dt = rep.dtype
    nb = rep.shape[0]
    N = reductors.shape[-1]
    S = Dmat.shape[2]
    F = N * S
    Zf = rep.new_zeros((nb, F))
    coeff_norm = math.sqrt(N) / sigma                                 # hadamard_features.py:93
    for ei, mask in _element_masks(Z, counts, elements):
        mol = torch.where(mask)[0]
        if mol.numel() == 0:
            continue
        sub = rep[mask] @ reductors[ei].to(dt)                        # dimensionality_reduction.py:58
        c = sorf_coefficients(sub, Dmat[ei], coeff_norm, ntransforms).reshape(-1, F)
        feat = math.sqrt(2.0 / F) * torch.cos(c + bias[ei].to(dt))    # hadamard_kernel.cu:795-798
        Zf = Zf.index_add(0, mol, feat)
    return Zf @ alpha.to(dt), Zf


def rff_energy(rep, Z, counts, elements, reductors, W, b, alpha):
    """RFF model energies; random_features.py:69-102 (feature_normalisation = sqrt(2/D))."""
    dt = rep.dtype
    nb = rep.shape[0]
    Dn = W.shape[-1]
    Zf = rep.new_zeros((nb, Dn))
    for ei, mask in _element_masks(Z, counts, elements):
        mol = torch.where(mask)[0]
        if mol.numel() == 0:
            continue
        sub = rep[mask] @ reductors[ei].to(dt)
        feat = math.sqrt(2.0 / Dn) * torch.cos(sub @ W[ei].to(dt) + b[ei].to(dt)[None, :])
        Zf = Zf.index_add(0, mol, feat)
    return Zf @ alpha.to(dt), Zf


def energy_and_forces(X, Z, counts, p: FCHLParams, model: dict, batch: int = 64, forces: bool = True,
                      dtype=torch.float64, cell=None, inv_cell=None):
    """Energies ``[nb]`` and forces ``-dE/dX`` ``[nb,A,3]`` in host batches.

    ``model`` holds ``kind`` ('sorf' | 'rff'), ``elements``, ``reductors`` and
    either (``Dmat``, ``bias``, ``sigma``, ``ntransforms``) or (``W``, ``b``),
    plus ``alpha``.  Mirrors predict_opt (hadamard_features.py:125-179): forces
    are ``autograd.grad(-E.sum(), X)``.
    """
    nb = X.shape[0]
    Es, Fs = [], []
    for s in range(0, nb, batch):
        x = X[s:s + batch].to(dtype).clone().requires_grad_(forces)
        z = Z[s:s + batch]
        c = counts[s:s + batch]
        rep = fchl19_representation(x, z, c, p, cell=None if cell is None else cell[s:s + batch],
                                    inv_cell=None if cell is None else inv_cell[s:s + batch])
        if model['kind'] == 'sorf':
            E, _ = sorf_energy(rep, z, c, model['elements'], model['reductors'], model['Dmat'], model['bias'],
                               model['alpha'], model['sigma'], model['ntransforms'])
        else:
            E, _ = rff_energy(rep, z, c, model['elements'], model['reductors'], model['W'], model['b'],
                              model['alpha'])
        if forces:
            g, = torch.autograd.grad(-E.sum(), x)
            Fs.append(g.detach())
        Es.append(E.detach())
    E = torch.cat(Es)
    return (E, torch.cat(Fs)) if forces else E


def training_rows(X, Z, counts, p: FCHLParams, model: dict, dtype=torch.float64, cell=None, inv_cell=None):
    """Training rows for small cases: ``Zrows [nb,F]`` and ``G [nb,A,3,F] = -dZ/dr``.

    kernel.py:134-170 builds exactly these (energy rows, then one row per atom
    and axis); the sign follows compute_sin_coeffs_kernel (hadamard_kernel.cu:565-585),
    i.e. G already is the force feature.  One autograd pass per feature, so use
    only with a few hundred features.
    """
    x = X.to(dtype).clone().requires_grad_(True)
    rep = fchl19_representation(x, Z, counts, p, cell=cell, inv_cell=inv_cell)
    if model['kind'] == 'sorf':
        _, Zf = sorf_energy(rep, Z, counts, model['elements'], model['reductors'], model['Dmat'], model['bias'],
                            torch.zeros(model['Dmat'].shape[2] * model['reductors'].shape[-1]), model['sigma'],
                            model['ntransforms'])
    else:
        _, Zf = rff_energy(rep, Z, counts, model['elements'], model['reductors'], model['W'], model['b'],
                           torch.zeros(model['W'].shape[-1]))
    nb, F = Zf.shape
    G = torch.zeros(nb, X.shape[1], 3, F, dtype=dtype)
    for f in range(F):
        g, = torch.autograd.grad(Zf[:, f].sum(), x, retain_graph=True)
        G[..., f] = -g
    return Zf.detach(), G


def kahan_gram(M: torch.Tensor) -> torch.Tensor:
    """``M^T M`` the way ``use_specialized_matmul`` computes it upstream: build_Z_components passes
    ``Ztrain.float().T`` and ``Ztrain.float()`` (kernel.py:176-188) to matmul_and_reduce_kernel
    (utils_kernel.cu:70-129), which forms every entry as a Kahan-compensated float32 sum over the rows, each term
    entering through ``fma(a, b, -c)``, and adds ``(double) sum`` to the float64 matrix.  Returned as float64
    ``[F, F]`` (the contribution of one row block).  The fma is restated as a float64 product (exact for float32
    factors) minus ``c``, rounded once to float32."""
    import numpy as np
    A = M.to(torch.float32).double().numpy()
    F = A.shape[1]
    total = np.zeros((F, F), dtype=np.float32)
    c = np.zeros((F, F), dtype=np.float32)
    for k in range(A.shape[0]):
        y = (np.outer(A[k], A[k]) - c.astype(np.float64)).astype(np.float32)
        t = total + y
        c = (t - total) - y
        total = t
    return torch.from_numpy(total.astype(np.float64))
