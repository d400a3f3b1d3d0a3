"""Periodic boundary conditions: every FCHL19 entry point and the whole prediction path against the float64 oracle on
cells small enough that atoms see each other through the cell faces (minimum image of upstream
cuda/fchl_cuda_kernel.cu:16-49 and cuda/pairlist_kernel.cu:6-39), cubic and skewed."""
import numpy as np
import pytest
import torch

from oracle import energy_and_forces, fchl19_representation, neighbour_lists
from tests import helpers as H

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'
RCUT = 3.0


def periodic_batch(seed, nb=5, natoms=14, skew=False):
    """Random atoms (pairwise minimum-image distance >= 0.9) in cells whose perpendicular widths exceed 2 rcut; about half of
    the atoms are then moved by whole lattice vectors so that the stored coordinates lie outside the cell."""
    rng = np.random.default_rng(seed)
    species = [1, 6, 8]
    X = np.zeros((nb, natoms, 3), dtype=np.float32)
    Z = np.zeros((nb, natoms), dtype=np.float32)
    counts = np.zeros(nb, dtype=np.int32)
    cells = np.zeros((nb, 3, 3), dtype=np.float32)
    for b in range(nb):
        edge = rng.uniform(6.3, 7.0, size=3)
        h = np.diag(edge)
        if skew:
            h[0, 1], h[0, 2], h[1, 2] = rng.uniform(-1.2, 1.2, size=3)      # columns are the lattice vectors
        hinv = np.linalg.inv(h)
        n = natoms - (b % 3)
        pts = []
        while len(pts) < n:
            s = rng.uniform(0, 1, size=3)
            r = h @ s
            ok = True
            for q in pts:
                ds = hinv @ (r - q)
                ds -= np.round(ds)
                if np.linalg.norm(h @ ds) < 0.9:
                    ok = False
                    break
            if ok:
                pts.append(r)
        pts = np.array(pts)
        shift = rng.integers(-1, 2, size=(n, 3)) * (rng.uniform(size=(n, 1)) < 0.5)
        pts = pts + shift @ h.T
        X[b, :n] = pts
        Z[b, :n] = rng.choice(species, size=n, p=[0.5, 0.3, 0.2])
        counts[b] = n
        cells[b] = h
    inv = np.linalg.inv(cells.astype(np.float64)).astype(np.float32)
    return (torch.from_numpy(X), torch.from_numpy(Z), torch.from_numpy(counts), species, torch.from_numpy(cells),
            torch.from_numpy(inv))


@pytest.fixture(scope='module')
def cabi():
    from qml_lightning_b200 import cabi
    return cabi


@pytest.mark.parametrize('skew', [False, True])
def test_periodic_neighbour_lists(cabi, skew):
    X, Z, c, species, cell, inv = periodic_batch(11, skew=skew)
    cnt_ref, lists = neighbour_lists(X.double(), c, RCUT, cell.double(), inv.double())
    free_ref, _ = neighbour_lists(X.double(), c, RCUT)
    assert (cnt_ref > free_ref).any()                        # the cell does add neighbours through its faces
    nn = cabi.num_neighbours(X.to(DEV), c.to(DEV), RCUT, cell.to(DEV), inv.to(DEV)).cpu()
    assert torch.equal(nn.long(), cnt_ref)
    nl = cabi.neighbour_list(X.to(DEV), c.to(DEV), int(nn.max()), RCUT, cell.to(DEV), inv.to(DEV)).cpu()
    for m in range(X.shape[0]):
        for i in range(int(c[m])):
            want = lists[m][i]
            assert nl[m, i, :len(want)].tolist() == want
            assert (nl[m, i, len(want):] == -1).all()


@pytest.mark.parametrize('skew', [False, True])
def test_periodic_forward_and_vjp(cabi, skew):
    X, Z, c, species, cell, inv = periodic_batch(12, skew=skew)
    p = H.fchl_params(species, rcut=RCUT)
    kp = H.kernel_params(p, DEV)
    x = X.double().clone().requires_grad_(True)
    ref = fchl19_representation(x, Z, c, p, cell=cell.double(), inv_cell=inv.double())
    free = fchl19_representation(X.double(), Z, c, p)
    assert (ref.detach() - free).abs().max() > 1e-2 * ref.detach().abs().max()      # the images matter in this case
    rep = cabi.fchl19_forward(X.to(DEV), Z.to(DEV), c.to(DEV), kp, cell.to(DEV), inv.to(DEV)).cpu().double()
    assert (rep - ref.detach()).abs().max() <= 2e-6 * ref.detach().abs().max()
    g = torch.from_numpy(np.random.default_rng(3).normal(size=tuple(ref.shape))).double() * 0.1
    gX_ref, = torch.autograd.grad((ref * g).sum(), x)
    gX = cabi.fchl19_backward(X.to(DEV), Z.to(DEV), c.to(DEV), kp, g.float().to(DEV), cell.to(DEV), inv.to(DEV)).cpu().double()
    assert (gX - gX_ref).abs().max() <= 2e-5 * gX_ref.abs().max()


def test_periodic_jacobian(cabi):
    X, Z, c, species, cell, inv = periodic_batch(13, nb=2, natoms=9, skew=True)
    p = H.fchl_params(species, rcut=RCUT, nRs2=6, nRs3=5)
    kp = H.kernel_params(p, DEV)
    rep, jac = cabi.fchl19_forward_jacobian(X.to(DEV), Z.to(DEV), c.to(DEV), kp, cell.to(DEV), inv.to(DEV))
    rep, jac = rep.cpu().double(), jac.cpu().double()
    x = X.double().clone().requires_grad_(True)
    ref = fchl19_representation(x, Z, c, p, cell=cell.double(), inv_cell=inv.double())
    assert (rep - ref.detach()).abs().max() <= 2e-6 * ref.detach().abs().max()
    nb, A, R = ref.shape
    jref = torch.zeros(nb, A, A, 3, R, dtype=torch.float64)
    for i in range(A):
        for col in range(R):
            gi, = torch.autograd.grad(ref[:, i, col].sum(), x, retain_graph=True)
            jref[:, i, :, :, col] = gi
    assert (jac - jref).abs().max() <= 2e-5 * jref.abs().max()


@pytest.mark.parametrize('skew', [False, True])
def test_periodic_energy_and_forces(cabi, skew):
    X, Z, c, species, cell, inv = periodic_batch(14, nb=6, skew=skew)
    p = H.fchl_params(species, rcut=RCUT)
    kp = H.kernel_params(p, DEV)
    rep = fchl19_representation(X.double(), Z, c, p, cell=cell.double(), inv_cell=inv.double()).numpy()
    from qml_lightning_b200.utils import synthetic as syn
    red = torch.from_numpy(syn.svd_reductors(rep, Z.numpy(), c.numpy(), species, 32, 7))
    D, bias, alpha = (torch.from_numpy(a) for a in syn.sorf_parameters(8, len(species), 32, 8, 1))
    model = dict(kind='sorf', elements=species, reductors=red, Dmat=D, bias=bias, alpha=alpha, sigma=2.0, ntransforms=1)
    E_ref, F_ref = energy_and_forces(X, Z, c, p, model, cell=cell.double(), inv_cell=inv.double())
    packed = cabi.sorf_pack(D.to(DEV), bias.to(DEV), alpha.to(DEV))
    E, gX = cabi.sorf_predict(X.to(DEV), Z.to(DEV), c.to(DEV), kp, torch.tensor(species, dtype=torch.float32, device=DEV),
                              red.to(DEV), packed, 8, 1, 2.0, cell.to(DEV), inv.to(DEV))
    assert ((E.cpu().double() - E_ref).abs() <= H.energy_tolerance(E_ref)).all()
    assert (-gX.cpu().double() - F_ref).abs().max() <= 1e-4
