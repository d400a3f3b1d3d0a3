"""Edge cases of the prediction path on the GPU: tiny and empty inputs, missing neighbours, unknown species,
collinear triplets, a large molecule, and the shared-memory limit."""
import numpy as np
import pytest
import torch

from oracle import energy_and_forces, fchl19_representation
from tests import helpers as H

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def predict(X, Z, c, species, model, p):
    from qml_lightning_b200 import cabi
    kp = H.kernel_params(p, DEV)
    packed = cabi.sorf_pack(model['Dmat'].to(DEV), model['bias'].to(DEV), model['alpha'].to(DEV))
    E, g = cabi.sorf_predict(X.to(DEV), Z.to(DEV), c.to(DEV), kp, torch.tensor(model['elements'], dtype=torch.float32, device=DEV),
                             model['reductors'].to(DEV), packed, model['Dmat'].shape[2], model['ntransforms'], model['sigma'])
    return E.cpu().double(), -g.cpu().double()


def small_model(species, npcas=32, nstacks=4, seed=3):
    p = H.fchl_params(species)
    Xb, Zb, cb, _ = H.batch_mixed(20, seed=seed, max_atoms=10) if len(species) == 5 else H.batch_c0(20, seed=seed)
    return p, H.sorf_model(Xb, Zb, cb, p, species, npcas, nstacks)


def test_single_atom_pair_and_isolated_atoms():
    species = [1, 6, 8]
    p, model = small_model(species)
    X = torch.zeros(4, 3, 3)
    Z = torch.zeros(4, 3)
    c = torch.tensor([1, 2, 3, 2], dtype=torch.int32)
    Z[0, 0] = 6                                             # one atom, no neighbour at all
    Z[1, :2] = torch.tensor([1., 8.]); X[1, 1, 0] = 1.1      # one pair: two-body terms only
    Z[2, :3] = torch.tensor([6., 1., 1.]); X[2, 1, 0] = 1.0; X[2, 2, 0] = 20.0   # third atom beyond the cut-off
    Z[3, :2] = torch.tensor([1., 1.]); X[3, 1, 2] = 9.0      # two atoms that do not see each other
    E_ref, F_ref = energy_and_forces(X, Z, c, p, model)
    E, F = predict(X, Z, c, species, model, p)
    assert torch.isfinite(E).all() and torch.isfinite(F).all()
    assert ((E - E_ref).abs() <= H.energy_tolerance(E_ref)).all()
    assert (F - F_ref).abs().max() <= 1e-4
    assert (F[0] == 0).all() and (F[3] == 0).all()           # nothing to differentiate without neighbours


def test_empty_batch_and_absent_element():
    from qml_lightning_b200 import cabi
    species = [1, 6, 8]
    p, model = small_model(species)
    kp = H.kernel_params(p, DEV)
    packed = cabi.sorf_pack(model['Dmat'].to(DEV), model['bias'].to(DEV), model['alpha'].to(DEV))
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    E, g = cabi.sorf_predict(torch.zeros(0, 5, 3, device=DEV), torch.zeros(0, 5, device=DEV), torch.zeros(0, dtype=torch.int32, device=DEV),
                             kp, el, model['reductors'].to(DEV), packed, 4, 1, model['sigma'])
    assert E.shape == (0,) and g.shape == (0, 5, 3)
    # a batch without any oxygen: that element group is empty
    X, Z, c, _ = H.batch_c0(3, seed=5)
    Z = torch.where(Z == 8, torch.full_like(Z, 6.0), Z)
    E_ref, F_ref = energy_and_forces(X, Z, c, p, model)
    E, F = predict(X, Z, c, species, model, p)
    assert ((E - E_ref).abs() <= H.energy_tolerance(E_ref)).all() and (F - F_ref).abs().max() <= 1e-4


def test_unknown_species_is_ignored():
    """An atom whose charge is in neither the representation's species nor the model's elements contributes nothing
    and is not a neighbour of anybody (upstream would index out of bounds)."""
    species = [1, 6, 8]
    p, model = small_model(species)
    X, Z, c, _ = H.batch_c0(2, seed=6)
    Zx = Z.clone()
    Zx[:, 3] = 17.0                                           # chlorine: unknown
    keep = [0, 1, 2, 4, 5, 6, 7, 8]
    E_ref, F_ref = energy_and_forces(X[:, keep], Z[:, keep], c - 1, p, model)
    E, F = predict(X, Zx, c, species, model, p)
    assert ((E - E_ref).abs() <= H.energy_tolerance(E_ref)).all()
    assert (F[:, keep] - F_ref).abs().max() <= 1e-4 and (F[:, 3] == 0).all()


def test_collinear_triplet_is_finite_and_matches_energy():
    species = [1, 6, 8]
    p, model = small_model(species)
    X = torch.zeros(1, 3, 3)
    X[0, 1, 0] = 1.2
    X[0, 2, 0] = -1.1                                         # exactly collinear: sin(theta) = 0 for the centre atom
    Z = torch.tensor([[6., 1., 8.]])
    c = torch.tensor([3], dtype=torch.int32)
    E_ref = energy_and_forces(X, Z, c, p, model, forces=False)
    E, F = predict(X, Z, c, species, model, p)
    assert torch.isfinite(F).all()
    assert ((E - E_ref).abs() <= H.energy_tolerance(E_ref)).all()
    assert F[0, :, 1:].abs().max() <= 1e-3                    # no force perpendicular to the axis by symmetry


def test_large_molecule_and_shared_memory_limit():
    from qml_lightning_b200 import cabi
    species = [1, 6, 8]
    p = H.fchl_params(species)
    rng = np.random.default_rng(0)
    n = 70                                                    # more than 32 neighbours per atom: multi-chunk ballots
    from qml_lightning_b200.utils.synthetic import random_cluster
    X = torch.from_numpy(random_cluster(rng, n, 1.0, 1.5)).float()[None]
    Z = torch.from_numpy(rng.choice(species, size=n)).float()[None]
    c = torch.tensor([n], dtype=torch.int32)
    kp = H.kernel_params(p, DEV)
    x = X.double().clone().requires_grad_(True)
    ref = fchl19_representation(x, Z, c, p)
    rep = cabi.fchl19_forward(X.to(DEV), Z.to(DEV), c.to(DEV), kp).cpu().double()
    assert (rep - ref.detach()).abs().max() <= 3e-6 * ref.detach().abs().max()
    g = torch.from_numpy(rng.normal(size=tuple(ref.shape))) * 0.1
    gref, = torch.autograd.grad((ref * g).sum(), x)
    gX = cabi.fchl19_backward(X.to(DEV), Z.to(DEV), c.to(DEV), kp, g.float().to(DEV)).cpu().double()
    assert (gX - gref).abs().max() <= 3e-5 * gref.abs().max()
    # a padded width that cannot fit the per-warp slabs in shared memory is refused with a clear error
    big = 4000
    with pytest.raises(RuntimeError, match='shared memory'):
        cabi.fchl19_forward(torch.zeros(1, big, 3, device=DEV), torch.zeros(1, big, device=DEV),
                            torch.zeros(1, dtype=torch.int32, device=DEV), kp)


def test_row_capacity_too_small_gives_nan_not_wrong_numbers():
    """``atomIDs`` shorter than the batch (the row capacity is derived from its length): the molecules whose atoms found
    no row come back as NaN in energies and gradients, every other molecule is unchanged, nothing is dropped silently."""
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_c0(200, seed=61)
    p = H.fchl_params(species)
    kp = H.kernel_params(p, DEV)
    model = H.sorf_model(X, Z, c, p, species, 64, 4)
    packed = cabi.sorf_pack(model['Dmat'].to(DEV), model['bias'].to(DEV), model['alpha'].to(DEV))
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    args = (X.to(DEV), Z.to(DEV), c.to(DEV), kp, el, model['reductors'].to(DEV), packed, 4, 1, model['sigma'])
    E_full, G_full = cabi.sorf_predict(*args)
    total = int(c.sum())
    # 200 molecules x 9 atoms = 1,800 atoms in 1280 (H) + 512 (C) + 256 (O) = 2,048 element-grouped rows; claiming 1,500
    # atoms gives 1,920 rows: the oxygen atoms of the last molecules find no row
    E, G = cabi.sorf_predict(*args, n_atoms_upper=1500)
    torch.cuda.synchronize()
    bad = torch.isnan(E)
    assert bool(bad.any()) and not bool(bad.all()), (int(bad.sum()), total)
    assert torch.equal(torch.isnan(G).flatten(1).any(dim=1), bad)               # the same molecules in the gradient
    assert torch.allclose(E[~bad], E_full[~bad], rtol=0, atol=0) and torch.equal(G[~bad], G_full[~bad])


def test_stage_ranges_flag_changes_nothing_but_the_annotation():
    """With the NVTX flag set every stage wrapper pushes and pops a named range; results are the same bits."""
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_c0(4)
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    a = cabi.group_by_element(Z.to(DEV), c.to(DEV), el)
    cabi.NVTX_RANGES = True
    try:
        b = cabi.group_by_element(Z.to(DEV), c.to(DEV), el)
    finally:
        cabi.NVTX_RANGES = False
    assert torch.equal(a.row_of_slot, b.row_of_slot) and torch.equal(a.group_start, b.group_start)


def test_format_data_through_the_pinned_stage_is_reusable():
    """Two batches formatted back to back share one page-locked staging buffer: the device tensors of the first batch
    must not change when the second overwrites the stage, and both must equal a plain host construction."""
    import qml_lightning_b200 as q
    from tests.test_gpu_models import build_model
    X, Z, c, species = H.batch_mixed(40, seed=5, max_atoms=12)
    _, _, m = build_model(X[:8], Z[:8], c[:8], species, 32, 2)
    counts = c.tolist()
    Xl = [X[i, :counts[i]].numpy() for i in range(40)]
    Zl = [Z[i, :counts[i]].numpy() for i in range(40)]

    def plain(lo, hi):
        A = max(counts[lo:hi])
        co = torch.zeros(hi - lo, A, 3)
        ch = torch.zeros(hi - lo, A)
        for i in range(lo, hi):
            co[i - lo, :counts[i]] = X[i, :counts[i]]
            ch[i - lo, :counts[i]] = Z[i, :counts[i]]
        atom = torch.cat([torch.arange(n, dtype=torch.int32) for n in counts[lo:hi]])
        mol = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(counts[lo:hi])])
        return co, ch, torch.tensor(counts[lo:hi], dtype=torch.int32), atom, mol

    first = m.format_data(Xl[:30], Zl[:30])
    second = m.format_data(Xl[30:], Zl[30:])
    torch.cuda.synchronize()
    for data, ref in ((first, plain(0, 30)), (second, plain(30, 40))):
        for key, want in zip(('coordinates', 'charges', 'natom_counts', 'atomIDs', 'molIDs'), ref):
            got = data[key].cpu()
            assert got.dtype == want.dtype and torch.equal(got, want), key
    assert m._stage.buffer.is_pinned()
