"""Size-independent properties of the prediction path at the full benchmark sizes, where the CPU oracle is out of reach:

* c1 (10,000 conformers x 21 atoms, npcas 256, 65,536 SORF features), c2 (200,000 mixed molecules with 4-29 atoms and
  five elements, npcas 128, 32,768 features) and the RFF configuration on 20,000 of the c1 conformers (16,384 features);
* the energy is invariant under rigid translation and rotation, so the forces of every molecule sum to zero, carry no
  net torque, and rotate with the molecule;
* molecules are independent: a sub-batch, taken alone and in another order, reproduces its energies and forces;
* a sample of the batch agrees with the float64 oracle (the parity tests proper run on small batches).
Random orthonormal reductors stand in for the SVD ones (the properties do not depend on them).
"""
import numpy as np
import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def _rotation(seed):
    q, _ = np.linalg.qr(np.random.default_rng(seed).normal(size=(3, 3)))
    if np.linalg.det(q) < 0:
        q[:, 0] = -q[:, 0]
    return torch.from_numpy(q.astype(np.float32))


def _check_invariances(predict, X, Z, c):
    """predict(X, Z, c) -> (E [nb], dE/dX [nb, A, 3]) on the device."""
    nb, A = Z.shape
    mask = (torch.arange(A)[None, :] < c[:, None]).to(DEV)
    Xd, Zd, cd = X.to(DEV), Z.to(DEV), c.to(DEV)
    E, G = predict(Xd, Zd, cd)
    assert torch.isfinite(E).all() and torch.isfinite(G).all()
    assert (G[~mask] == 0).all()                                   # padding atoms carry no gradient
    # translation invariance: the forces of a molecule sum to zero
    net = G.sum(dim=1).abs().max().item()
    assert net <= 5e-5, net                                        # measured 4e-6 .. 6e-6 (forces up to ~10)
    # rotation invariance: no net torque (about the centroid of the real atoms)
    cen = (Xd * mask[..., None]).sum(1, keepdim=True) / cd[:, None, None]
    torque = torch.cross((Xd - cen) * mask[..., None], G, dim=2).sum(1).abs().max().item()
    assert torque <= 3e-4, torque                                  # measured 1e-5 .. 7e-5
    # a rigidly moved copy has the same energies and co-rotated gradients
    R = _rotation(5).to(DEV)
    shift = torch.tensor([0.37, -1.2, 2.1], device=DEV)
    X2 = ((Xd @ R.T) + shift) * mask[..., None]
    E2, G2 = predict(X2, Zd, cd)
    rms = float(torch.sqrt(torch.mean(E.double() ** 2)))
    assert ((E2 - E).abs() <= 2e-5 * torch.clamp(E.abs(), min=rms)).all(), float((E2 - E).abs().max())
    # measured 3e-5 (conformers) and 2e-4 (mixed clusters: fp32 rounding of the moved coordinates times stiff contacts)
    assert (G2 - G @ R.T).abs().max().item() <= 5e-4
    # independence of the molecules: a permuted sub-batch alone
    idx = torch.from_numpy(np.random.default_rng(9).permutation(nb)[:max(64, nb // 50)].copy()).to(DEV)
    E3, G3 = predict(Xd[idx].contiguous(), Zd[idx].contiguous(), cd[idx].contiguous())
    assert ((E3 - E[idx]).abs() <= 2e-6 * torch.clamp(E[idx].abs(), min=rms)).all()
    assert (G3 - G[idx]).abs().max().item() <= 2e-5
    return E, G


def _oracle_sample(X, Z, c, p, model, E, G, n=6):
    from oracle import energy_and_forces
    sel = np.random.default_rng(3).choice(X.shape[0], size=n, replace=False)
    sel.sort()
    Xs, Zs, cs = X[sel], Z[sel], c[sel]
    E_ref, F_ref = energy_and_forces(Xs, Zs, cs, p, model, dtype=torch.float64)
    Es, Gs = E[sel].cpu().double(), G[sel].cpu().double()
    rms = float(torch.sqrt(torch.mean(E.double() ** 2)))
    assert ((Es - E_ref).abs() <= 1e-5 * torch.clamp(E_ref.abs(), min=rms)).all(), float((Es - E_ref).abs().max())
    assert (-Gs - F_ref).abs().max() <= 1e-4


@pytest.mark.parametrize('name', ['c1', 'c2'])
def test_sorf_full_size_properties(name):
    from qml_lightning_b200 import cabi
    from qml_lightning_b200.utils import synthetic as syn
    if name == 'c1':
        Xn, Zn, cn = syn.conformers(1001, syn.C1_CHARGES, 10000)
        species, npcas, nstacks = [1, 6, 8], 256, 256
    else:
        Xn, Zn, cn = syn.mixed_molecules(1002, 200000)
        species, npcas, nstacks = [1, 6, 7, 8, 9], 128, 256
    X, Z, c = torch.from_numpy(Xn), torch.from_numpy(Zn), torch.from_numpy(cn)
    p = H.fchl_params(species)
    kp = H.kernel_params(p, DEV)
    repsize = len(species) * p.nRs2 + len(species) * (len(species) + 1) * p.nRs3
    red = torch.from_numpy(syn.random_orthonormal_reductors(7, len(species), repsize, npcas)).float()
    D, b, a = syn.sorf_parameters(8, len(species), npcas, nstacks, 1)
    model = dict(kind='sorf', elements=species, reductors=red, Dmat=torch.from_numpy(D), bias=torch.from_numpy(b),
                 alpha=torch.from_numpy(a), sigma=2.0, ntransforms=1)
    packed = cabi.sorf_pack(model['Dmat'].to(DEV), model['bias'].to(DEV), model['alpha'].to(DEV))
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    redd = red.to(DEV)
    natoms = int(c.sum())
    before = cabi.tc_timeouts()

    def predict(Xd, Zd, cd):
        E, G = cabi.sorf_predict(Xd, Zd, cd, kp, el, redd, packed, nstacks, 1, 2.0, n_atoms_upper=min(natoms, Zd.numel()))
        return E.clone(), G.clone()

    E, G = _check_invariances(predict, X, Z, c)
    assert cabi.tc_timeouts() == before
    _oracle_sample(X, Z, c, p, model, E, G)


def test_rff_full_width_properties():
    from qml_lightning_b200 import cabi
    from qml_lightning_b200.utils import synthetic as syn
    Xn, Zn, cn = syn.conformers(1001, syn.C1_CHARGES, 20000)
    species, npcas, D = [1, 6, 8], 256, 16384
    X, Z, c = torch.from_numpy(Xn), torch.from_numpy(Zn), torch.from_numpy(cn)
    p = H.fchl_params(species)
    kp = H.kernel_params(p, DEV)
    repsize = len(species) * p.nRs2 + len(species) * (len(species) + 1) * p.nRs3
    red = torch.from_numpy(syn.random_orthonormal_reductors(7, len(species), repsize, npcas)).float()
    W, b, a = syn.rff_parameters(9, len(species), npcas, D, 2.0)
    model = dict(kind='rff', elements=species, reductors=red, W=torch.from_numpy(W), b=torch.from_numpy(b), alpha=torch.from_numpy(a))
    packed = cabi.rff_pack(model['W'].to(DEV), model['b'].to(DEV), model['alpha'].to(DEV))
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    redd = red.to(DEV)
    before = cabi.tc_timeouts()

    def predict(Xd, Zd, cd):
        E, G = cabi.rff_predict_packed(Xd, Zd, cd, kp, el, redd, packed)
        return E.clone(), G.clone()

    E, G = _check_invariances(predict, X, Z, c)
    assert cabi.tc_timeouts() == before
    _oracle_sample(X, Z, c, p, model, E, G)


def test_normal_equations_full_width_linearity():
    """Training configuration at full width (npcas 256, nstacks 128: 32,768 features, a 32,768^2 float64 matrix): the
    normal equations accumulated over 64 conformers in one batch and in two batches of 32 agree to 1e-10 relative, the
    matrix is symmetric, and Z^T y follows the same split."""
    import qml_lightning_b200 as q
    from qml_lightning_b200.utils import synthetic as syn
    Xn, Zn, cn = syn.conformers(1004, syn.C1_CHARGES, 64)
    species, npcas, nstacks = [1, 6, 8], 256, 128
    rep = q.FCHLCuda(species=np.array(species), rcut=6.0, nRs2=24, nRs3=22, eta2=0.32, eta3=2.7, two_body_decay=1.8,
                     three_body_weight=13.4, three_body_decay=0.57, device=DEV)
    m = q.HadamardFeaturesModel(rep=rep, elements=np.array(species), ntransforms=1, sigma=2.0, llambda=1e-5, npcas=npcas,
                                nstacks=nstacks, nbatch_train=64, nbatch_test=64)
    m.reductors = torch.from_numpy(syn.random_orthonormal_reductors(7, len(species), rep.get_repsize(), npcas)).float().to(DEV)
    m._parameters_changed()
    rng = np.random.default_rng(11)
    Xl, Zl = [x for x in Xn], [z for z in Zn]
    E = rng.normal(size=64)
    Fl = [rng.normal(size=(21, 3)) for _ in range(64)]
    A1, y1 = m.build_Z_components(Xl, Zl, E, Fl, print_info=False)
    m.nbatch_train = 32
    A2, y2 = m.build_Z_components(Xl, Zl, E, Fl, print_info=False)
    scale = float(A1.abs().max())
    assert scale > 0 and torch.isfinite(A1).all()
    assert float((A1 - A2).abs().max()) <= 1e-10 * scale
    assert float((A1 - A1.T).abs().max()) == 0.0
    assert float((y1 - y2).abs().max()) <= 1e-10 * float(y1.abs().max())


def test_normal_equations_full_width_against_float64_matmul():
    """One c4 row block (64 conformers x 64 rows = 4,096 rows, 32,768 features) through the in-tree float64 kernel
    against ``torch.matmul`` in float64 on the same rows: 1e-10 relative on the upper triangle (the benchmark
    contract), the lower triangle untouched, Z^T y likewise; the specialised path differs by float32 rounding only."""
    from qml_lightning_b200 import cabi
    gen = torch.Generator(device=DEV).manual_seed(4)
    rows, F = 4096, 32768
    M = torch.randn(rows, F, generator=gen, device=DEV, dtype=torch.float64) * torch.logspace(-2, 0, F, device=DEV, dtype=torch.float64)
    y = torch.randn(rows, generator=gen, device=DEV, dtype=torch.float64)
    ZTZ = torch.zeros(F, F, device=DEV, dtype=torch.float64)
    ZTy = torch.zeros(F, 1, device=DEV, dtype=torch.float64)
    cabi.normal_equations_accumulate(M, y, ZTZ, ZTy)
    refy = M.T @ y[:, None]
    assert float((ZTy - refy).abs().max()) <= 1e-10 * float(refy.abs().max())
    scale = None
    for c0 in range(0, F, 4096):                                   # column panels: the reference never needs a second 8.6 GB matrix
        ref = M.T @ M[:, c0:c0 + 4096]                             # [F, 4096]
        got = ZTZ[:, c0:c0 + 4096]
        scale = float(ref.abs().max()) if scale is None else max(scale, float(ref.abs().max()))
        i = torch.arange(F, device=DEV)[:, None]
        j = c0 + torch.arange(4096, device=DEV)[None, :]
        upper = j >= i
        assert float(((got - ref) * upper).abs().max()) <= 1e-10 * scale
        assert float((got * (~upper)).abs().max()) == 0.0
        del ref, got, upper
    cabi.symmetrize_upper(ZTZ)
    assert float((ZTZ[:4096, :4096] - ZTZ[:4096, :4096].T).abs().max()) == 0.0


def test_sorf_training_rows_full_width():
    """SORF training rows at the training configuration's width (npcas 256, 128 stacks = 32,768 features) against the
    float64 oracle on two sampled stacks (512 features; the oracle differentiates feature by feature)."""
    import math
    import qml_lightning_b200 as q
    from oracle import training_rows
    X, Z, c, species = H.batch_c1(3, seed=51)
    p = H.fchl_params(species)
    npcas, nstacks = 256, 128
    ref = H.sorf_model(X, Z, c, p, species, npcas, nstacks)
    rep = q.FCHLCuda(species=np.array(species), rcut=p.rcut, nRs2=p.nRs2, nRs3=p.nRs3, eta2=p.eta2, eta3=p.eta3,
                     two_body_decay=p.two_body_decay, three_body_weight=p.three_body_weight,
                     three_body_decay=p.three_body_decay, device=DEV)
    m = q.HadamardFeaturesModel(rep=rep, elements=np.array(species), ntransforms=1, sigma=ref['sigma'], npcas=npcas, nstacks=nstacks)
    m.reductors, m.Dmat, m.bias = ref['reductors'].to(DEV), ref['Dmat'].to(DEV), ref['bias'].to(DEV)
    m.set_alpha(ref['alpha'].to(DEV))
    counts = c.tolist()
    data = m.format_data([X[i, :counts[i]].numpy() for i in range(len(counts))], [Z[i, :counts[i]].numpy() for i in range(len(counts))])
    Zt, Gt = m.training_rows(data, with_forces=True)
    A = data['charges'].shape[1]
    stacks = [5, 127]
    cols = torch.cat([torch.arange(s * npcas, (s + 1) * npcas) for s in stacks])
    sub = dict(ref, Dmat=ref['Dmat'][:, :, stacks].contiguous(), bias=ref['bias'][:, cols].contiguous(), alpha=ref['alpha'][cols])
    Zr, Gr = training_rows(X, Z, c, p, sub)
    scale = math.sqrt(len(cols) / (npcas * nstacks))               # the oracle normalises by its own feature count
    Zr, Gr = Zr * scale, Gr * scale
    assert (Zt.cpu()[:, cols] - Zr).abs().max() <= 2e-6 * max(float(Zr.abs().max()), 1e-2)
    assert (Gt.cpu()[..., cols] - Gr[:, :A]).abs().max() <= 2e-5 * float(Gr.abs().max())
