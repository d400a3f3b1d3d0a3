"""The function-level surface of the upstream extension modules (``qml_lightning_b200.cuda.*``, ``features.SORF``).

The bodies of upstream ``calculate_features`` (models/hadamard_features.py:66-80 and models/random_features.py:60-67)
and of the element loop of ``build_Z_components`` (models/kernel.py:134-170) are restated here with the upstream
function names; their result must equal ``training_rows``, which the model classes use.
"""
import numpy as np
import pytest
import torch

from tests import helpers as H
from tests.test_gpu_models import build_model

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def _batch(m, X, Z, c):
    Xl = [X[i, :int(c[i])].numpy() for i in range(X.shape[0])]
    Zl = [Z[i, :int(c[i])].numpy() for i in range(X.shape[0])]
    return m.format_data(Xl, Zl)


def _projected_rows(m, data):
    """Per element: projected representation rows, projected Jacobian rows and molecule indexes, as the element loop of
    build_Z_components prepares them (kernel.py:141-160), through the upstream-named fchl_gpu functions."""
    from qml_lightning_b200.cuda import fchl_gpu, pairlist_gpu
    r = m.rep
    X, Zc, counts = data['coordinates'], data['charges'], data['natom_counts']
    et = fchl_gpu.get_element_types_gpu(X, Zc, counts, r.species)
    nn = pairlist_gpu.get_num_neighbours_gpu(X, counts, float(r.rcut), data['cells'], data['inv_cells'])
    nl = pairlist_gpu.get_neighbour_list_gpu(X, counts, int(nn.max()), float(r.rcut), data['cells'], data['inv_cells'])
    rep, jac = fchl_gpu.get_fchl_and_derivative(X, Zc, r.species, et, data['cells'], data['inv_cells'], data['atomIDs'],
                                                data['molIDs'], nl, nn, r.Rs2, r.Rs3, float(r.eta2), float(r.eta3),
                                                float(r.two_body_decay), float(r.three_body_weight),
                                                float(r.three_body_decay), float(r.rcut), True)
    out = []
    for e in m.elements.tolist():
        mask = Zc.int() == int(e)
        if not bool(mask.any()):
            continue
        ei = int(m.element2index[int(e)])
        idx = torch.where(mask)[0].type(torch.int)
        sub = torch.matmul(rep[mask], m.reductors[ei])
        sub_grad = torch.einsum('jmnk,kl->jmnl', jac[mask], m.reductors[ei])
        out.append((e, ei, idx, sub.contiguous(), sub_grad.contiguous()))
    return out


def test_upstream_sorf_calculate_features_body():
    from qml_lightning_b200.cuda.sorf_gpu import (compute_hadamard_features, compute_molecular_featurization_derivative,
                                                  compute_partial_feature_derivatives, sorf_matrix_gpu)
    X, Z, c, species = H.batch_mixed(6, seed=21, max_atoms=9)
    p, ref, m = build_model(X, Z, c, species, 64, 4, T=2)
    data = _batch(m, X, Z, c)
    nb, A = data['charges'].shape
    Ztrain = torch.zeros(nb, m.nfeatures(), dtype=torch.float64, device=DEV)
    Gtrain = torch.zeros(nb, A, 3, m.nfeatures(), dtype=torch.float64, device=DEV)
    for e, ei, idx, sub, sub_grad in _projected_rows(m, data):
        # hadamard_features.py:66-80
        coeff_normalisation = np.sqrt(sub.shape[1]) / m.sigma
        coeffs = coeff_normalisation * sorf_matrix_gpu(sub, m.Dmat[ei])
        compute_hadamard_features(coeffs, m.bias[ei], idx, Ztrain)
        cos_derivs = torch.zeros(coeffs.shape, device=coeffs.device, dtype=torch.float64)
        compute_partial_feature_derivatives(coeffs, m.bias[ei], cos_derivs)
        compute_molecular_featurization_derivative(cos_derivs, coeff_normalisation, m.Dmat[ei], sub_grad, idx, Gtrain)
    Zt, Gt = m.training_rows(data, with_forces=True)
    assert (Ztrain - Zt).abs().max() <= 2e-6
    assert (Gtrain - Gt).abs().max() <= 2e-5 * max(1.0, float(Gt.abs().max()))
    # and the model's own calculate_features with upstream's arguments
    Z2 = torch.zeros_like(Ztrain)
    G2 = torch.zeros_like(Gtrain)
    for e, ei, idx, sub, sub_grad in _projected_rows(m, data):
        m.calculate_features(sub, e, idx, Z2, sub_grad, G2)
    assert (Z2 - Zt).abs().max() <= 2e-6
    assert (G2 - Gt).abs().max() <= 2e-5 * max(1.0, float(Gt.abs().max()))


def test_upstream_rff_calculate_features_body():
    import qml_lightning_b200 as q
    from qml_lightning_b200.cuda.rff_gpu import get_rff, get_rff_derivatives
    X, Z, c, species = H.batch_mixed(6, seed=22, max_atoms=9)
    p = H.fchl_params(species)
    ref = H.rff_model(X, Z, c, p, species, 32, 256)
    rep = q.FCHLCuda(species=np.array(species), rcut=p.rcut, nRs2=p.nRs2, nRs3=p.nRs3, eta2=p.eta2, eta3=p.eta3,
                     two_body_decay=p.two_body_decay, three_body_weight=p.three_body_weight,
                     three_body_decay=p.three_body_decay, device=DEV)
    m = q.RandomFourrierFeaturesModel(rep=rep, elements=np.array(species), sigma=2.0, npcas=32, nstacks=8)
    m.reductors, m.W, m.b = ref['reductors'].to(DEV), ref['W'].to(DEV), ref['b'].to(DEV)
    m.set_alpha(ref['alpha'].to(DEV))
    data = _batch(m, X, Z, c)
    nb, A = data['charges'].shape
    Ztrain = torch.zeros(nb, m.nfeatures(), dtype=torch.float64, device=DEV)
    Gtrain = torch.zeros(nb, A, 3, m.nfeatures(), dtype=torch.float64, device=DEV)
    for e, ei, idx, sub, sub_grad in _projected_rows(m, data):
        # random_features.py:60-67
        get_rff(sub, m.W[ei].double(), m.b[ei].double(), idx, Ztrain)
        get_rff_derivatives(sub, sub_grad, m.W[ei].double(), m.b[ei].double(), idx, Gtrain)
    Zt, Gt = m.training_rows(data, with_forces=True)
    assert (Ztrain - Zt).abs().max() <= 2e-6
    assert (Gtrain - Gt).abs().max() <= 2e-5 * max(1.0, float(Gt.abs().max()))


def test_autograd_function_wrappers():
    """features.SORF.SORFTransformCuda / CosFeatures differentiate like the TorchScript operators of the same stages."""
    from qml_lightning_b200.features.SORF import CosFeatures, SORFTransformCuda
    gen = torch.Generator().manual_seed(3)
    n, N, S, T, nmol = 37, 64, 5, 2, 4
    u = torch.randn(n, N, generator=gen).to(DEV).requires_grad_(True)
    D = (torch.randint(0, 2, (T, S, N), generator=gen).float() * 2 - 1).to(DEV)
    b = (torch.rand(S * N, generator=gen) * 6.28).to(DEV)
    idx = torch.sort(torch.randint(0, nmol, (n,), generator=gen))[0].int().to(DEV)
    w = torch.randn(nmol, S * N, generator=gen).to(DEV)
    co = SORFTransformCuda.apply(u, D, 1.7, T)
    feats = CosFeatures.apply(co.view(n, S * N), b, nmol, idx)
    g1, = torch.autograd.grad((feats * w).sum(), u)
    u2 = u.detach().clone().requires_grad_(True)
    co2 = torch.ops.qml_lightning_sorf.get_SORF_coefficients(u2, D, torch.tensor(1.7), torch.tensor(T))
    f2 = torch.ops.qml_lightning_sorf.get_cos_features(co2.view(n, S * N), b, torch.tensor(nmol), idx)
    g2, = torch.autograd.grad((f2 * w).sum(), u2)
    assert torch.equal(feats, f2) and torch.equal(g1, g2)


def test_matmul_and_reduce_accumulates_in_place():
    """utils_gpu.matmul_and_reduce with upstream's call pattern (kernel.py:176-188): no further from a float64 product
    than the float32 Kahan product it replaces (oracle.kahan_gram restates cuda/utils_kernel.cu:70-129)."""
    from oracle import kahan_gram
    from qml_lightning_b200.cuda.utils_gpu import matmul_and_reduce
    gen = torch.Generator().manual_seed(5)
    rows, F = 300, 256
    Ztrain = torch.randn(rows, F, generator=gen, dtype=torch.float64) * torch.logspace(-3, 0, F, dtype=torch.float64)
    C0 = torch.randn(F, F, generator=gen, dtype=torch.float64)
    C = C0.clone().to(DEV)
    Zd = Ztrain.to(DEV)
    matmul_and_reduce(Zd.float().T, Zd.float(), C)
    exact = Ztrain.float().double().T @ Ztrain.float().double()
    err_new = (C.cpu() - C0 - exact).abs().max()
    err_kahan = (kahan_gram(Ztrain) - exact).abs().max()
    assert err_new <= max(2.0 * float(err_kahan), 1e-7 * float(exact.abs().max())), (float(err_new), float(err_kahan))
