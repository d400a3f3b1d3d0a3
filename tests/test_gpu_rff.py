"""GPU parity of the RFF path (feature stage, whole prediction, model class) against the float64 oracle.

The upstream repository ships no RFF fixture (its unit_test_rff.py loads a model file that is not in the tree), so the
RFF arithmetic is pinned only through the oracle restatement of models/random_features.py:69-102.
"""
import math

import numpy as np
import pytest
import torch

from oracle import energy_and_forces
from tests import helpers as H

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


@pytest.mark.parametrize('K', [32, 64, 128, 256])
@pytest.mark.parametrize('fast', [False, True])
@pytest.mark.parametrize('kernel,D', [('ffma', 200), ('tc', 200), ('tc', 32), ('tc', 1000), ('tc', 1120)])
def test_rff_energy_grad_matches_oracle(K, fast, kernel, D):
    """Both feature kernels (fp32 FFMA; tcgen05 on fp16 hi/lo pairs) against a float64 evaluation.  The feature counts
    cover a ragged last chunk (200, 1000), a single chunk (32), and odd / even chunk counts with one flush group (7) and
    several (32, 35)."""
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_mixed(14, seed=K)
    nel = len(species)
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), el)
    gen = torch.Generator().manual_seed(K)
    x = torch.randn(g.rows_cap, K, generator=gen)
    W = torch.randn(nel, K, D, generator=gen) * 0.5
    b = torch.rand(nel, D, generator=gen) * 2 * math.pi
    alpha = torch.randn(D, generator=gen)
    if kernel == 'tc':
        before = cabi.tc_timeouts()
        packed = cabi.rff_pack(W.to(DEV), b.to(DEV), alpha.to(DEV))
        e_atom, gx = cabi.rff_energy_grad_tc(x.to(DEV), g, packed, nel, fast_math=fast)
        assert cabi.tc_timeouts() == before
    else:
        e_atom, gx = cabi.rff_energy_grad(x.to(DEV), g, W.to(DEV), b.to(DEV), alpha.to(DEV), fast_math=fast)
    e_atom, gx = e_atom.cpu().double(), gx.cpu().double()
    gs, sor = g.group_start.cpu(), g.slot_of_row.cpu()
    tol = 3e-5 if fast else 5e-6
    for ei in range(nel):
        r0, r1 = int(gs[ei]), int(gs[ei + 1])
        if r1 == r0:
            continue
        xs = x[r0:r1].double().clone().requires_grad_(True)
        e_ref = (math.sqrt(2.0 / D) * torch.cos(xs @ W[ei].double() + b[ei].double()) * alpha.double()).sum(-1)
        g_ref, = torch.autograd.grad(e_ref.sum(), xs)
        live = sor[r0:r1] >= 0
        assert (e_atom[r0:r1][live] - e_ref.detach()[live]).abs().max() <= tol * max(1.0, float(e_ref.abs().max()))
        assert (gx[r0:r1][live] - g_ref[live]).abs().max() <= tol * max(1.0, float(g_ref.abs().max()))
        assert (e_atom[r0:r1][~live] == 0).all() and (gx[r0:r1][~live] == 0).all()


@pytest.mark.parametrize('name,build,nconf,npcas,D', [('c1', H.batch_c1, 6, 256, 1024), ('mixed', H.batch_mixed, 40, 128, 512)])
def test_rff_predict_and_model_class(name, build, nconf, npcas, D):
    import qml_lightning_b200 as q
    X, Z, c, species = build(nconf)
    p = H.fchl_params(species)
    ref = H.rff_model(X, Z, c, p, species, npcas, D)
    E_ref, F_ref = energy_and_forces(X, Z, c, p, ref, dtype=torch.float64)
    rep = q.FCHLCuda(species=np.array(species), rcut=p.rcut, nRs2=p.nRs2, nRs3=p.nRs3, eta2=p.eta2, eta3=p.eta3,
                     two_body_decay=p.two_body_decay, three_body_weight=p.three_body_weight,
                     three_body_decay=p.three_body_decay, device=DEV)
    m = q.RandomFourrierFeaturesModel(rep=rep, elements=np.array(species), sigma=2.0, nstacks=D // npcas, npcas=npcas)
    m.reductors, m.W, m.b = ref['reductors'].to(DEV), ref['W'].to(DEV), ref['b'].to(DEV)
    m.set_alpha(ref['alpha'].to(DEV))
    counts = c.tolist()
    atomIDs = torch.cat([torch.arange(n, dtype=torch.int32) for n in counts]).to(DEV)
    molIDs = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(counts)]).to(DEV)
    E, F = m.predict_opt(X.to(DEV), Z.to(DEV), atomIDs, molIDs, c.to(DEV))
    assert ((E.cpu().double() - E_ref).abs() <= H.energy_tolerance(E_ref)).all(), float((E.cpu().double() - E_ref).abs().max())
    assert (F.cpu().double() - F_ref).abs().max() <= 1e-4
    Xd = X.to(DEV).requires_grad_(True)
    Ef = m.forward(Xd, Z.to(DEV), atomIDs, molIDs, c.to(DEV))
    Ff, = torch.autograd.grad(-Ef.sum(), Xd)
    assert torch.equal(Ef.detach(), E) and (Ff - F).abs().max() <= 1e-5
    scripted = torch.jit.script(m)
    Es = scripted.forward(X.to(DEV), Z.to(DEV), atomIDs, molIDs, c.to(DEV))
    assert torch.equal(Es, E)


def test_rff_model_of_another_width_runs_on_the_next_kernel_width():
    """Upstream accepts any npcas; the kernels exist for 32, 64, 128 and 256.  A 48-component model is evaluated with
    zero-padded projection matrices and weights: predictions, the scripted forward and the training rows agree with
    the oracle at the model's own width."""
    import qml_lightning_b200 as q
    from oracle import training_rows
    npcas, D = 48, 384
    X, Z, c, species = H.batch_mixed(24, seed=31, max_atoms=9)
    p = H.fchl_params(species)
    ref = H.rff_model(X, Z, c, p, species, npcas, D)
    E_ref, F_ref = energy_and_forces(X, Z, c, p, ref, dtype=torch.float64)
    rep = q.FCHLCuda(species=np.array(species), rcut=p.rcut, nRs2=p.nRs2, nRs3=p.nRs3, eta2=p.eta2, eta3=p.eta3,
                     two_body_decay=p.two_body_decay, three_body_weight=p.three_body_weight,
                     three_body_decay=p.three_body_decay, device=DEV)
    m = q.RandomFourrierFeaturesModel(rep=rep, elements=np.array(species), sigma=2.0, nstacks=D // npcas, npcas=npcas)
    assert m.reductors.shape[-1] == npcas and m.W.shape[1:] == (npcas, D)
    m.reductors, m.W, m.b = ref['reductors'].to(DEV), ref['W'].to(DEV), ref['b'].to(DEV)
    m.set_alpha(ref['alpha'].to(DEV))
    counts = c.tolist()
    atomIDs = torch.cat([torch.arange(n, dtype=torch.int32) for n in counts]).to(DEV)
    molIDs = torch.cat([torch.full((n,), i, dtype=torch.int32) for i, n in enumerate(counts)]).to(DEV)
    E, F = m.predict_opt(X.to(DEV), Z.to(DEV), atomIDs, molIDs, c.to(DEV))
    assert ((E.cpu().double() - E_ref).abs() <= H.energy_tolerance(E_ref)).all(), float((E.cpu().double() - E_ref).abs().max())
    assert (F.cpu().double() - F_ref).abs().max() <= 1e-4
    scripted = torch.jit.script(m)
    Xd = X.to(DEV).requires_grad_(True)
    Es = scripted.forward(Xd, Z.to(DEV), atomIDs, molIDs, c.to(DEV))
    Fs, = torch.autograd.grad(-Es.sum(), Xd)
    assert torch.equal(Es.detach(), E) and (Fs - F).abs().max() <= 1e-5
    Xl = [X[i, :counts[i]].numpy() for i in range(6)]
    Zl = [Z[i, :counts[i]].numpy() for i in range(6)]
    data = m.format_data(Xl, Zl)
    Zt, Gt = m.training_rows(data, with_forces=True)
    Zr, Gr = training_rows(X[:6], Z[:6], c[:6], p, ref)
    A = data['charges'].shape[1]
    assert (Zt.cpu() - Zr).abs().max() <= 2e-6
    assert (Gt.cpu() - Gr[:, :A]).abs().max() <= 2e-5 * max(1.0, float(Gr.abs().max()))
    with pytest.raises(ValueError, match='npcas'):
        q.RandomFourrierFeaturesModel(rep=rep, elements=np.array(species), sigma=2.0, nstacks=2, npcas=320)


def test_rff_rejects_unsupported_width():
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_c0(2)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), torch.tensor(species, dtype=torch.float32, device=DEV))
    with pytest.raises(RuntimeError, match='npcas'):
        cabi.rff_energy_grad(torch.zeros(g.rows_cap, 48, device=DEV), g, torch.zeros(3, 48, 64, device=DEV),
                             torch.zeros(3, 64, device=DEV), torch.zeros(64, device=DEV))


def test_rff_tc_matches_ffma_on_large_feature_count():
    """16,384 features (512 chunks, 32 flush groups), wide argument range: the tensor-core kernel stays within fp32
    rounding of the FFMA kernel and of a float64 evaluation."""
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_c1(12)
    nel, K, D = len(species), 256, 16384
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), torch.tensor(species, dtype=torch.float32, device=DEV))
    gen = torch.Generator().manual_seed(5)
    x = (torch.randn(g.rows_cap, K, generator=gen) * 0.3).to(DEV)
    W = (torch.randn(nel, K, D, generator=gen) * 0.5).to(DEV)
    b = (torch.rand(nel, D, generator=gen) * 2 * math.pi).to(DEV)
    alpha = torch.randn(D, generator=gen).to(DEV)
    e0, g0 = cabi.rff_energy_grad(x, g, W, b, alpha, fast_math=True)
    e1, g1 = cabi.rff_energy_grad_tc(x, g, cabi.rff_pack(W, b, alpha), nel, fast_math=True)
    used = int(g.group_start[-1])
    live = (g.slot_of_row[:used] >= 0)
    gs = g.group_start.cpu()
    e_ref = torch.zeros(used, dtype=torch.float64, device=DEV)
    g_ref = torch.zeros(used, K, dtype=torch.float64, device=DEV)
    for ei in range(nel):
        r0, r1 = int(gs[ei]), int(gs[ei + 1])
        arg = x[r0:r1].double() @ W[ei].double() + b[ei].double()
        a = alpha.double() * math.sqrt(2.0 / D)
        e_ref[r0:r1] = (torch.cos(arg) * a).sum(-1)
        g_ref[r0:r1] = -(torch.sin(arg) * a) @ W[ei].double().T
    se, sg = float(e_ref[live].abs().max()), float(g_ref[live].abs().max())
    for e, gx in ((e0, g0), (e1, g1)):
        assert float((e[:used].double() - e_ref)[live].abs().max()) <= 5e-6 * se
        assert float((gx[:used].double() - g_ref)[live].abs().max()) <= 1e-5 * sg
    assert (e1[:used][~live] == 0).all() and (g1[:used][~live] == 0).all()


def test_rff_tc_refuses_foreign_parameters():
    """Parameters packed for another npcas: the kernel does nothing and reports through the tensor-core event counter."""
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_c0(2)
    nel = len(species)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), torch.tensor(species, dtype=torch.float32, device=DEV))
    packed = cabi.rff_pack(torch.zeros(nel, 64, 96, device=DEV), torch.zeros(nel, 96, device=DEV), torch.zeros(96, device=DEV))
    before = cabi.tc_timeouts()
    cabi.rff_energy_grad_tc(torch.zeros(g.rows_cap, 128, device=DEV), g, packed, nel)
    assert cabi.tc_timeouts() > before
    with pytest.raises(RuntimeError, match='unsupported'):
        cabi.rff_pack(torch.zeros(nel, 48, 96, device=DEV), torch.zeros(nel, 96, device=DEV), torch.zeros(96, device=DEV))


@pytest.mark.parametrize('xscale,ascale', [(1e-6, 1.0), (3e3, 1e-4), (1.0, 1e5)])
def test_rff_tc_operand_scaling(xscale, ascale):
    """The fp16 hi/lo pairs are formed after power-of-two scaling of x (per row tile), W and alpha (per model), so
    tiny / large inputs and weights keep fp32-level accuracy; alpha additionally spans six orders of magnitude."""
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_c0(20)
    nel, K, D = len(species), 64, 512
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), torch.tensor(species, dtype=torch.float32, device=DEV))
    gen = torch.Generator().manual_seed(11)
    x = (torch.randn(g.rows_cap, K, generator=gen) * xscale).to(DEV)
    W = (torch.randn(nel, K, D, generator=gen) * (0.3 / xscale)).to(DEV)       # arguments stay of order one
    b = (torch.rand(nel, D, generator=gen) * 2 * math.pi).to(DEV)
    alpha = (torch.randn(D, generator=gen) * ascale * torch.logspace(-6, 0, D)).to(DEV)
    e1, g1 = cabi.rff_energy_grad_tc(x, g, cabi.rff_pack(W, b, alpha), nel, fast_math=False)
    used = int(g.group_start[-1])
    live = g.slot_of_row[:used] >= 0
    gs = g.group_start.cpu()
    a = alpha.double() * math.sqrt(2.0 / D)
    for ei in range(nel):
        r0, r1 = int(gs[ei]), int(gs[ei + 1])
        arg = x[r0:r1].double() @ W[ei].double() + b[ei].double()
        e_ref = (torch.cos(arg) * a).sum(-1)
        g_ref = -(torch.sin(arg) * a) @ W[ei].double().T
        lv = live[r0:r1]
        if not bool(lv.any()):
            continue
        assert float((e1[r0:r1].double() - e_ref)[lv].abs().max()) <= 5e-6 * float(e_ref[lv].abs().max())
        assert float((g1[r0:r1].double() - g_ref)[lv].abs().max()) <= 1e-5 * float(g_ref[lv].abs().max())


def test_rff_golden_vectors_on_gpu():
    """CUDA RFF path (tensor-core prediction, float64 training rows) against the committed oracle vectors
    (tests/golden/make_golden.py)."""
    import os
    import qml_lightning_b200 as q
    from qml_lightning_b200 import cabi
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), 'golden', 'rff_small.npz'))
    X, Z, c = (torch.from_numpy(g[f'c0_{k}']) for k in ('X', 'Z', 'counts'))
    species = g['c0_species'].tolist()
    p = H.fchl_params(species)
    kp = H.kernel_params(p, DEV)
    W, b, alpha, red = (torch.from_numpy(g[f'c0_{k}']).to(DEV) for k in ('W', 'b', 'alpha', 'reductors'))
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    E, gX = cabi.rff_predict_packed(X.to(DEV), Z.to(DEV), c.to(DEV), kp, el, red, cabi.rff_pack(W, b, alpha))
    E_ref = torch.from_numpy(g['c0_E'])
    assert ((E.cpu().double() - E_ref).abs() <= H.energy_tolerance(E_ref)).all()
    assert np.abs(-gX.cpu().double().numpy() - g['c0_F']).max() <= 1e-4
    rep = q.FCHLCuda(species=np.array(species), rcut=p.rcut, nRs2=p.nRs2, nRs3=p.nRs3, eta2=p.eta2, eta3=p.eta3,
                     two_body_decay=p.two_body_decay, three_body_weight=p.three_body_weight,
                     three_body_decay=p.three_body_decay, device=DEV)
    m = q.RandomFourrierFeaturesModel(rep=rep, elements=np.array(species), sigma=2.0, nstacks=int(g['c0_nfeatures']) // int(g['c0_npcas']),
                                      npcas=int(g['c0_npcas']))
    m.reductors, m.W, m.b = red, W, b
    counts = c.tolist()
    data = m.format_data([X[i, :counts[i]].numpy() for i in range(len(counts))], [Z[i, :counts[i]].numpy() for i in range(len(counts))])
    Zt, Gt = m.training_rows(data, with_forces=True)
    A = data['charges'].shape[1]
    assert np.abs(Zt.cpu().numpy() - g['c0_Zrows']).max() <= 2e-6
    assert np.abs(Gt.cpu().numpy() - g['c0_Grows'][:, :A]).max() <= 2e-5 * max(1.0, float(np.abs(g['c0_Grows']).max()))


def test_rff_training_rows_full_width():
    """Training rows at the benchmark width (npcas 256, 16,384 features): against the float64 oracle from coordinates on
    sampled features, and -- fed with the kernel's own float32 inputs -- against a float64 evaluation of upstream's
    formula (cuda/random_features_kernel.cu:5-94: float64 dot products of float32 inputs), which the kernel must
    reproduce to float64 rounding.  Prints how far a float32 evaluation of the same rows would be."""
    import qml_lightning_b200 as q
    from oracle import training_rows
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_c1(4, seed=41)
    p = H.fchl_params(species)
    npcas, D = 256, 16384
    ref = H.rff_model(X, Z, c, p, species, npcas, D)
    rep = q.FCHLCuda(species=np.array(species), rcut=p.rcut, nRs2=p.nRs2, nRs3=p.nRs3, eta2=p.eta2, eta3=p.eta3,
                     two_body_decay=p.two_body_decay, three_body_weight=p.three_body_weight,
                     three_body_decay=p.three_body_decay, device=DEV)
    m = q.RandomFourrierFeaturesModel(rep=rep, elements=np.array(species), sigma=2.0, nstacks=D // npcas, npcas=npcas)
    m.reductors, m.W, m.b = ref['reductors'].to(DEV), ref['W'].to(DEV), ref['b'].to(DEV)
    counts = c.tolist()
    data = m.format_data([X[i, :counts[i]].numpy() for i in range(len(counts))], [Z[i, :counts[i]].numpy() for i in range(len(counts))])
    Zt, Gt = m.training_rows(data, with_forces=True)
    nb, A = data['charges'].shape
    # (1) from coordinates, sampled features: the oracle normalises by its own feature count
    idx = torch.tensor([0, 63, 64, 4097, 9999, 16383])
    sub = dict(ref, W=ref['W'][..., idx].contiguous(), b=ref['b'][..., idx].contiguous(), alpha=ref['alpha'][idx])
    Zr, Gr = training_rows(X, Z, c, p, sub)
    scale = math.sqrt(len(idx) / D)
    Zr, Gr = Zr * scale, Gr * scale
    assert (Zt.cpu()[:, idx] - Zr).abs().max() <= 2e-6 * max(float(Zr.abs().max()), 1e-2)
    assert (Gt.cpu()[..., idx] - Gr[:, :A]).abs().max() <= 2e-5 * float(Gr.abs().max())
    # (2) stage level, identical float32 inputs, all features
    Xd, Zd, cd = data['coordinates'], data['charges'], data['natom_counts']
    kp = rep.kernel_params(DEV)
    g = cabi.group_by_element(Zd, cd, m.species, data['atomIDs'].shape[0])
    rep_rows, jac_rows = cabi.fchl19_forward_jacobian(Xd, Zd, cd, kp, grouping=g)
    dx = cabi.pca_project_jacobian(jac_rows, m.reductors, g)
    x = cabi.pca_project(rep_rows, m.reductors, g)
    Z2, G2 = cabi.rff_train_features(x, dx, m.W, m.b, g, cd, nb, A)
    assert torch.equal(Z2, Zt) and torch.equal(G2, Gt)
    normf = math.sqrt(2.0 / D)
    Z64 = torch.zeros(nb, D, dtype=torch.float64, device=DEV)
    G64 = torch.zeros(nb, A, 3, D, dtype=torch.float64, device=DEV)
    Z32 = torch.zeros(nb, D, dtype=torch.float64, device=DEV)
    G32 = torch.zeros(nb, A, 3, D, dtype=torch.float64, device=DEV)
    tf32 = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    sor, gs = g.slot_of_row.cpu(), g.group_start.cpu()
    for e in range(len(species)):
        for row in range(int(gs[e]), int(gs[e + 1])):
            slot = int(sor[row])
            if slot < 0:
                continue
            mol = slot // A
            arg = x[row].double() @ m.W[e].double() + m.b[e].double()
            Z64[mol] += normf * torch.cos(arg)
            G64[mol] += normf * torch.sin(arg) * (dx[row].double() @ m.W[e].double())
            arg32 = x[row] @ m.W[e] + m.b[e]
            Z32[mol] += (normf * torch.cos(arg32)).double()
            G32[mol] += (normf * torch.sin(arg32) * (dx[row] @ m.W[e])).double()
    torch.backends.cuda.matmul.allow_tf32 = tf32
    gmax, zmax = float(G64.abs().max()), float(Z64.abs().max())
    print(f"RFF rows at K=256, D=16384: kernel vs float64 formula: Z {float((Zt - Z64).abs().max()) / zmax:.2e}, "
          f"G {float((Gt - G64).abs().max()) / gmax:.2e}; a float32 evaluation: Z {float((Z32 - Z64).abs().max()) / zmax:.2e}, "
          f"G {float((G32 - G64).abs().max()) / gmax:.2e} (relative to the largest entry)")
    assert (Zt - Z64).abs().max() <= 1e-12 * zmax
    assert (Gt - G64).abs().max() <= 1e-12 * gmax
