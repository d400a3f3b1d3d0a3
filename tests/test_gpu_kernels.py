"""GPU parity tests, stage by stage: every C entry point against the float64 CPU oracle on seeded inputs."""
import math

import numpy as np
import pytest
import torch

from oracle import FCHLParams, fchl19_representation, fwht, sorf_coefficients
from oracle.qml_oracle import element_types as oracle_element_types
from tests import helpers as H

pytestmark = pytest.mark.gpu

DEV = 'cuda:0'


@pytest.fixture(scope='module')
def cabi():
    from qml_lightning_b200 import cabi
    return cabi


def _cases():
    return {'c0': H.batch_c0(24), 'c1': H.batch_c1(6), 'mixed': H.batch_mixed(40)}


@pytest.mark.parametrize('name', ['c0', 'c1', 'mixed'])
def test_element_types_and_neighbours(cabi, name):
    X, Z, c, species = _cases()[name]
    sp = torch.tensor(species, dtype=torch.float32, device=DEV)
    et = cabi.element_types(X.to(DEV), Z.to(DEV), c.to(DEV), sp).cpu()
    ref = oracle_element_types(Z, species)
    real = torch.arange(Z.shape[1])[None, :] < c[:, None]
    assert torch.equal(et[real].long(), ref[real])
    # neighbour rule 0 < r^2 < rcut^2, ascending j, -1 padding (pairlist_kernel.cu:372-390)
    for rcut in (6.0, 2.5):
        nn = cabi.num_neighbours(X.to(DEV), c.to(DEV), rcut).cpu()
        d2 = ((X[:, :, None, :] - X[:, None, :, :]) ** 2).sum(-1)
        ok = (d2 < np.float32(rcut) ** 2) & (d2 > 0) & real[:, :, None] & real[:, None, :]
        assert torch.equal(nn.long(), ok.sum(-1))
        mx = int(nn.max())
        nl = cabi.neighbour_list(X.to(DEV), c.to(DEV), mx, rcut).cpu()
        for m in range(0, X.shape[0], 7):
            for i in range(int(c[m])):
                want = torch.where(ok[m, i])[0].int()
                assert torch.equal(nl[m, i, :len(want)], want)
                assert (nl[m, i, len(want):] == -1).all()


@pytest.mark.parametrize('name', ['c0', 'c1', 'mixed'])
def test_fchl19_forward_matches_oracle(cabi, name):
    X, Z, c, species = _cases()[name]
    p = H.fchl_params(species)
    ref = fchl19_representation(X.double(), Z, c, p)
    kp = H.kernel_params(p, DEV)
    rep = cabi.fchl19_forward(X.to(DEV), Z.to(DEV), c.to(DEV), kp).cpu().double()
    scale = ref.abs().max()
    assert (rep - ref).abs().max() <= 2e-6 * scale          # fp32 kernel vs fp64 oracle
    real = torch.arange(Z.shape[1])[None, :] < c[:, None]
    assert (rep[~real] == 0).all()                           # padded atoms are zero rows


@pytest.mark.parametrize('name', ['c0', 'c1', 'mixed'])
def test_fchl19_backward_matches_autograd(cabi, name):
    X, Z, c, species = _cases()[name]
    p = H.fchl_params(species)
    x = X.double().clone().requires_grad_(True)
    ref = fchl19_representation(x, Z, c, p)
    g = torch.from_numpy(np.random.default_rng(3).normal(size=tuple(ref.shape))).double() * 0.1
    gX_ref, = torch.autograd.grad((ref * g).sum(), x)
    kp = H.kernel_params(p, DEV)
    gX = cabi.fchl19_backward(X.to(DEV), Z.to(DEV), c.to(DEV), kp, g.float().to(DEV)).cpu().double()
    assert (gX - gX_ref).abs().max() <= 2e-5 * gX_ref.abs().max()
    real = torch.arange(Z.shape[1])[None, :] < c[:, None]
    assert (gX[~real] == 0).all()


def test_fchl19_jacobian_matches_autograd(cabi):
    X, Z, c, species = H.batch_mixed(3, seed=5, max_atoms=9)
    p = H.fchl_params(species, nRs2=6, nRs3=5)
    kp = H.kernel_params(p, DEV)
    rep, jac = cabi.fchl19_forward_jacobian(X.to(DEV), Z.to(DEV), c.to(DEV), kp)
    rep, jac = rep.cpu().double(), jac.cpu().double()
    x = X.double().clone().requires_grad_(True)
    ref = fchl19_representation(x, Z, c, p)
    assert (rep - ref.detach()).abs().max() <= 2e-6 * ref.abs().max()
    nb, A, R = ref.shape
    jref = torch.zeros(nb, A, A, 3, R, dtype=torch.float64)
    for i in range(A):
        for col in range(R):
            gi, = torch.autograd.grad(ref[:, i, col].sum(), x, retain_graph=True)
            jref[:, i, :, :, col] = gi
    assert (jac - jref).abs().max() <= 2e-5 * jref.abs().max()


def test_fchl19_periodic_minimum_image(cabi):
    # A molecule far from the origin in a large box equals the same molecule without a cell (fchl_cuda_kernel.cu:16-49)
    X, Z, c, species = H.batch_c0(4)
    p = H.fchl_params(species)
    kp = H.kernel_params(p, DEV)
    box = 40.0
    cell = torch.eye(3).repeat(4, 1, 1) * box
    inv = torch.eye(3).repeat(4, 1, 1) / box
    Xw = X.clone()
    Xw[:, ::2, 0] += box                                     # wrap every other atom by one box length
    a = cabi.fchl19_forward(X.to(DEV), Z.to(DEV), c.to(DEV), kp).cpu()
    b = cabi.fchl19_forward(Xw.to(DEV), Z.to(DEV), c.to(DEV), kp, cell.to(DEV), inv.to(DEV)).cpu()
    assert (a - b).abs().max() <= 2e-4 * a.abs().max()


@pytest.mark.parametrize('name', ['c0', 'mixed'])
def test_group_by_element_is_a_sorted_permutation(cabi, name):
    X, Z, c, species = _cases()[name]
    elements = species[:-1] if name == 'mixed' else species      # mixed: one species is not a model element
    el = torch.tensor(elements, dtype=torch.float32, device=DEV)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), el)
    ros, sor, gs = g.row_of_slot.cpu(), g.slot_of_row.cpu(), g.group_start.cpu()
    A = Z.shape[1]
    real = (torch.arange(A)[None, :] < c[:, None]).flatten()
    zf = Z.flatten()
    assert g.rows_cap % cabi.ROW_TILE == 0 and int(gs[-1]) <= g.rows_cap
    for ei, e in enumerate(elements):
        slots = torch.where(real & (zf == e))[0]
        rows = ros[slots].long()
        assert int(gs[ei]) % cabi.ROW_TILE == 0
        assert torch.equal(rows, int(gs[ei]) + torch.arange(len(slots)))   # (molecule, atom) order inside the group
        assert torch.equal(sor[rows].long(), slots)
    others = torch.ones_like(real)
    for e in elements:
        others &= ~(real & (zf == e))
    assert (ros[others] == -1).all()
    assert int((sor >= 0).sum()) == int((ros >= 0).sum())


@pytest.mark.parametrize('repsize,npcas', [(336, 128), (780, 256), (50, 16)])
def test_pca_project_both_directions(cabi, repsize, npcas):
    X, Z, c, species = H.batch_mixed(30)
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), el)
    gen = torch.Generator().manual_seed(1)
    red = torch.randn(len(species), repsize, npcas, generator=gen)
    inp = torch.randn(g.rows_cap, repsize, generator=gen)
    out = cabi.pca_project(inp.to(DEV), red.to(DEV), g).cpu().double()
    gs = g.group_start.cpu()
    for ei in range(len(species)):
        r0, r1 = int(gs[ei]), int(gs[ei + 1])
        ref = inp[r0:r1].double() @ red[ei].double()
        assert (out[r0:r1] - ref).abs().max() <= 1e-5 * max(1.0, float(ref.abs().max()))
    back = cabi.pca_project(out.float().to(DEV), red.to(DEV), g, transpose=True).cpu().double()
    for ei in range(len(species)):
        r0, r1 = int(gs[ei]), int(gs[ei + 1])
        ref = out[r0:r1].float().double() @ red[ei].double().T
        assert (back[r0:r1] - ref).abs().max() <= 1e-5 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize('repsize,npcas', [(336, 128), (336, 256), (780, 128), (50, 16), (37, 24)])
def test_pca_tensor_core_kernel_matches_fp32_reference(cabi, repsize, npcas):
    """tcgen05 3xTF32 projection against a float64 product, with the fp32 FFMA kernel as the yardstick: the split
    must keep fp32-level accuracy (a single-pass TF32 product would be ~1e-3)."""
    X, Z, c, species = H.batch_mixed(30, seed=repsize)
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), el)
    gen = torch.Generator().manual_seed(2)
    red = torch.randn(len(species), repsize, npcas, generator=gen)
    inp = torch.randn(g.rows_cap, repsize, generator=gen)
    gs = g.group_start.cpu()
    events_before = cabi.tc_timeouts()
    for transpose, src in ((False, inp), (True, torch.randn(g.rows_cap, npcas, generator=gen))):
        tc = cabi.pca_project(src.to(DEV), red.to(DEV), g, transpose=transpose, tensor_cores=True).cpu().double()
        ff = cabi.pca_project(src.to(DEV), red.to(DEV), g, transpose=transpose).cpu().double()
        for ei in range(len(species)):
            r0, r1 = int(gs[ei]), int(gs[ei + 1])
            ref = src[r0:r1].double() @ (red[ei].double().T if transpose else red[ei].double())
            scale = max(1.0, float(ref.abs().max()))
            assert (ff[r0:r1] - ref).abs().max() <= 3e-6 * scale
            assert (tc[r0:r1] - ref).abs().max() <= 6e-6 * scale
    assert cabi.tc_timeouts() == events_before


@pytest.mark.parametrize('N', [8, 32, 64, 128, 256, 512, 1024, 2048])
@pytest.mark.parametrize('T', [1, 2, 3])
def test_sorf_coefficients_and_backward(cabi, N, T):
    gen = torch.Generator().manual_seed(N + T)
    n, S = 37, 5
    u = torch.randn(n, N, generator=gen)
    D = (torch.randint(0, 2, (T, S, N), generator=gen).float() * 2 - 1)
    norm = math.sqrt(N) / 2.0
    ref = sorf_coefficients(u.double(), D, norm, T)
    out = cabi.sorf_coefficients(u.to(DEV), D.to(DEV), norm, T).cpu().double()
    assert (out - ref).abs().max() <= 1e-5 * ref.abs().max()
    g = torch.randn(n, S, N, generator=gen)
    ud = u.double().clone().requires_grad_(True)
    gref, = torch.autograd.grad((sorf_coefficients(ud, D, norm, T) * g.double()).sum(), ud)
    gout = cabi.sorf_coefficients_backward(g.to(DEV), D.to(DEV), norm, T).cpu().double()
    assert (gout - gref).abs().max() <= 1e-5 * gref.abs().max()


def test_sorf_coefficients_rejects_non_power_of_two(cabi):
    with pytest.raises(RuntimeError, match='power of 2'):        # hadamard_kernel.cu:730
        cabi.sorf_coefficients(torch.zeros(2, 96, device=DEV), torch.ones(1, 2, 96, device=DEV), 1.0, 1)


@pytest.mark.parametrize('order', ['sorted', 'shuffled'])
def test_cos_features_and_backward(cabi, order):
    gen = torch.Generator().manual_seed(5)
    n, F, nmol = 300, 1000, 17
    coeffs = torch.randn(n, F, generator=gen) * 3
    bias = torch.rand(F, generator=gen) * 2 * math.pi
    mol = torch.sort(torch.randint(0, nmol, (n,), generator=gen))[0].int()
    if order == 'shuffled':
        mol = mol[torch.randperm(n, generator=gen)]
    ref = torch.zeros(nmol, F, dtype=torch.float64).index_add(0, mol.long(), math.sqrt(2.0 / F) * torch.cos(coeffs.double() + bias.double()))
    out = cabi.cos_features(coeffs.to(DEV), bias.to(DEV), nmol, mol.to(DEV)).cpu().double()
    assert (out - ref).abs().max() <= 1e-5
    grads = torch.randn(nmol, F, generator=gen)
    gref = grads.double()[mol.long()] * -torch.sin(coeffs.double() + bias.double()) * math.sqrt(2.0 / F)
    gout = cabi.cos_features_backward(grads.to(DEV), coeffs.to(DEV), bias.to(DEV), mol.to(DEV)).cpu().double()
    assert (gout - gref).abs().max() <= 1e-6


@pytest.mark.parametrize('N', [16, 32, 64, 128, 256, 512])
@pytest.mark.parametrize('T', [1, 2, 3])
@pytest.mark.parametrize('fast', [False, True])
def test_fused_sorf_energy_grad(cabi, N, T, fast):
    """Fused kernel vs oracle: per-atom energy and d(energy)/dx for every supported npcas and several [HD] depths."""
    X, Z, c, species = H.batch_mixed(12, seed=N + T)
    nel, S, sigma = len(species), 7, 2.0                         # 7 stacks: exercises the ragged last group of stacks
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), el)
    gen = torch.Generator().manual_seed(N * 10 + T)
    x = torch.randn(g.rows_cap, N, generator=gen) * 1.5
    D = torch.randint(0, 2, (nel, T, S, N), generator=gen).float() * 2 - 1
    bias = torch.rand(nel, S * N, generator=gen) * 2 * math.pi
    alpha = torch.randn(S * N, generator=gen)
    packed = cabi.sorf_pack(D.to(DEV), bias.to(DEV), alpha.to(DEV))
    e_atom, gx = cabi.sorf_energy_grad(x.to(DEV), g, packed, N, S, T, sigma, fast_math=fast)
    e_atom, gx = e_atom.cpu().double(), gx.cpu().double()
    gs, sor = g.group_start.cpu(), g.slot_of_row.cpu()
    F = S * N
    tol = 3e-5 if fast else 5e-6
    for ei in range(nel):
        r0, r1 = int(gs[ei]), int(gs[ei + 1])
        if r1 == r0:
            continue
        xs = x[r0:r1].double().clone().requires_grad_(True)
        cf = sorf_coefficients(xs, D[ei], math.sqrt(N) / sigma, T).reshape(-1, F)
        e_ref = (math.sqrt(2.0 / F) * torch.cos(cf + bias[ei].double()) * alpha.double()).sum(-1)
        g_ref, = torch.autograd.grad(e_ref.sum(), xs)
        live = sor[r0:r1] >= 0
        assert (e_atom[r0:r1][live] - e_ref.detach()[live]).abs().max() <= tol * max(1.0, float(e_ref.abs().max()))
        assert (gx[r0:r1][live] - g_ref[live]).abs().max() <= tol * max(1.0, float(g_ref.abs().max()))
        assert (e_atom[r0:r1][~live] == 0).all()


@pytest.mark.parametrize('N', [32, 128, 256])
@pytest.mark.parametrize('log2_scale,bias_step', [(5, 1.0 / 256), (12, 1.0)])
def test_accurate_sin_cos_on_exactly_representable_large_arguments(cabi, N, log2_scale, bias_step):
    """fast_math=False evaluates sin/cos in float32 without the SFU.  Integer-valued inputs, sign diagonals of +-1, a
    power-of-two scale and a bias on a binary grid make every argument scale*u + b exact in float32, so the only error
    left is the sin/cos evaluation itself: arguments up to 2.5e4 (scale 32: the branch-free reduction) and up to 3e6
    (scale 4096: mostly the large-argument path, the small transforms still on the branch-free one)."""
    X, Z, c, species = H.batch_mixed(10, seed=N)
    nel, S, T = len(species), 6, 1
    sigma = 2.0 ** -log2_scale
    el = torch.tensor(species, dtype=torch.float32, device=DEV)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), el)
    gen = torch.Generator().manual_seed(N + log2_scale)
    x = torch.randint(-3, 4, (g.rows_cap, N), generator=gen).float()
    D = torch.randint(0, 2, (nel, T, S, N), generator=gen).float() * 2 - 1
    bias = torch.randint(0, int(6 / bias_step), (nel, S * N), generator=gen).float() * bias_step
    alpha = torch.randn(S * N, generator=gen)
    packed = cabi.sorf_pack(D.to(DEV), bias.to(DEV), alpha.to(DEV))
    e_atom, gx = cabi.sorf_energy_grad(x.to(DEV), g, packed, N, S, T, sigma, fast_math=False)
    e_atom, gx = e_atom.cpu().double(), gx.cpu().double()
    gs, sor = g.group_start.cpu(), g.slot_of_row.cpu()
    F = S * N
    largest = 0.0
    for ei in range(nel):
        r0, r1 = int(gs[ei]), int(gs[ei + 1])
        if r1 == r0:
            continue
        xs = x[r0:r1].double().clone().requires_grad_(True)
        cf = sorf_coefficients(xs, D[ei], math.sqrt(N) / sigma, T).reshape(-1, F)
        arg = cf + bias[ei].double()
        snap = (arg.detach().float().double() - arg.detach())                 # sqrt(N) / sqrt(N) leaves 1e-16 relative noise
        assert snap.abs().max() <= 1e-9                                        # ... on arguments that are exact in float32
        arg = arg + snap
        largest = max(largest, float(arg.abs().max()))
        e_ref = (math.sqrt(2.0 / F) * torch.cos(arg) * alpha.double()).sum(-1)
        g_ref, = torch.autograd.grad(e_ref.sum(), xs)
        live = sor[r0:r1] >= 0
        assert (e_atom[r0:r1][live] - e_ref.detach()[live]).abs().max() <= 5e-6 * max(1.0, float(e_ref.abs().max()))
        assert (gx[r0:r1][live] - g_ref[live]).abs().max() <= 5e-6 * max(1.0, float(g_ref.abs().max()))
    assert largest > (1e5 if log2_scale == 12 else 1e3)


@pytest.mark.parametrize('repsize,npcas', [(336, 256), (780, 128), (100, 32), (336, 512), (72, 16), (130, 48)])
def test_pca_project_packed_matches_float64(repsize, npcas):
    """The pipeline's projection kernel (pre-split projection matrices, up to 256 columns per block, bulk-copied B
    operand) in both directions: widths that need one column tile, several (512, 780), ragged k chunks (100, 130, 72)
    and a width that is not a multiple of 16 per tile (48 -> tile of 48, 130 -> 144)."""
    from qml_lightning_b200 import cabi
    X, Z, c, species = H.batch_mixed(40, seed=repsize)
    g = cabi.group_by_element(Z.to(DEV), c.to(DEV), torch.tensor(species, dtype=torch.float32, device=DEV))
    gen = torch.Generator().manual_seed(npcas)
    red = torch.randn(len(species), repsize, npcas, generator=gen) / repsize ** 0.5
    gs = g.group_start.cpu()
    events_before = cabi.tc_timeouts()
    for transpose in (False, True):
        src = torch.randn(g.rows_cap, npcas if transpose else repsize, generator=gen)
        out = cabi.pca_project_packed(src.to(DEV), red.to(DEV), g, transpose=transpose).cpu().double()
        for ei in range(len(species)):
            r0, r1 = int(gs[ei]), int(gs[ei + 1])
            if r1 == r0:
                continue
            ref = src[r0:r1].double() @ (red[ei].double().T if transpose else red[ei].double())
            assert (out[r0:r1] - ref).abs().max() <= 3e-6 * max(1.0, float(ref.abs().max()))
    assert cabi.tc_timeouts() == events_before
