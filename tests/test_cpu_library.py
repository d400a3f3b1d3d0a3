"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, the golden vectors
match the oracle, and the host-side logic (formatting, sharding, model construction, scripting) behaves."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, 'include', 'qmlb200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(qmlb_[a-z0-9_]+)\s*\(', text)))


def test_library_exports_every_declared_symbol():
    from qml_lightning_b200 import _lib
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f'{name} declared in include/qmlb200.h but not exported'
    # and the ctypes table covers the header
    assert set(names) == set(_lib.SIGNATURES), set(names) ^ set(_lib.SIGNATURES)


def test_host_only_entry_points():
    from qml_lightning_b200 import _lib
    lib = _lib.load()
    assert lib.qmlb_version() >= 100
    assert lib.qmlb_fchl19_repsize(3, 24, 22) == 336          # FCHL.py:42
    assert lib.qmlb_fchl19_repsize(5, 24, 22) == 780
    assert lib.qmlb_rows_capacity(1000, 3) % 128 == 0 and lib.qmlb_rows_capacity(1000, 3) >= 1000
    assert lib.qmlb_sorf_pack_bytes(3, 256, 255, 1) == lib.qmlb_sorf_pack_bytes(3, 256, 256, 1)   # stacks padded to pairs
    assert lib.qmlb_predict_workspace_bytes(10000, 21, 210000, 3, 336, 256) > 210000 * (336 + 512) * 4
    # argument validation happens before any device work
    assert lib.qmlb_sorf_coefficients(None, None, 1, 96, 1, 1, 1.0, None, None) == 1
    assert b'null' in lib.qmlb_last_error()


def test_packing_sizes_of_the_tensor_core_stages():
    from qml_lightning_b200 import _lib
    lib = _lib.load()
    # RFF: 256-byte header + one blob per element and 32-feature chunk: fp16 hi and lo images of [npcas, 32] + 3 x 32 floats
    assert lib.qmlb_rff_pack_bytes(3, 256, 16384) == 256 + 3 * 512 * (2 * 256 * 32 * 2 + 384)
    assert lib.qmlb_rff_pack_bytes(3, 256, 1000) == lib.qmlb_rff_pack_bytes(3, 256, 1024)          # features padded to 32
    assert lib.qmlb_rff_pack_bytes(3, 48, 1024) == 0                                               # unsupported npcas
    # PCA: per element, column tile and 32-k chunk the hi and lo TF32 images of [tile columns, 32]
    assert lib.qmlb_pca_pack_bytes(3, 336, 256, 0) == 3 * 1 * 11 * (2 * 256 * 32 * 4)              # 336 -> 11 chunks
    assert lib.qmlb_pca_pack_bytes(3, 336, 256, 1) == 3 * 2 * 8 * (2 * 176 * 32 * 4)               # 336 columns -> 2 tiles of 176
    assert lib.qmlb_pca_pack_bytes(5, 780, 128, 1) == 5 * 4 * 4 * (2 * 208 * 32 * 4)               # 780 columns -> 4 tiles of 208
    assert lib.qmlb_pca_pack(None, 3, 336, 256, 0, None, 0, None) == 1 and b'null' in lib.qmlb_last_error()


def test_missing_library_is_an_error_not_a_fallback(tmp_path):
    import subprocess
    import sys
    env = dict(os.environ, QMLB200_LIB=str(tmp_path / 'nowhere' / 'libqmlb200.so'))
    r = subprocess.run([sys.executable, '-c', 'from qml_lightning_b200 import _lib; _lib.load()'], cwd=ROOT, env=env,
                       capture_output=True, text=True)
    assert r.returncode != 0 and 'no CPU or PyTorch fallback' in r.stderr


def test_torch_operator_schemas_match_upstream_argument_lists():
    import qml_lightning_b200  # noqa: F401
    get = torch._C._jit_get_schemas_for_operator
    assert len(get('qml_lightning_fchl::fchl_forwards')[0].arguments) == 16          # FCHL19.cpp:318-320
    assert len(get('qml_lightning_fchl::get_fchl_and_derivative')[0].arguments) == 17
    assert len(get('qml_lightning_fchl::get_num_neighbours')[0].arguments) == 5
    assert len(get('qml_lightning_fchl::get_neighbour_list')[0].arguments) == 6
    assert len(get('qml_lightning_fchl::get_element_types')[0].arguments) == 4
    assert len(get('qml_lightning_sorf::get_SORF_coefficients')[0].arguments) == 4   # SORF.cpp:138
    assert len(get('qml_lightning_sorf::get_cos_features')[0].arguments) == 4


def test_product_refuses_cpu_tensors():
    from qml_lightning_b200 import cabi
    with pytest.raises(RuntimeError, match='CUDA'):
        cabi.sorf_coefficients(torch.zeros(2, 32), torch.ones(1, 2, 32), 1.0, 1)


def test_product_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, 'qml_lightning_b200')
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(('.py', '.cu', '.cuh', '.cpp', '.h')):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r'^\s*(from|import)\s+oracle\b', src, flags=re.M), os.path.join(dirpath, f)


def test_golden_vectors_match_oracle():
    from oracle import energy_and_forces, fchl19_representation
    from tests import helpers as H
    g = np.load(os.path.join(ROOT, 'tests', 'golden', 'sorf_small.npz'))
    for name in ('c0', 'mixed'):
        X, Z, c = (torch.from_numpy(g[f'{name}_{k}']) for k in ('X', 'Z', 'counts'))
        species = g[f'{name}_species'].tolist()
        p = H.fchl_params(species)
        model = dict(kind='sorf', elements=species, reductors=torch.from_numpy(g[f'{name}_reductors']),
                     Dmat=torch.from_numpy(g[f'{name}_Dmat']), bias=torch.from_numpy(g[f'{name}_bias']),
                     alpha=torch.from_numpy(g[f'{name}_alpha']), sigma=float(g[f'{name}_sigma']),
                     ntransforms=int(g[f'{name}_ntransforms']))
        rep = fchl19_representation(X.double(), Z, c, p)
        E, F = energy_and_forces(X, Z, c, p, model)
        assert np.allclose(rep.numpy(), g[f'{name}_rep'], rtol=1e-12, atol=1e-14)
        assert np.allclose(E.numpy(), g[f'{name}_E'], rtol=1e-10, atol=1e-12)
        assert np.allclose(F.numpy(), g[f'{name}_F'], rtol=1e-9, atol=1e-11)


def test_rff_golden_vectors_match_oracle():
    from oracle import energy_and_forces, training_rows
    from tests import helpers as H
    g = np.load(os.path.join(ROOT, 'tests', 'golden', 'rff_small.npz'))
    X, Z, c = (torch.from_numpy(g[f'c0_{k}']) for k in ('X', 'Z', 'counts'))
    species = g['c0_species'].tolist()
    p = H.fchl_params(species)
    model = dict(kind='rff', elements=species, reductors=torch.from_numpy(g['c0_reductors']), W=torch.from_numpy(g['c0_W']),
                 b=torch.from_numpy(g['c0_b']), alpha=torch.from_numpy(g['c0_alpha']))
    E, F = energy_and_forces(X, Z, c, p, model)
    Zr, Gr = training_rows(X, Z, c, p, model)
    assert np.allclose(E.numpy(), g['c0_E'], rtol=1e-10, atol=1e-12)
    assert np.allclose(F.numpy(), g['c0_F'], rtol=1e-9, atol=1e-11)
    assert np.allclose(Zr.numpy(), g['c0_Zrows'], rtol=1e-10, atol=1e-12)
    assert np.allclose(Gr.numpy(), g['c0_Grows'], rtol=1e-9, atol=1e-11)


def test_oracle_forces_match_finite_differences():
    from oracle import energy_and_forces
    from tests import helpers as H
    X, Z, c, species = H.batch_c0(2, seed=77)
    p = H.fchl_params(species)
    model = H.sorf_model(X, Z, c, p, species, 16, 3)
    E, F = energy_and_forces(X, Z, c, p, model)
    h = 1e-5
    for (m, a, x) in [(0, 0, 0), (1, 4, 2), (0, 8, 1)]:
        Xp, Xm = X.double().clone(), X.double().clone()
        Xp[m, a, x] += h
        Xm[m, a, x] -= h
        Ep = energy_and_forces(Xp, Z, c, p, model, forces=False)
        Em = energy_and_forces(Xm, Z, c, p, model, forces=False)
        fd = -(Ep[m] - Em[m]) / (2 * h)
        assert abs(float(fd) - float(F[m, a, x])) <= 1e-6 * max(1.0, abs(float(fd)))


def test_fwht_is_the_sylvester_hadamard_matrix():
    from oracle import fwht
    from scipy.linalg import hadamard
    for N in (2, 8, 64):
        assert np.array_equal(fwht(torch.eye(N, dtype=torch.float64)).numpy(), hadamard(N).astype(np.float64))


def test_format_data_layout_and_self_energies():
    import qml_lightning_b200 as q
    rep = q.FCHLCuda(species=np.array([1, 6, 8]), nRs3=22, device='cpu')
    model = q.HadamardFeaturesModel(rep=rep, elements=np.array([1, 6, 8]), ntransforms=1, npcas=16, nstacks=2)
    rng = np.random.default_rng(0)
    X = [rng.normal(size=(n, 3)) for n in (3, 5, 1, 4)]
    Q = [rng.choice([1, 6, 8], size=n) for n in (3, 5, 1, 4)]
    F = [rng.normal(size=(n, 3)) for n in (3, 5, 1, 4)]
    E = [1.0, 2.0, 3.0, 4.0]
    d = model.format_data(X, Q, E=E, F=F)
    assert d['coordinates'].shape == (4, 5, 3) and d['coordinates'].dtype == torch.float32
    assert d['charges'].shape == (4, 5) and d['natom_counts'].tolist() == [3, 5, 1, 4]
    assert d['atomIDs'].dtype == torch.int32 and d['molIDs'].dtype == torch.int32
    assert d['atomIDs'].tolist() == [0, 1, 2, 0, 1, 2, 3, 4, 0, 0, 1, 2, 3]
    assert d['molIDs'].tolist() == [0] * 3 + [1] * 5 + [2] + [3] * 4
    for m in range(4):
        n = len(Q[m])
        assert np.allclose(d['coordinates'][m, :n].numpy(), X[m].astype(np.float32))
        assert (d['coordinates'][m, n:] == 0).all() and (d['charges'][m, n:] == 0).all()
        assert np.allclose(d['forces'][m, :n].numpy(), F[m])
    assert d['energies'].dtype == torch.float64 and d['forces'].dtype == torch.float64
    assert d['cells'].shape == (0, 3, 3)
    # self energies (kernel.py:556-599) are subtracted per atom when enabled
    model.calculate_self_energy(Q, E)
    model.set_subtract_self_energies(True)
    d2 = model.format_data(X, Q, E=E)
    se = model.self_energy
    for m in range(4):
        assert abs(float(d2['energies'][m]) - (E[m] - float(se[torch.from_numpy(Q[m]).long()].sum()))) < 1e-9
    # empty batch and single atom are legal
    assert model.format_data([], [])['coordinates'].shape[0] == 0


def test_model_attributes_and_scripting():
    import qml_lightning_b200 as q
    rep = q.FCHLCuda(species=np.array([1, 6, 7, 8]), device='cpu')
    assert rep.get_repsize() == 4 * 24 + 4 * 5 * 20
    assert abs(float(rep.three_body_weight) - np.sqrt(2.7 / np.pi) * 13.4) < 1e-5      # FCHL.py:35
    assert rep.Rs2.shape == (24,) and abs(float(rep.Rs2[-1]) - 6.0) < 1e-6 and float(rep.Rs2[0]) > 0
    m = q.HadamardFeaturesModel(rep=rep, elements=np.array([1, 6, 7, 8]), ntransforms=2, npcas=32, nstacks=4)
    assert m.nfeatures() == 128 and tuple(m.Dmat.shape) == (4, 2, 4, 32) and tuple(m.bias.shape) == (4, 128)
    assert set(torch.unique(m.Dmat).tolist()) == {-1.0, 1.0}
    assert float(m.bias.min()) >= 0 and float(m.bias.max()) <= 2 * np.pi + 1e-6
    assert tuple(m.reductors.shape) == (4, rep.get_repsize(), 32)
    assert m.element2index.tolist()[1] == 0 and m.element2index.tolist()[8] == 3
    scripted = torch.jit.script(m)                       # forward stays scriptable (save_jit_model)
    assert 'sorf_energy' in scripted.code
    with pytest.raises(RuntimeError, match='train'):
        m.predict_opt(torch.zeros(1, 1, 3), torch.zeros(1, 1), torch.zeros(1), torch.zeros(1), torch.ones(1))


def test_shard_bounds_cover_and_balance():
    from qml_lightning_b200.utils.sharding import shard_bounds
    rng = np.random.default_rng(3)
    counts = rng.integers(4, 30, size=1000)
    for world in (1, 2, 3, 8):
        b = shard_bounds(counts, world)
        assert b[0][0] == 0 and b[-1][1] == 1000
        assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
        loads = [counts[s:e].sum() for s, e in b]
        assert max(loads) - min(loads) <= 2 * 29
    assert shard_bounds([5, 5], 4) == [(0, 0), (0, 1), (1, 1), (1, 2)] or sum(e - s for s, e in shard_bounds([5, 5], 4)) == 2
    assert shard_bounds([], 2) == [(0, 0), (0, 0)]
