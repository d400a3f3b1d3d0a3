"""Two-GPU checks (skipped with fewer than two devices): sharded normal equations + NCCL all-reduce, and the
multi-rank benchmark launch."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _torchrun(script_args, port):
    cmd = [sys.executable, '-m', 'torch.distributed.run', '--nnodes=1', '--nproc-per-node', '2', '--master-addr', '127.0.0.1',
           '--master-port', str(port)] + script_args
    env = dict(os.environ, NCCL_NVLS_ENABLE='0')
    return subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_sharded_normal_equations_match_single_rank():
    r = _torchrun([os.path.join(ROOT, 'tests', 'workers', 'dist_normal_equations.py')], 29621)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count('sharded vs full') == 2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_bench_two_ranks_weak_scaling_line():
    r = _torchrun([os.path.join(ROOT, 'bench.py'), '--gpus', '2', '--steps', '2', '--warmup', '3', '--conformers', '2000'], 29622)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith('{')][-1])
    assert line['n_gpus'] == 2 and line['scaling'] == 'weak' and line['value'] > 0
    assert line['config']['molecules_per_gpu'] == 2000


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason='needs two GPUs')
def test_model_on_second_device_while_first_is_current():
    """The ctypes wrappers make the device of their tensors current: a model on cuda:1 predicts and builds training rows
    correctly while cuda:0 is the current device (kernel launches, the cuBLAS handle cache and the built-in scratch
    address are all per current device)."""
    import numpy as np
    import tests.test_gpu_models as tm
    from oracle import energy_and_forces
    from tests import helpers as H
    X, Z, c, species = H.batch_mixed(12, seed=71, max_atoms=9)
    old = tm.DEV
    tm.DEV = 'cuda:1'
    try:
        torch.cuda.set_device(0)
        p, ref, m = tm.build_model(X, Z, c, species, 32, 4)
        E_ref, F_ref = energy_and_forces(X, Z, c, p, ref)
        atomIDs, molIDs = tm.ids(c, X.shape[1])
        E, F = m.predict_opt(X.to('cuda:1'), Z.to('cuda:1'), atomIDs, molIDs, c.to('cuda:1'))
        assert torch.cuda.current_device() == 0
        assert ((E.cpu().double() - E_ref).abs() <= H.energy_tolerance(E_ref)).all()
        assert (F.cpu().double() - F_ref).abs().max() <= 1e-4
        Xl = [X[i, :int(c[i])].numpy() for i in range(12)]
        Zl = [Z[i, :int(c[i])].numpy() for i in range(12)]
        rng = np.random.default_rng(0)
        A, y = m.build_Z_components(Xl, Zl, rng.normal(size=12), [rng.normal(size=(int(c[i]), 3)) for i in range(12)], print_info=False)
        assert A.device == torch.device('cuda:1') and bool(torch.isfinite(A).all()) and float(A.abs().max()) > 0
    finally:
        tm.DEV = old
