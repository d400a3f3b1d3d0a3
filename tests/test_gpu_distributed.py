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
