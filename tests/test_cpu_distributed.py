"""world_size-2 gloo test of the multi-rank logic bench.py relies on: disjoint molecule shards, barrier, and the
max-over-ranks reduction of the timed region (no data-path collective)."""
import os
import socket
import subprocess
import sys
import time

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


def _worker(rank, world, port, counts, out_dir):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    from qml_lightning_b200.utils.sharding import my_shard
    s, e = my_shard(counts, rank, world)
    # "work": a per-rank partial result that needs no exchange, plus a fake per-rank time
    partial = torch.tensor([float(np.sum(counts[s:e]))], dtype=torch.float64)
    t = torch.tensor([10.0 + rank], dtype=torch.float64)
    dist.barrier()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    gathered = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(gathered, partial)
    np.save(os.path.join(out_dir, f'r{rank}.npy'), np.array([s, e, float(t), float(sum(g.item() for g in gathered))]))
    dist.destroy_process_group()


def test_two_rank_sharding_and_max_time(tmp_path):
    counts = np.random.default_rng(1).integers(4, 30, size=257)
    port = _free_port()
    mp.spawn(_worker, args=(2, port, counts, str(tmp_path)), nprocs=2, join=True)
    r0, r1 = (np.load(tmp_path / f'r{r}.npy') for r in (0, 1))
    assert r0[0] == 0 and r0[1] == r1[0] and r1[1] == 257          # disjoint, contiguous, complete
    assert r0[2] == r1[2] == 11.0                                   # max over ranks
    assert r0[3] == r1[3] == float(counts.sum())


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(world, timeout_s, mode):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR='127.0.0.1', MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, os.path.join(ROOT, 'tests', 'workers', 'dist_failure.py'), str(timeout_s), mode],
                                      env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    return procs


def test_packed_allreduce_of_normal_equations_two_ranks():
    """Healthy run: the all-reduce of the packed triangle equals the sum of the full matrices, mirrored."""
    outs = [p.communicate(timeout=120) for p in _launch(2, 30, 'ok')]
    assert all('COMPLETED' in o[0] for o in outs), outs


def test_failed_rank_is_detected():
    """Failure detection on the host: rank 1 raises before the all-reduce; rank 0 must get an exception from the
    collective within the group's timeout instead of waiting for ever."""
    t0 = time.time()
    procs = _launch(2, 8, 'fail')
    out0, err0 = procs[0].communicate(timeout=90)
    out1, err1 = procs[1].communicate(timeout=90)
    assert procs[1].returncode != 0 and 'injected failure' in err1
    assert procs[0].returncode == 0 and 'DETECTED' in out0, (out0, err0[-2000:])
    assert time.time() - t0 < 80
