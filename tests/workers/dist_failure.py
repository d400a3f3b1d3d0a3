"""Worker of tests/test_cpu_distributed.py::test_failed_rank_is_detected (gloo, CPU): the last rank raises before the
all-reduce of the normal equations; every other rank must come out of the collective with an exception within the
process group's timeout and says so on stdout."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from qml_lightning_b200.utils import distributed as D  # noqa: E402

rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
D.init_process_group('gloo', timeout_s=float(sys.argv[1]), rank=rank, world_size=world)
F = 64
g = torch.Generator().manual_seed(rank)
M = torch.randn(40, F, dtype=torch.float64, generator=g)
ZTZ = torch.triu(M.T @ M)
ZTy = M.T @ torch.randn(40, 1, dtype=torch.float64, generator=g)
if len(sys.argv) > 2 and sys.argv[2] == 'fail' and rank == world - 1:
    raise RuntimeError('injected failure before the all-reduce')
t0 = time.time()
try:
    D.allreduce_normal_equations(ZTZ, ZTy)
except Exception as e:  # gloo reports a closed connection or the timeout as RuntimeError
    print(f'rank {rank}: DETECTED after {time.time() - t0:.1f} s: {type(e).__name__}', flush=True)
    os._exit(0)
ref = sum(torch.triu((m := torch.randn(40, F, dtype=torch.float64, generator=torch.Generator().manual_seed(r))).T @ m)
          for r in range(world))
ref = ref + torch.triu(ref, 1).T
assert torch.allclose(ZTZ, ref, rtol=1e-13, atol=1e-13), 'packed all-reduce differs from the sum of the full matrices'
print(f'rank {rank}: COMPLETED', flush=True)
torch.distributed.destroy_process_group()
