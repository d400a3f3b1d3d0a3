"""Worker of tests/test_gpu_distributed.py: every rank accumulates the normal equations of its molecule shard, the
partial sums are combined with one NCCL all-reduce, and the result must equal the single-rank accumulation."""
import os, sys, torch, numpy as np
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import torch.distributed as dist
rank = int(os.environ['RANK']); world = int(os.environ['WORLD_SIZE']); local = int(os.environ['LOCAL_RANK'])
torch.cuda.set_device(local)
from qml_lightning_b200.utils.distributed import init_process_group
init_process_group('nccl', timeout_s=120, device=torch.device('cuda', local))
from tests import helpers as H
from tests.test_gpu_models import build_model
import tests.test_gpu_models as tm
tm.DEV = f'cuda:{local}'
X, Z, c, species = H.batch_mixed(40, seed=12, max_atoms=8)
p, ref, m = build_model(X, Z, c, species, 32, 2)
Xl = [X[i, :int(c[i])].numpy() for i in range(40)]; Zl = [Z[i, :int(c[i])].numpy() for i in range(40)]
rng = np.random.default_rng(0); E = rng.normal(size=40); Fl = [rng.normal(size=(int(c[i]),3)) for i in range(40)]
m.nbatch_train = 7
A1, y1 = m.build_Z_components(Xl, Zl, E, Fl, print_info=False, distributed=False)
A2, y2 = m.build_Z_components(Xl, Zl, E, Fl, print_info=False, distributed=True)
err = float((A1 - A2).abs().max() / A1.abs().max()); erry = float((y1 - y2).abs().max() / y1.abs().max())
print(f'rank {rank}: sharded vs full ZTZ rel err {err:.3e}, ZTy {erry:.3e}')
assert err < 1e-12 and erry < 1e-12
assert float((A2 - A2.T).abs().max()) == 0.0
# train(distributed=True): rank 0 solves, every rank receives the same weights; equal to the single-rank solve
m.train(Xl, Zl, E, Fl, print_info=False, distributed=True)
a_dist = m.alpha.clone()
m.train(Xl, Zl, E, Fl, print_info=False, distributed=False)
assert float((a_dist - m.alpha).abs().max()) <= 1e-8 * float(m.alpha.abs().max())
dist.destroy_process_group()
