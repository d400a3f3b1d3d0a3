#!/usr/bin/env python
"""Benchmark of the energy+force prediction hot path (FCHL19 -> PCA -> SORF -> energy -> forces).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--conformers M]

Workload (``config.workload`` = "c1"): 10,000 seeded conformers of a 21-atom C9H8O4 molecule per GPU, FCHL19 with
rcut 6.0 / nRs2 24 / nRs3 22, npcas 256, nstacks 256 (65,536 SORF features), fp32.  One step = one pass of the
whole prediction path over that batch.  With N > 1 (torchrun, one rank per GPU) every rank predicts its own batch
and no data-path collective is involved (weak scaling); the reported value is molecules of all ranks divided by the
slowest rank's time.

Prints ONE JSON line.  ``value`` is device-timed with the batch resident in HBM; ``e2e`` goes through the public
model API from pinned host buffers and back; ``roofline`` covers the dominant kernel (fused SORF energy/gradient; for
``--workload c3`` the tensor-core RFF kernel, against the measured dense bf16 rate) timed live with CUDA events; ``cpu_baseline`` is the CPU oracle timed on a bounded sample (rank 0, N = 1 only).
``--impl reference`` times the CPU oracle alone (the upstream project has no CPU implementation of this path, so the
oracle port is the CPU reference).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

NPCAS, NSTACKS, SIGMA = 256, 256, 2.0
SPECIES = [1, 6, 8]
# name -> (species, npcas, nstacks, molecules per GPU (c2: in total), description)
WORKLOADS = {
    'c1': ([1, 6, 8], 256, 256, 10000, '21-atom C9H8O4 conformers, weak scaling'),
    'c0': ([1, 6, 8], 128, 128, 1000, '9-atom conformers'),
    'c2': ([1, 6, 7, 8, 9], 128, 256, 200000, 'mixed molecules with 4-29 atoms, sharded over the ranks (strong scaling)'),
    'c3': ([1, 6, 8], 256, 64, 100000, 'RFF model (dense Gaussian projection, 16,384 features) on the 21-atom conformers, weak scaling'),
    'c4': ([1, 6, 8], 256, 128, 512, 'training normal equations: Z^T Z (fp64, 32768^2) over 21-atom conformers, 64 rows each'),
}
# count, scan, assign, fchl forward, 2 x pca pack, pca (tcgen05), sorf fused or rff (tcgen05), pca^T (tcgen05), fchl backward
KERNELS_PER_STEP = 10


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='c1', choices=sorted(WORKLOADS))
    ap.add_argument('--conformers', type=int, default=0, help='molecules per GPU (0 = the workload default)')
    ap.add_argument('--cpu-sample', type=int, default=256, help='conformers per CPU-baseline step')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    return ap.parse_args()


def workload(nconf, seed, name='c1'):
    from qml_lightning_b200.utils import synthetic as syn
    if name == 'c2':
        return syn.mixed_molecules(seed, nconf)
    X, Z, counts = syn.conformers(seed, syn.C1_CHARGES if name == 'c1' else syn.C0_CHARGES, nconf)
    return X, Z, counts


def algorithmic_bytes_per_atom(repsize, npcas=NPCAS, nstacks=NSTACKS):
    """Inter-stage tensors of the unfused chain written once and read once, plus 40 bytes of input/output."""
    F = npcas * nstacks
    return 4 * (2 * F + 4 * repsize + 4 * npcas) + 40


def sorf_kernel_bytes_per_atom(npcas=NPCAS, nstacks=NSTACKS):
    """Dominant kernel: coefficient tensor out and back, projected input in, gradient out, atom energy."""
    F = npcas * nstacks
    return 4 * (2 * F + 2 * npcas) + 4


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ('index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,'
         'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap')

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits', '-lms', '100',
                                          '-i', str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {'sm_mhz': None, 'sm_max_mhz': None, 'reasons': ['nvidia-smi unavailable']}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(',')]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), f[5:9]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        busy = [s for s in sm if s > 0.5 * max(mx)] if sm else []
        use = busy or sm
        return {'sm_mhz': float(np.median(use)) if use else None, 'sm_max_mhz': max(mx) if mx else None,
                'reasons': sorted(reasons), 'samples': len(sm)}


def build_model(device, X, Z, counts, species=SPECIES, npcas=NPCAS, nstacks=NSTACKS, kind='sorf'):
    """Model through the public API: FCHLCuda + HadamardFeaturesModel (or RandomFourrierFeaturesModel), reductors from
    SVD of our own representation."""
    import qml_lightning_b200 as q
    np.random.seed(1234)
    torch.manual_seed(1234)
    rep = q.FCHLCuda(species=np.array(species), rcut=6.0, nRs2=24, nRs3=22, eta2=0.32, eta3=2.7, two_body_decay=1.8,
                     three_body_weight=13.4, three_body_decay=0.57, device=device)
    if kind == 'rff':
        model = q.RandomFourrierFeaturesModel(rep=rep, elements=np.array(species), sigma=SIGMA, llambda=1e-5, npcas=npcas,
                                              nstacks=nstacks, nbatch_train=64, nbatch_test=len(X))
    else:
        model = q.HadamardFeaturesModel(rep=rep, elements=np.array(species), ntransforms=1, sigma=SIGMA, llambda=1e-5,
                                        npcas=npcas, nstacks=nstacks, nbatch_train=64, nbatch_test=len(X))
    nsub = min(len(X), 2048)      # enough atoms of the rarest species for the SVD
    Xl = [X[i, :counts[i]] for i in range(nsub)]
    Zl = [Z[i, :counts[i]] for i in range(nsub)]
    model.nbatch_train = nsub
    model.get_reductors(Xl, Zl, npcas=npcas, npca_choice=512, nsamples=512, print_info=False)
    model.set_alpha(torch.from_numpy(np.random.default_rng(5).normal(size=model.nfeatures()).astype(np.float32)))
    return rep, model


def cpu_oracle_rate(model, rep, X, Z, counts, nsample, steps=1, warmup=0):
    """Molecules/s of the torch-CPU oracle (fp32, all host threads) on the first ``nsample`` conformers."""
    from oracle import FCHLParams, energy_and_forces
    torch.set_num_threads(os.cpu_count())
    p = FCHLParams(species=SPECIES, rcut=6.0, nRs2=24, nRs3=22, eta2=0.32, eta3=2.7, two_body_decay=1.8,
                   three_body_weight=13.4, three_body_decay=0.57)
    m = dict(kind='sorf', elements=SPECIES, reductors=model.reductors.cpu(), Dmat=model.Dmat.cpu(), bias=model.bias.cpu(),
             alpha=model.alpha.cpu(), sigma=SIGMA, ntransforms=1)
    Xs, Zs, cs = (torch.from_numpy(a[:nsample]) for a in (X, Z, counts))
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        energy_and_forces(Xs, Zs, cs, p, m, batch=16, dtype=torch.float32)
        times.append(time.perf_counter() - t0)
    dt = float(np.mean(times[warmup:]))
    return nsample / dt, dt


def run_reference(args, rank, world):
    """CPU reference arm: the oracle port on the host cores (rank 0 only)."""
    if rank != 0:
        return
    X, Z, counts = workload(max(args.cpu_sample, 64), 1001)
    dev = torch.device('cuda', 0) if torch.cuda.is_available() else None
    if dev is None:
        print(json.dumps({'impl': 'reference', 'unavailable': 'model set-up (reductors) needs the CUDA representation kernel'}))
        return
    rep, model = build_model(dev, X, Z, counts)
    rate, dt = cpu_oracle_rate(model, rep, X, Z, counts, args.cpu_sample, steps=args.steps, warmup=min(args.warmup, 1))
    line = {
        'impl': 'reference', 'metric': 'energy+force predictions', 'value': rate, 'unit': 'molecules/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': min(args.warmup, 1), 'ms_per_step': dt * 1e3, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'c1', 'atoms_per_molecule': 21, 'npcas': NPCAS, 'nstacks': NSTACKS,
                   'features': NPCAS * NSTACKS, 'conformers_per_step': args.cpu_sample},
        'cpu_baseline': {'value': rate, 'unit': 'molecules/s', 'cores': os.cpu_count(), 'kind': 'port',
                         'sample': f'{args.cpu_sample} conformers of the c1 workload per step, torch CPU fp32 oracle'},
        'e2e': {'value': rate, 'unit': 'molecules/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    print(json.dumps(line))


def run_training(args, rank, world, local):
    """c4: normal-equation accumulation over a bounded number of conformers per rank (the full configuration has
    50,000; the cost is linear in the conformers), one all-reduce of the partial sums at the end."""
    dev = torch.device('cuda', local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=dev)
    species, npcas, nstacks, default_n, _ = WORKLOADS['c4']
    n = args.conformers or default_n
    X, Z, counts = workload(n, 1004 + rank, 'c1')
    rep, model = build_model(dev, X, Z, counts, species, npcas, nstacks)
    model.nbatch_train = 64
    rng = np.random.default_rng(7)
    Xl, Zl = [x for x in X], [z for z in Z]
    E = rng.normal(size=n)
    Fl = [rng.normal(size=(21, 3)) for _ in range(n)]
    model.build_Z_components(Xl[:64], Zl[:64], E[:64], Fl[:64], print_info=False)     # warm-up (cuBLAS handle, allocator)
    torch.cuda.synchronize()
    if dist is not None:
        warm = torch.ones(1 << 20, dtype=torch.float64, device=dev)
        dist.all_reduce(warm)                      # communicator set-up stays out of the timed all-reduce
        dist.barrier()
    t0 = time.perf_counter()
    ZTZ, ZTy = model.build_Z_components(Xl, Zl, E, Fl, print_info=False)
    torch.cuda.synchronize()
    t_acc = time.perf_counter() - t0
    t1 = time.perf_counter()
    model.allreduce_normal_equations(ZTZ, ZTy)
    torch.cuda.synchronize()
    t_red = time.perf_counter() - t1
    t2 = time.perf_counter()
    alpha = model.solve_normal_equations(ZTZ, ZTy)      # replicated on every rank
    torch.cuda.synchronize()
    t_solve = time.perf_counter() - t2
    solved = bool(torch.isfinite(alpha).all())
    del ZTZ
    tt = torch.tensor([t_acc, t_red, t_solve], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    if rank == 0:
        F = npcas * nstacks
        t_acc, t_red, t_solve = float(tt[0]), float(tt[1]), float(tt[2])
        flops = 2.0 * 64 * F * F * n * world          # algorithmic: full Z^T Z product per conformer
        print(json.dumps({
            'metric': 'normal-equation accumulation', 'value': n * world / t_acc, 'unit': 'conformers/s', 'n_gpus': world,
            'steps': 1, 'warmup': 1, 'ms_per_step': t_acc * 1e3, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
            'dtype': 'f64', 'data': 'synthetic',
            'config': {'workload': 'c4', 'conformers_per_gpu': n, 'rows_per_conformer': 64, 'features': F, 'nbatch_train': 64},
            'fp64_algorithmic_tflops': flops / t_acc / 1e12, 'allreduce_ms': t_red * 1e3,
            'allreduce_bytes': int(F * F * 8 + F * 8), 'solve_ms': t_solve * 1e3, 'solve_finite': solved,
            'solver': 'Cholesky (potrf + potrs, fp64), llambda 1e-5'}))
    if dist is not None:
        dist.destroy_process_group()


def main():
    args = parse_args()
    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))
    if args.impl == 'reference':
        run_reference(args, rank, world)
        return
    if args.workload == 'c4':
        run_training(args, rank, world, local)
        return
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the prediction path has no CPU fallback')
    dev = torch.device('cuda', local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group('nccl', device_id=dev)

    from qml_lightning_b200 import cabi
    from qml_lightning_b200.utils.sharding import my_shard
    species, npcas, nstacks, default_n, _ = WORKLOADS[args.workload]
    nreq = args.conformers or default_n
    if args.workload == 'c2':
        # one global batch, contiguous atom-balanced shards (strong scaling)
        X, Z, counts = workload(nreq, 1002, 'c2')
        lo, hi = my_shard(counts, rank, world)
        X, Z, counts = X[lo:hi], Z[lo:hi], counts[lo:hi]
        nglobal = nreq
    else:
        X, Z, counts = workload(nreq, 1001 + rank, 'c1' if args.workload == 'c3' else args.workload)  # every rank owns its own molecules
        nglobal = nreq * world
    kind = 'rff' if args.workload == 'c3' else 'sorf'
    rep, model = build_model(dev, X, Z, counts, species, npcas, nstacks, kind)
    nconf, A = Z.shape
    natoms = int(counts.sum())
    kp = rep.kernel_params(dev)
    Xd, Zd, cd = (torch.from_numpy(a).to(dev) for a in (X, Z, counts))
    atomIDs = torch.from_numpy(np.concatenate([np.arange(n, dtype=np.int32) for n in counts])).to(dev)
    molIDs = torch.from_numpy(np.repeat(np.arange(nconf, dtype=np.int32), counts)).to(dev)
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB L2
    E = torch.empty(nconf, dtype=torch.float32, device=dev)
    G = torch.empty(nconf, A, 3, dtype=torch.float32, device=dev)

    def step():
        if kind == 'rff':
            cabi.rff_predict_packed(Xd, Zd, cd, kp, model.species, model.reductors, model.packed, n_atoms_upper=natoms,
                                    fast_math=model.fast_math, energy=E, grad_X=G)
        else:
            cabi.sorf_predict(Xd, Zd, cd, kp, model.species, model.reductors, model.packed, nstacks, 1, SIGMA,
                              n_atoms_upper=natoms, fast_math=model.fast_math, energy=E, grad_X=G)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for s, e in evs:
        flush.fill_(1)          # evict L2 between steps (outside the timed events)
        s.record()
        step()
        e.record()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = float(np.mean([s.elapsed_time(e) for s, e in evs]))
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    value = nglobal / (ms_max * 1e-3)

    # ---- dominant kernel alone, CUDA events on the launching stream -------------------------------------------------
    g = cabi.group_by_element(Zd, cd, model.species, natoms)
    repbuf = torch.empty(g.rows_cap, rep.get_repsize(), dtype=torch.float32, device=dev)
    cabi.fchl19_forward(Xd, Zd, cd, kp, row_of_slot=g.row_of_slot, out=repbuf)
    xproj = cabi.pca_project(repbuf, model.reductors, g)
    def sorf_alone():
        if kind == 'rff':
            cabi.rff_energy_grad_tc(xproj, g, model.packed, len(species), model.fast_math)
        else:
            cabi.sorf_energy_grad(xproj, g, model.packed, npcas, nstacks, 1, SIGMA, model.fast_math)

    for _ in range(3):          # warm-up: also lets the caching allocator keep the output blocks
        sorf_alone()
    torch.cuda.synchronize()
    kev = []
    for _ in range(max(5, min(args.steps, 20))):
        flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        sorf_alone()
        e.record()
        kev.append((s, e))
    torch.cuda.synchronize()
    k_ms = float(np.median([s.elapsed_time(e) for s, e in kev]))

    # ---- end to end through the public API: pinned host -> device -> predict_opt -> host ----------------------------
    hX, hZ, hc = (torch.from_numpy(a).pin_memory() for a in (X, Z, counts))
    hA, hM = atomIDs.cpu().pin_memory(), molIDs.cpu().pin_memory()
    hE = torch.empty(nconf, dtype=torch.float32).pin_memory()
    hF = torch.empty(nconf, A, 3, dtype=torch.float32).pin_memory()
    h2d = sum(t_.numel() * t_.element_size() for t_ in (hX, hZ, hc, hA, hM))
    d2h = hE.numel() * 4 + hF.numel() * 4

    def e2e_step():
        dX, dZ, dc, dA, dM = (t_.to(dev, non_blocking=True) for t_ in (hX, hZ, hc, hA, hM))
        en, fo = model.predict_opt(dX, dZ, dA, dM, dc, forces=True)
        hE.copy_(en, non_blocking=True)
        hF.copy_(fo, non_blocking=True)

    for _ in range(args.warmup):
        e2e_step()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = nglobal / (float(t.item()) * 1e-3)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks, peak_src = {}, 'fallback'
    pk_path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(pk_path):
        with open(pk_path) as fh:
            peaks = json.load(fh)
        peak_src = 'measured'
    hbm = float(peaks.get('hbm_gbs', 6650.0))
    k_bytes = sorf_kernel_bytes_per_atom(npcas, nstacks) * natoms
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    pipe_bytes = algorithmic_bytes_per_atom(rep.get_repsize(), npcas, nstacks) * natoms * world
    pipe_gbs = pipe_bytes / (ms_max * 1e-3) / 1e9
    line = {
        'metric': 'energy+force predictions', 'value': value, 'unit': 'molecules/s', 'n_gpus': world, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': ms_max, 'higher_is_better': True,
        'scaling': 'strong' if args.workload == 'c2' else 'weak', 'vs_baseline': None,
        'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': args.workload, 'molecules_per_gpu': nconf, 'atoms_per_molecule': A if args.workload != 'c2' else 'ragged 4-29 (padded to 29)',
                   'species': species, 'npcas': npcas, 'nstacks': nstacks, 'features': npcas * nstacks,
                   'parallelism': f'molecule shards x{world}, no collective',
                   'l2': 'flushed between steps (512 MB write outside the timed events); per-step workspace > L2',
                   'fast_math': bool(model.fast_math)},
        'e2e': {'value': e2e_value, 'unit': 'molecules/s', 'h2d_bytes_per_step': h2d, 'd2h_bytes_per_step': d2h},
        'gpu_launches': KERNELS_PER_STEP * args.steps,
        'clocks': clocks,
        'roofline': {'bound': 'hbm', 'kernel': 'sorf_energy_grad_kernel', 'achieved': achieved, 'peak': hbm, 'unit': 'GB/s',
                     'frac': achieved / hbm, 'traffic': SORF_KERNEL_DRAM_BYTES_PER_ATOM * natoms if (SORF_KERNEL_DRAM_BYTES_PER_ATOM and args.workload == 'c1') else None,
                     'peak_source': peak_src, 'kernel_ms': k_ms, 'algorithmic_bytes_per_launch': k_bytes,
                     'pipeline_hbm_equivalent_gbs': pipe_gbs / world, 'pipeline_frac': pipe_gbs / world / hbm},
    }
    if kind == 'rff':
        # The dominant kernel is a pair of dense contractions: 2 x (2 npcas D) flops per atom.  `achieved` counts those
        # algorithmic flops; the tensor cores execute three fp16 products for each (hi*hi + hi*lo + lo*hi).
        D = npcas * nstacks
        k_flops = 4.0 * npcas * D * natoms
        tf = k_flops / (k_ms * 1e-3) / 1e12
        peak_tf = float(peaks.get('bf16_tflops', 1590.0))
        line['config']['features'] = D
        line['roofline'] = {'bound': 'tensor', 'kernel': 'rff_tc_kernel', 'achieved': tf, 'peak': peak_tf, 'unit': 'TFLOP/s',
                            'frac': tf / peak_tf, 'traffic': None, 'peak_source': peak_src, 'kernel_ms': k_ms,
                            'algorithmic_flops_per_launch': k_flops, 'issued_mma_tflops': 3.0 * tf,
                            'issued_frac': 3.0 * tf / peak_tf,
                            # whole step: both PCA products and both RFF products, 2 (2 repsize npcas) + 2 (2 npcas D) per atom
                            'pipeline_tflops': (4.0 * rep.get_repsize() * npcas + 4.0 * npcas * D) * natoms / (ms_max * 1e-3) / 1e12}
    if world == 1 and not args.no_cpu_baseline and args.workload == 'c1':
        rate, dt = cpu_oracle_rate(model, rep, X, Z, counts, args.cpu_sample)
        line['cpu_baseline'] = {'value': rate, 'unit': 'molecules/s', 'cores': os.cpu_count(), 'kind': 'port',
                                'sample': f'{args.cpu_sample} conformers of the c1 workload, torch CPU fp32 oracle, {dt:.1f} s'}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


# DRAM bytes per atom of the fused SORF kernel from an ncu capture of one full-size launch (dram__bytes_read.sum +
# dram__bytes_write.sum divided by the atoms of the captured launch: 218.3 MB read + 174.2 MB written for 210,000
# atoms).
SORF_KERNEL_DRAM_BYTES_PER_ATOM = 1869

if __name__ == '__main__':
    main()
