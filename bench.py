#!/usr/bin/env python
"""Benchmark of the energy+force prediction hot path (FCHL19 -> PCA -> SORF -> energy -> forces).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c0..c4] [--no-extras]

Headline workload (``config.workload`` = "c1"): 10,000 seeded conformers of a 21-atom C9H8O4 molecule per GPU, FCHL19
with rcut 6.0 / nRs2 24 / nRs3 22, npcas 256, nstacks 256 (65,536 SORF features), fp32.  One step = one pass of the
whole prediction path over that batch.  With N > 1 (torchrun, one rank per GPU) every rank predicts its own batch and
no data-path collective is involved (weak scaling); the reported value is molecules of all ranks divided by the
slowest rank's time.

Prints ONE JSON line.  ``value`` is device-timed with the batch resident in HBM; ``e2e`` goes through the public model
API from pinned host buffers and back; ``roofline`` covers the dominant kernel (fused SORF energy/gradient) timed live
with CUDA events, as the HBM-equivalent fraction of the contract and as the physical FP32-pipe fraction;
``cpu_baseline`` is the CPU oracle timed on a bounded sample (rank 0, N = 1 only).  ``extra`` carries the other
configurations, each measured in the same process after the headline:

* ``c2``  200,000 mixed molecules (4-29 atoms, five species) sharded over the N ranks by atom count (strong scaling);
* ``c4``  training: float64 normal equations at 32,768 features -- accumulation of 64 conformers per rank (in-tree
          DMMA kernel and cuBLAS DSYRK back to back), the NCCL all-reduce of the packed triangle, the solve on rank 0;
* at N = 1 also ``c0`` (1,000 9-atom conformers), ``c3`` (RFF model, 100,000 conformers, tensor-core kernel against
  the measured dense bf16 rate), ``c1_accurate`` (the headline with accurate sin/cos instead of the SFU) and
  ``reference_cuda``: upstream's own CUDA operators with the 72-byte shared-memory allocation fix of
  baseline/build_ref.py, timed on identical inputs in a child process, with the three parity distances (present only
  when those operator libraries have been built).

``--impl reference`` times the CPU oracle alone, without touching CUDA (the upstream project has no CPU implementation
of this path, so the oracle port is the CPU reference).
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

SIGMA = 2.0
FCHL = dict(rcut=6.0, nRs2=24, nRs3=22, eta2=0.32, eta3=2.7, two_body_decay=1.8, three_body_weight=13.4, three_body_decay=0.57)
# name -> (species, npcas, nstacks, molecules per GPU (c2: in total), description)
WORKLOADS = {
    'c1': ([1, 6, 8], 256, 256, 10000, '21-atom C9H8O4 conformers, weak scaling'),
    'c0': ([1, 6, 8], 128, 128, 1000, '9-atom conformers'),
    'c2': ([1, 6, 7, 8, 9], 128, 256, 200000, 'mixed molecules with 4-29 atoms, sharded over the ranks (strong scaling)'),
    'c3': ([1, 6, 8], 256, 64, 100000, 'RFF model (dense Gaussian projection, 16,384 features) on the 21-atom conformers, weak scaling'),
    'c4': ([1, 6, 8], 256, 128, 64, 'training normal equations: Z^T Z (fp64, 32768^2) over 21-atom conformers, 64 rows each'),
}
# group (count, scan, assign; one launch for batches of at most 1,024 molecules), fchl forward, pca (tcgen05),
# sorf fused or rff (tcgen05), pca^T (tcgen05), fchl backward
KERNELS_PER_STEP = 8
KERNELS_PER_STEP_SMALL = 6
# DRAM bytes per atom of the fused SORF kernel from an ncu capture of one full-size c1 launch (dram__bytes_read.sum +
# dram__bytes_write.sum divided by the atoms of the captured launch: 218.3 MB read + 174.2 MB written for 210,000 atoms).
SORF_KERNEL_DRAM_BYTES_PER_ATOM = 1869
SM_COUNT, FP32_LANES_PER_SM = 148, 128


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=10)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours', choices=['ours', 'reference'])
    ap.add_argument('--workload', default='c1', choices=sorted(WORKLOADS))
    ap.add_argument('--conformers', type=int, default=0, help='molecules per GPU (0 = the workload default)')
    ap.add_argument('--cpu-sample', type=int, default=1000, help='conformers of the CPU-baseline sample')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-extras', action='store_true', help='headline workload only')
    ap.add_argument('--nstacks', type=int, default=0, help='c4 only: override the stack count (small cases for profiling)')
    ap.add_argument('--rows-only', action='store_true', help='c4 only: training rows without the normal equations')
    return ap.parse_args()


def workload(nconf, seed, name='c1'):
    from qml_lightning_b200.utils import synthetic as syn
    if name == 'c2':
        return syn.mixed_molecules(seed, nconf)
    return syn.conformers(seed, syn.C0_CHARGES if name == 'c0' else syn.C1_CHARGES, nconf)


def repsize_of(species):
    n = len(species)
    return n * FCHL['nRs2'] + n * (n + 1) * FCHL['nRs3']


def algorithmic_bytes_per_atom(repsize, npcas, nstacks):
    """Inter-stage tensors of the unfused chain written once and read once, plus 40 bytes of input/output."""
    F = npcas * nstacks
    return 4 * (2 * F + 4 * repsize + 4 * npcas) + 40


def sorf_kernel_bytes_per_atom(npcas, nstacks):
    """Dominant kernel: coefficient tensor out and back, projected input in, gradient out, atom energy."""
    F = npcas * nstacks
    return 4 * (2 * F + 2 * npcas) + 4


def sorf_fp32_lane_ops_per_atom(npcas, nstacks, ntransforms=1):
    """FP32 lane operations the fused SORF kernel cannot avoid, per atom: per stack and transform one sign flip per
    element and N log2 N butterfly additions on the way forward and the same on the way back (2 T (N + N log2 N)),
    plus per stack the argument FMA, the two range-reduced SFU results scaled by the weight (energy FMA, gradient
    multiply) and the accumulation of the stack's gradient into the atom's (4 N).  Transcendentals themselves run on
    the SFU and are not counted."""
    N, S, T = npcas, nstacks, ntransforms
    return S * (2 * T * (N + N * int(np.log2(N))) + 4 * N)


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


def build_model(device, X, Z, counts, species, npcas, nstacks, kind='sorf', fast_math=True):
    """Model through the public API: FCHLCuda + HadamardFeaturesModel (or RandomFourrierFeaturesModel), reductors from
    SVD of our own representation."""
    import qml_lightning_b200 as q
    np.random.seed(1234)
    torch.manual_seed(1234)
    rep = q.FCHLCuda(species=np.array(species), device=device, **FCHL)
    if kind == 'rff':
        model = q.RandomFourrierFeaturesModel(rep=rep, elements=np.array(species), sigma=SIGMA, llambda=1e-5, npcas=npcas,
                                              nstacks=nstacks, nbatch_train=64, nbatch_test=len(X), fast_math=fast_math)
    else:
        model = q.HadamardFeaturesModel(rep=rep, elements=np.array(species), ntransforms=1, sigma=SIGMA, llambda=1e-5,
                                        npcas=npcas, nstacks=nstacks, nbatch_train=64, nbatch_test=len(X), fast_math=fast_math)
    nsub = min(len(X), 2048)      # enough atoms of the rarest species for the SVD
    Xl = [X[i, :counts[i]] for i in range(nsub)]
    Zl = [Z[i, :counts[i]] for i in range(nsub)]
    model.nbatch_train = nsub
    model.get_reductors(Xl, Zl, npcas=npcas, npca_choice=512, nsamples=512, print_info=False)
    model.nbatch_train = 64
    model.set_alpha(torch.from_numpy(np.random.default_rng(5).normal(size=model.nfeatures()).astype(np.float32)))
    return rep, model


def _load_by_path(name, *relpath):
    """Import one source file without importing the package around it (the package loads the CUDA libraries)."""
    import importlib.util
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, *relpath))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def cpu_oracle_rate(species, npcas, nstacks, X, Z, counts, reductors, Dmat, bias, alpha, nsample, steps=1, warmup=0):
    """Molecules/s of the torch-CPU oracle (fp32, all host threads) on the first ``nsample`` molecules; CPU tensors only."""
    from oracle import FCHLParams, energy_and_forces
    torch.set_num_threads(os.cpu_count())
    p = FCHLParams(species=species, **FCHL)
    m = dict(kind='sorf', elements=species, reductors=reductors, Dmat=Dmat, bias=bias, alpha=alpha, sigma=SIGMA, ntransforms=1)
    Xs, Zs, cs = (torch.from_numpy(np.ascontiguousarray(a[:nsample])) for a in (X, Z, counts))
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        energy_and_forces(Xs, Zs, cs, p, m, batch=16, dtype=torch.float32)
        times.append(time.perf_counter() - t0)
    dt = float(np.mean(times[warmup:]))
    return nsample / dt, dt


def run_reference(args, rank, world):
    """CPU reference arm: the oracle port on the host cores (rank 0 only), no CUDA library loaded and no CUDA call made.
    Same model configuration as the headline (species, FCHL19 parameters, npcas 256, nstacks 256); the projection
    matrices are random orthonormal columns instead of an SVD of representations (same shapes, same arithmetic cost).
    A step is a bounded sample of the 10,000-conformer batch, sized from a short trial so that the whole run stays
    within about three minutes."""
    if rank != 0:
        return
    syn = _load_by_path('qmlb200_synthetic', 'qml_lightning_b200', 'utils', 'synthetic.py')
    species, npcas, nstacks, nfull, _ = WORKLOADS['c1']
    X, Z, counts = syn.conformers(1001, syn.C1_CHARGES, 1024)
    red = torch.from_numpy(syn.random_orthonormal_reductors(3, len(species), repsize_of(species), npcas))
    D, bias, alpha = (torch.from_numpy(a) for a in syn.sorf_parameters(4, len(species), npcas, nstacks, 1))
    trial_rate, _ = cpu_oracle_rate(species, npcas, nstacks, X, Z, counts, red, D, bias, alpha, 32)
    warm = min(args.warmup, 1)
    budget_s = 150.0
    sample = int(max(32, min(1000, budget_s * trial_rate / (args.steps + warm))))
    rate, dt = cpu_oracle_rate(species, npcas, nstacks, X, Z, counts, red, D, bias, alpha, sample, steps=args.steps, warmup=warm)
    # c0 in full: 1,000 conformers of the 9-atom molecule, 16,384 features
    s0, n0, st0, nc0, _ = WORKLOADS['c0']
    X0, Z0, c0 = syn.conformers(1000, syn.C0_CHARGES, nc0)
    red0 = torch.from_numpy(syn.random_orthonormal_reductors(5, len(s0), repsize_of(s0), n0))
    D0, b0, a0 = (torch.from_numpy(a) for a in syn.sorf_parameters(6, len(s0), n0, st0, 1))
    rate0, dt0 = cpu_oracle_rate(s0, n0, st0, X0, Z0, c0, red0, D0, b0, a0, nc0)
    line = {
        'impl': 'reference', 'metric': 'energy+force predictions', 'value': rate, 'unit': 'molecules/s', 'n_gpus': args.gpus,
        'steps': args.steps, 'warmup': warm, 'ms_per_step': dt * 1e3, 'higher_is_better': True,
        'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': 'c1', 'atoms_per_molecule': 21, 'species': species, 'npcas': npcas, 'nstacks': nstacks,
                   'features': npcas * nstacks, 'conformers_per_step': sample,
                   'same_config': {'model': True, 'fchl19_parameters': True, 'precision': 'f32',
                                   'molecules_per_step': f'{sample} of the headline batch of {nfull} (bounded CPU sample; the rate '
                                                         'does not depend on the batch size)',
                                   'projection_matrices': 'random orthonormal (the GPU arm takes them from an SVD); same shapes',
                                   'warmup': f'{warm} of the requested {args.warmup} (each CPU step takes {dt:.1f} s)'}},
        'cpu_baseline': {'value': rate, 'unit': 'molecules/s', 'cores': os.cpu_count(), 'kind': 'port',
                         'sample': f'{sample} conformers of the c1 workload per step, torch CPU fp32 oracle, no CUDA'},
        'e2e': {'value': rate, 'unit': 'molecules/s', 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
        'extra': {'c0': {'value': rate0, 'unit': 'molecules/s', 'ms_per_step': dt0 * 1e3,
                         'sample': f'all {nc0} conformers of the 9-atom workload, one pass'}},
    }
    print(json.dumps(line))


class Dist:
    """The few collective calls the benchmark needs (barrier, max over ranks); no-ops with one rank."""

    def __init__(self, world, dev):
        self.world, self.dev, self.d = world, dev, None
        if world > 1:
            import torch.distributed as d
            from qml_lightning_b200.utils.distributed import init_process_group
            init_process_group('nccl', device=dev)
            self.d = d

    def barrier(self):
        if self.d is not None:
            self.d.barrier()

    def max(self, values):
        t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=self.dev)
        if self.d is not None:
            self.d.all_reduce(t, op=self.d.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def close(self):
        if self.d is not None:
            self.d.destroy_process_group()


def time_prediction(name, dev, dist, rank, steps, warmup, X, Z, counts, nglobal, fast_math=True, sampler=None, e2e=True):
    """Device-timed steps, the dominant kernel alone and the end-to-end API path of one workload on this rank's molecules.
    Returns a dict; times are the max over ranks."""
    from qml_lightning_b200 import cabi
    species, npcas, nstacks, _, _ = WORKLOADS[name]
    kind = 'rff' if name == 'c3' else 'sorf'
    rep, model = build_model(dev, X, Z, counts, species, npcas, nstacks, kind, fast_math)
    nconf, A = Z.shape
    natoms = int(counts.sum())
    kp = rep.kernel_params(dev)
    Xd, Zd, cd = (torch.from_numpy(np.ascontiguousarray(a)).to(dev) for a in (X, Z, counts))
    atomIDs = torch.from_numpy(np.concatenate([np.arange(n, dtype=np.int32) for n in counts])).to(dev)
    molIDs = torch.from_numpy(np.repeat(np.arange(nconf, dtype=np.int32), counts)).to(dev)
    flush = torch.empty(512 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB L2
    E = torch.empty(nconf, dtype=torch.float32, device=dev)
    G = torch.empty(nconf, A, 3, dtype=torch.float32, device=dev)
    pca_packed = model.pca_packed()

    def step():
        if kind == 'rff':
            cabi.rff_predict_packed(Xd, Zd, cd, kp, model.species, model.reductors, model.packed, n_atoms_upper=natoms,
                                    fast_math=model.fast_math, energy=E, grad_X=G, pca_packed=pca_packed)
        else:
            cabi.sorf_predict(Xd, Zd, cd, kp, model.species, model.reductors, model.packed, nstacks, 1, SIGMA,
                              n_atoms_upper=natoms, fast_math=model.fast_math, energy=E, grad_X=G, pca_packed=pca_packed)

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    if sampler is not None:
        sampler.start()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s, e in evs:
        flush.fill_(1)          # evict L2 between steps (outside the timed events)
        s.record()
        step()
        e.record()
    torch.cuda.synchronize()
    dist.barrier()
    clocks = sampler.stop() if sampler is not None else None
    ms = float(np.mean([s.elapsed_time(e) for s, e in evs]))

    # ---- dominant kernel alone, CUDA events on the launching stream -------------------------------------------------
    g = cabi.group_by_element(Zd, cd, model.species, natoms)
    repbuf = torch.empty(g.rows_cap, rep.get_repsize(), dtype=torch.float32, device=dev)
    cabi.fchl19_forward(Xd, Zd, cd, kp, row_of_slot=g.row_of_slot, out=repbuf)
    xproj = cabi.pca_project(repbuf, model.reductors, g)

    def feature_stage():
        if kind == 'rff':
            cabi.rff_energy_grad_tc(xproj, g, model.packed, len(species), model.fast_math)
        else:
            cabi.sorf_energy_grad(xproj, g, model.packed, npcas, nstacks, 1, SIGMA, model.fast_math)

    for _ in range(3):          # warm-up: also lets the caching allocator keep the output blocks
        feature_stage()
    torch.cuda.synchronize()
    kev = []
    for _ in range(max(5, min(steps, 20))):
        flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        feature_stage()
        e.record()
        kev.append((s, e))
    torch.cuda.synchronize()
    k_ms = float(np.median([s.elapsed_time(e) for s, e in kev]))
    del repbuf, xproj

    # ---- end to end through the public API: pinned host -> device -> predict_opt -> host ----------------------------
    e2e_ms, h2d, d2h = None, 0, 0
    if e2e:
        hX, hZ, hc = (torch.from_numpy(np.ascontiguousarray(a)).pin_memory() for a in (X, Z, counts))
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

        for _ in range(warmup):
            e2e_step()
        torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    ms_max, e2e_max, natoms_max = dist.max([ms, e2e_ms or 0.0, natoms])
    del flush
    return dict(model=model, rep=rep, ms=ms_max, ms_local=ms, kernel_ms=k_ms, e2e_ms=e2e_max if e2e else None, h2d=h2d, d2h=d2h,
                natoms=natoms, natoms_max=int(natoms_max), nconf=nconf, A=A, clocks=clocks, species=species, npcas=npcas,
                nstacks=nstacks, kind=kind, value=nglobal / (ms_max * 1e-3),
                e2e_value=(nglobal / (e2e_max * 1e-3)) if e2e else None)


def peaks():
    pk, src = {}, 'fallback'
    path = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(path):
        with open(path) as fh:
            pk = json.load(fh)
        src = 'measured'
    return float(pk.get('hbm_gbs', 6650.0)), float(pk.get('bf16_tflops', 1590.0)), src


def sorf_roofline(r, world, sm_mhz):
    """Roofline block of a SORF workload: HBM-equivalent fraction of the contract and physical FP32-pipe fraction."""
    hbm, _, src = peaks()
    k_bytes = sorf_kernel_bytes_per_atom(r['npcas'], r['nstacks']) * r['natoms']
    achieved = k_bytes / (r['kernel_ms'] * 1e-3) / 1e9
    pipe_bytes = algorithmic_bytes_per_atom(repsize_of(r['species']), r['npcas'], r['nstacks']) * r['natoms_max']
    pipe_gbs = pipe_bytes / (r['ms'] * 1e-3) / 1e9
    lane_ops = sorf_fp32_lane_ops_per_atom(r['npcas'], r['nstacks']) * r['natoms']
    clock = (sm_mhz or 1965.0) * 1e6
    fp32_peak = SM_COUNT * FP32_LANES_PER_SM * clock
    return {'bound': 'hbm', 'kernel': 'sorf_energy_grad_kernel', 'achieved': achieved, 'peak': hbm, 'unit': 'GB/s',
            'frac': achieved / hbm, 'peak_source': src, 'kernel_ms': r['kernel_ms'], 'algorithmic_bytes_per_launch': k_bytes,
            'traffic': SORF_KERNEL_DRAM_BYTES_PER_ATOM * r['natoms'] if (r['npcas'], r['nstacks']) == (256, 256) else None,
            'pipeline_hbm_equivalent_gbs': pipe_gbs, 'pipeline_frac': pipe_gbs / hbm,
            'physical': {'bound': 'fp32 pipe', 'lane_ops_per_launch': lane_ops,
                         'achieved_lane_ops_per_s': lane_ops / (r['kernel_ms'] * 1e-3),
                         'peak_lane_ops_per_s': fp32_peak, 'frac': lane_ops / (r['kernel_ms'] * 1e-3) / fp32_peak,
                         'clock_mhz': clock / 1e6,
                         'note': 'minimum FP32 lane operations of the fused kernel (butterflies, sign flips, per-element FMAs) '
                                 'over SMs x 128 lanes x sampled SM clock; the HBM-equivalent frac above counts a coefficient '
                                 'stream that the fused kernel never writes'}}


def rff_roofline(r):
    """The dominant kernel is a pair of dense contractions: 2 x (2 npcas D) flops per atom.  ``achieved`` counts those
    algorithmic flops; the tensor cores execute three fp16 products for each (hi*hi + hi*lo + lo*hi)."""
    _, peak_tf, src = peaks()
    D = r['npcas'] * r['nstacks']
    k_flops = 4.0 * r['npcas'] * D * r['natoms']
    tf = k_flops / (r['kernel_ms'] * 1e-3) / 1e12
    return {'bound': 'tensor', 'kernel': 'rff_tc_kernel', 'achieved': tf, 'peak': peak_tf, 'unit': 'TFLOP/s', 'frac': tf / peak_tf,
            'traffic': None, 'peak_source': src, 'kernel_ms': r['kernel_ms'], 'algorithmic_flops_per_launch': k_flops,
            'issued_mma_tflops': 3.0 * tf, 'issued_frac': 3.0 * tf / peak_tf,
            # whole step: both PCA products and both RFF products, 2 (2 repsize npcas) + 2 (2 npcas D) per atom
            'pipeline_tflops': (4.0 * repsize_of(r['species']) * r['npcas'] + 4.0 * r['npcas'] * D) * r['natoms_max']
                               / (r['ms'] * 1e-3) / 1e12}


def run_c4(dev, dist, rank, world, nconf, nstacks_override=0, rows_only=False):
    """Training normal equations at 32,768 features: ``nconf`` conformers on every rank (64 rows each), accumulated with
    the in-tree float64 kernel (and, for comparison, cuBLAS DSYRK on the same rows), one all-reduce of the packed
    triangle, the Cholesky solve on rank 0 and the broadcast of the weights."""
    from qml_lightning_b200 import cabi
    from qml_lightning_b200.utils import distributed as D
    species, npcas, nstacks, _, _ = WORKLOADS['c4']
    nstacks = nstacks_override or nstacks
    X, Z, counts = workload(nconf, 1004 + rank, 'c1')
    rep, model = build_model(dev, X, Z, counts, species, npcas, nstacks)
    F = npcas * nstacks
    rng = np.random.default_rng(7 + rank)
    data = model.format_data([x for x in X], [z for z in Z], E=rng.normal(size=nconf), F=[rng.normal(size=(21, 3)) for _ in range(nconf)])

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def timed(fn):
        s, e = ev(), ev()
        s.record()
        out = fn()
        e.record()
        torch.cuda.synchronize()
        return out, s.elapsed_time(e)

    model.training_rows(data, with_forces=True)                                  # warm-up
    (Ztrain, Gtrain), rows_ms = timed(lambda: model.training_rows(data, with_forces=True))
    if rows_only:
        return {'workload': 'c4', 'features': F, 'conformers_per_gpu': nconf, 'training_rows_ms': dist.max([rows_ms])[0],
                'conformers_per_s': nconf * world / (rows_ms * 1e-3), 'accumulate_ms': 0.0}
    rows = torch.cat((Ztrain, Gtrain.reshape(-1, F)), dim=0)
    targets = torch.cat((data['energies'], data['forces'].flatten())).contiguous()
    del Ztrain, Gtrain
    ZTZ = torch.zeros(F, F, device=dev, dtype=torch.float64)
    ZTy = torch.zeros(F, 1, device=dev, dtype=torch.float64)
    cabi.normal_equations_accumulate(rows, targets, ZTZ, ZTy)                    # warm-up, discarded
    ZTZ.zero_()
    ZTy.zero_()
    _, own_ms = timed(lambda: cabi.normal_equations_accumulate(rows, targets, ZTZ, ZTy))
    lib = torch.zeros(F, F, device=dev, dtype=torch.float64)
    liby = torch.zeros(F, 1, device=dev, dtype=torch.float64)
    cabi.normal_equations_accumulate(rows, targets, lib, liby, library=True)     # warm-up (handle creation)
    lib.zero_()
    liby.zero_()
    _, lib_ms = timed(lambda: cabi.normal_equations_accumulate(rows, targets, lib, liby, library=True))
    sample = slice(0, 4096)
    agree = float((torch.triu(ZTZ[sample, sample]) - torch.triu(lib[sample, sample])).abs().max() / lib[sample, sample].abs().max())
    del lib, liby
    dist.barrier()
    if world > 1:                                                                # communicator set-up stays out of the timing
        warm = torch.ones(1 << 20, dtype=torch.float64, device=dev)
        dist.d.all_reduce(warm)
        torch.cuda.synchronize()
        dist.barrier()
    _, red_ms = timed(lambda: D.allreduce_normal_equations(ZTZ, ZTy))            # pack, all-reduce, unpack + mirror
    symmetric = bool(torch.equal(ZTZ[:2048, :2048], ZTZ[:2048, :2048].T))
    t0 = time.perf_counter()
    alpha = D.solve_on_rank0_and_broadcast(model.solve_normal_equations, ZTZ, ZTy, F, dev)
    torch.cuda.synchronize()
    solve_ms = (time.perf_counter() - t0) * 1e3
    finite = bool(torch.isfinite(alpha).all())
    del ZTZ
    rows_ms, own_ms, lib_ms, red_ms, solve_ms = dist.max([rows_ms, own_ms, lib_ms, red_ms, solve_ms])
    nrows = 64 * nconf
    alg_flops = 2.0 * nrows * F * F                      # the full product upstream forms; the triangle is half of it
    packed_bytes = F * (F + 1) // 2 * 8 + F * 8
    return {'workload': 'c4', 'features': F, 'conformers_per_gpu': nconf, 'rows_per_conformer': 64, 'n_gpus': world,
            'training_rows_ms': rows_ms, 'accumulate_ms': own_ms, 'accumulate_cublas_ms': lib_ms,
            'in_tree_over_cublas_rate': lib_ms / own_ms, 'in_tree_vs_cublas_max_rel_diff': agree,
            'fp64_algorithmic_tflops_per_gpu': alg_flops / (own_ms * 1e-3) / 1e12,
            'fp64_executed_tflops_per_gpu': 0.5 * alg_flops / (own_ms * 1e-3) / 1e12,
            'conformers_per_s': nconf * world / ((rows_ms + own_ms) * 1e-3),
            'allreduce_ms': red_ms, 'allreduce_bytes': packed_bytes if world > 1 else 0,
            'allreduce_gbs': (packed_bytes / (red_ms * 1e-3) / 1e9) if world > 1 else None,
            'allreduce_note': 'pack of the upper triangle + NCCL all-reduce of F(F+1)/2 float64 + unpack and mirror'
                              if world > 1 else 'single rank: pack, unpack and mirror only',
            'symmetric_after_exchange': symmetric, 'solve_ms': solve_ms, 'solve_finite': finite,
            'solver': 'Cholesky (potrf + potrs, fp64) on rank 0, weights broadcast; llambda 1e-5'}


def reference_cuda_comparison():
    """Upstream's own CUDA operators ("reference + 72-byte allocation fix", built by baseline/build_ref.py into the
    git-ignored baseline/_ref/) against this library on identical inputs, each workload in a child process
    (baseline/compare_ref_cuda.py).  Reported when the two operator libraries are present; a failure of the child is
    recorded, never fatal."""
    libs = [os.path.join(ROOT, 'baseline', '_ref', n) for n in ('libref_torchscript_fchl19.so', 'libref_torchscript_sorf.so')]
    if not all(os.path.exists(p) for p in libs):
        return {'unavailable': 'baseline/_ref operator libraries not built (python baseline/build_ref.py needs an upstream checkout)'}
    out = {'label': 'reference + 72-byte allocation fix (upstream sources otherwise unchanged, -O2, sm_100a)'}
    for name, nmol, batch in (('c0', 1000, 1000), ('c1', 2000, 1000)):
        try:
            r = subprocess.run([sys.executable, os.path.join(ROOT, 'baseline', 'compare_ref_cuda.py'), '--workload', name, '--nmol', str(nmol),
                                '--batch', str(batch)], capture_output=True, text=True, timeout=600)
            lines = [ln for ln in r.stdout.splitlines() if ln.startswith('{')]
            out[name] = json.loads(lines[-1]) if lines else {'unavailable': (r.stderr or r.stdout)[-300:]}
        except Exception as exc:  # noqa: BLE001  (a comparison that cannot run must not take the benchmark down)
            out[name] = {'unavailable': repr(exc)[:300]}
    return out


def extra_entry(r, world, sm_mhz, scaling):
    out = {'value': r['value'], 'unit': 'molecules/s', 'ms_per_step': r['ms'], 'scaling': scaling,
           'e2e': None if r['e2e_value'] is None else {'value': r['e2e_value'], 'unit': 'molecules/s',
                                                       'h2d_bytes_per_step': r['h2d'], 'd2h_bytes_per_step': r['d2h']},
           'molecules_this_rank': r['nconf'], 'atoms_this_rank': r['natoms'], 'atoms_max_over_ranks': r['natoms_max'],
           'fast_math': bool(r['model'].fast_math)}
    out['roofline'] = rff_roofline(r) if r['kind'] == 'rff' else sorf_roofline(r, world, sm_mhz)
    return out


def main():
    args = parse_args()
    rank = int(os.environ.get('RANK', 0))
    world = int(os.environ.get('WORLD_SIZE', 1))
    local = int(os.environ.get('LOCAL_RANK', 0))
    if args.impl == 'reference':
        run_reference(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit('bench.py needs a CUDA device: the prediction path has no CPU fallback')
    dev = torch.device('cuda', local)
    torch.cuda.set_device(dev)
    dist = Dist(world, dev)
    from qml_lightning_b200.utils.sharding import my_shard

    name = args.workload
    species, npcas, nstacks, default_n, _ = WORKLOADS[name]
    nreq = args.conformers or default_n
    if name == 'c4':
        out = run_c4(dev, dist, rank, world, nreq, args.nstacks, args.rows_only)
        if rank == 0:
            print(json.dumps({'metric': 'normal-equation accumulation', 'value': out['conformers_per_s'], 'unit': 'conformers/s',
                              'n_gpus': world, 'steps': 1, 'warmup': 1, 'ms_per_step': out['training_rows_ms'] + out['accumulate_ms'],
                              'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None, 'dtype': 'f64', 'data': 'synthetic',
                              'config': {'workload': 'c4'}, 'extra': {'c4': out}}))
        dist.close()
        return

    def shard(wname, n, seed_base):
        if wname == 'c2':      # one global batch, contiguous atom-balanced shards (strong scaling)
            X, Z, counts = workload(n, 1002, 'c2')
            lo, hi = my_shard(counts, rank, world)
            return X[lo:hi], Z[lo:hi], counts[lo:hi], n
        X, Z, counts = workload(n, seed_base + rank, 'c0' if wname == 'c0' else 'c1')   # every rank owns its own molecules
        return X, Z, counts, n * world

    X, Z, counts, nglobal = shard(name, nreq, 1001)
    sampler = ClockSampler(local) if rank == 0 else None
    r = time_prediction(name, dev, dist, rank, args.steps, args.warmup, X, Z, counts, nglobal, sampler=sampler)
    clocks = r['clocks']
    sm_mhz = clocks['sm_mhz'] if clocks else None
    small = r['nconf'] <= 1024
    line = {
        'metric': 'energy+force predictions', 'value': r['value'], 'unit': 'molecules/s', 'n_gpus': world, 'steps': args.steps,
        'warmup': args.warmup, 'ms_per_step': r['ms'], 'higher_is_better': True,
        'scaling': 'strong' if name == 'c2' else 'weak', 'vs_baseline': None, 'dtype': 'f32', 'data': 'synthetic',
        'config': {'workload': name, 'molecules_per_gpu': r['nconf'],
                   'atoms_per_molecule': r['A'] if name != 'c2' else 'ragged 4-29 (padded to 29)',
                   'species': species, 'npcas': npcas, 'nstacks': nstacks, 'features': npcas * nstacks,
                   'parallelism': f'molecule shards x{world}, no collective',
                   'l2': 'flushed between steps (512 MB write outside the timed events); per-step workspace > L2',
                   'fast_math': bool(r['model'].fast_math)},
        'e2e': {'value': r['e2e_value'], 'unit': 'molecules/s', 'h2d_bytes_per_step': r['h2d'], 'd2h_bytes_per_step': r['d2h']},
        'gpu_launches': (KERNELS_PER_STEP_SMALL if small else KERNELS_PER_STEP) * args.steps,
        'clocks': clocks,
        'roofline': rff_roofline(r) if r['kind'] == 'rff' else sorf_roofline(r, world, sm_mhz),
    }
    model_c1 = r.pop('model')
    r.pop('rep')
    if rank == 0 and world == 1 and not args.no_cpu_baseline and name == 'c1':
        rate, dt = cpu_oracle_rate(species, npcas, nstacks, X, Z, counts, model_c1.reductors.cpu(), model_c1.Dmat.cpu(),
                                   model_c1.bias.cpu(), model_c1.alpha.cpu(), args.cpu_sample)
        line['cpu_baseline'] = {'value': rate, 'unit': 'molecules/s', 'cores': os.cpu_count(), 'kind': 'port',
                                'sample': f'{args.cpu_sample} conformers of the c1 workload, torch CPU fp32 oracle, {dt:.1f} s'}
    del model_c1
    torch.cuda.empty_cache()

    if name == 'c1' and not args.no_extras:
        extra = {}
        xs = max(3, min(args.steps, 5))
        X2, Z2, c2, n2 = shard('c2', WORKLOADS['c2'][3], 0)
        e = time_prediction('c2', dev, dist, rank, xs, 3, X2, Z2, c2, n2)
        extra['c2'] = extra_entry(e, world, sm_mhz, 'strong')
        extra['c2']['molecules_total'] = n2
        del e, X2, Z2, c2
        torch.cuda.empty_cache()
        if world == 1:
            X0, Z0, c0, n0 = shard('c0', WORKLOADS['c0'][3], 1000)
            e = time_prediction('c0', dev, dist, rank, max(xs, 20), 5, X0, Z0, c0, n0)
            extra['c0'] = extra_entry(e, world, sm_mhz, 'weak')
            del e
            X3, Z3, c3, n3 = shard('c3', WORKLOADS['c3'][3], 1001)
            e = time_prediction('c3', dev, dist, rank, xs, 3, X3, Z3, c3, n3)
            extra['c3'] = extra_entry(e, world, sm_mhz, 'weak')
            del e, X3, Z3, c3
            torch.cuda.empty_cache()
            e = time_prediction('c1', dev, dist, rank, xs, 3, X, Z, counts, nglobal, fast_math=False)
            extra['c1_accurate'] = extra_entry(e, world, sm_mhz, 'weak')
            del e
            torch.cuda.empty_cache()
        extra['c4'] = run_c4(dev, dist, rank, world, WORKLOADS['c4'][3])
        if world == 1:
            torch.cuda.empty_cache()
            extra['reference_cuda'] = reference_cuda_comparison()
        line['extra'] = extra
    if rank == 0:
        print(json.dumps(line))
    dist.close()


if __name__ == '__main__':
    main()
