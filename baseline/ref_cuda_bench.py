"""Runs the upstream project's own CUDA operators (built by ``baseline/build_ref.py``: "reference + 72-byte allocation
fix") on a synthetic workload and prints one JSON line with the energy+force rate; optionally saves energies and
forces for a parity comparison.

    python baseline/ref_cuda_bench.py --workload c1 --nmol 2000 --batch 1000 --steps 3 [--save out.npz]

The forward pass is upstream's ``HadamardFeaturesModel.forward`` (qml_lightning/models/hadamard_features.py:82-123)
restated operator by operator -- representation, boolean-mask gather per element, projection, SORF coefficients, cosine
features, dot with the weights -- and the forces are ``torch.autograd.grad(-E.sum(), X)`` as in upstream's README.md:58-75
and predict_opt (:125-179).  Molecules are processed in host batches, as upstream does (``nbatch_test``): the coefficient
tensor of a batch has ``atoms x features`` float32 entries and must stay below 2^31 elements per element group.

This script must not import ``qml_lightning_b200``: both register operators under the names ``qml_lightning_fchl::*`` and
``qml_lightning_sorf::*``.  The inputs every element's atoms of which are model species only (an atom of another species
would index the representation with -1 in upstream's kernel).
"""
import argparse
import importlib.util
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
FCHL = dict(rcut=6.0, nRs2=24, nRs3=22, eta2=0.32, eta3=2.7, two_body_decay=1.8, three_body_weight=13.4, three_body_decay=0.57)
CONFIGS = {'c0': ([1, 6, 8], 128, 128), 'c1': ([1, 6, 8], 256, 256)}


def load_synthetic():
    spec = importlib.util.spec_from_file_location('qmlb200_synthetic', os.path.join(ROOT, 'qml_lightning_b200', 'utils', 'synthetic.py'))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def model_tensors(syn, species, npcas, nstacks, dev):
    n = len(species)
    repsize = n * FCHL['nRs2'] + n * (n + 1) * FCHL['nRs3']
    red = torch.from_numpy(syn.random_orthonormal_reductors(3, n, repsize, npcas)).to(dev)
    D, bias, alpha = (torch.from_numpy(a).to(dev) for a in syn.sorf_parameters(4, n, npcas, nstacks, 1))
    return red, D, bias, alpha


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--workload', default='c1', choices=sorted(CONFIGS))
    ap.add_argument('--nmol', type=int, default=2000)
    ap.add_argument('--batch', type=int, default=1000)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--warmup', type=int, default=1)
    ap.add_argument('--seed', type=int, default=1001)
    ap.add_argument('--save', default='')
    args = ap.parse_args()
    for lib in ('libref_torchscript_fchl19.so', 'libref_torchscript_sorf.so'):
        path = os.path.join(HERE, '_ref', lib)
        if not os.path.exists(path):
            print(json.dumps({'impl': 'reference_cuda', 'unavailable': f'{path} not built (python baseline/build_ref.py)'}))
            return
        torch.ops.load_library(path)
    dev = torch.device('cuda', 0)
    syn = load_synthetic()
    species, npcas, nstacks = CONFIGS[args.workload]
    charges = syn.C0_CHARGES if args.workload == 'c0' else syn.C1_CHARGES
    X, Z, counts = syn.conformers(args.seed, charges, args.nmol)
    red, Dmat, bias, alpha = model_tensors(syn, species, npcas, nstacks, dev)
    F = npcas * nstacks
    assert args.batch * max(charges.count(e) for e in set(charges)) * F < 2 ** 31, 'batch too large for 32-bit tensor indexing'
    sp = torch.tensor(species, dtype=torch.float32, device=dev)
    Rs2 = torch.linspace(0.0, FCHL['rcut'], FCHL['nRs2'] + 1)[1:].to(dev)
    Rs3 = torch.linspace(0.0, FCHL['rcut'], FCHL['nRs3'] + 1)[1:].to(dev)
    w3 = torch.tensor(np.sqrt(FCHL['eta3'] / np.pi) * FCHL['three_body_weight'], dtype=torch.float32)   # representations/FCHL.py:35
    t = lambda v: torch.tensor(v)
    cell = torch.empty(0, 3, 3, device=dev)
    norm = torch.sqrt(torch.tensor(float(npcas))) / 2.0          # sigma = 2
    ntr = torch.tensor(1)

    def forward(Xb, Zb, atomIDs, molIDs, cb):
        rep = torch.ops.qml_lightning_fchl.fchl_forwards(Xb, Zb, sp, atomIDs, molIDs, cb, cell, cell, Rs2, Rs3, t(FCHL['eta2']),
                                                         t(FCHL['eta3']), t(FCHL['two_body_decay']), w3, t(FCHL['three_body_decay']),
                                                         t(FCHL['rcut']))
        feats = torch.zeros(Xb.shape[0], F, device=dev, dtype=torch.float32)
        for i, e in enumerate(species):
            mask = Zb.int() == e
            idx = torch.where(mask)[0].type(torch.int)
            sub = rep[mask]
            if sub.shape[0] == 0:
                continue
            sub = torch.matmul(sub, red[i])
            co = torch.ops.qml_lightning_sorf.get_SORF_coefficients(sub, Dmat[i], norm, ntr)
            co = co.view(co.shape[0], co.shape[1] * co.shape[2])
            feats = feats + torch.ops.qml_lightning_sorf.get_cos_features(co, bias[i], torch.tensor(Xb.shape[0]), idx)
        return torch.matmul(feats, alpha)

    batches = []
    for s in range(0, args.nmol, args.batch):
        Xb = torch.from_numpy(X[s:s + args.batch]).to(dev)
        Zb = torch.from_numpy(Z[s:s + args.batch]).to(dev)
        cb = torch.from_numpy(counts[s:s + args.batch]).to(dev)
        nb, A = Zb.shape
        atomIDs = torch.arange(A, dtype=torch.int32, device=dev).repeat(nb)
        molIDs = torch.arange(nb, dtype=torch.int32, device=dev).repeat_interleave(A)
        batches.append((Xb, Zb, atomIDs, molIDs, cb))

    def one_pass():
        Es, Fs = [], []
        for Xb, Zb, atomIDs, molIDs, cb in batches:
            Xg = Xb.clone().requires_grad_(True)
            E = forward(Xg, Zb, atomIDs, molIDs, cb)
            Fo, = torch.autograd.grad(-E.sum(), Xg)
            Es.append(E.detach())
            Fs.append(Fo)
        return torch.cat(Es), torch.cat(Fs)

    torch.backends.cuda.matmul.allow_tf32 = False
    for _ in range(args.warmup):
        one_pass()
    torch.cuda.synchronize()
    times, results = [], []
    for _ in range(args.steps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        results.append(one_pass())
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    ms = float(np.mean(times))
    spread_E = spread_F = 0.0
    if len(results) > 1:       # upstream accumulates with float atomics: runs differ
        spread_E = float(max((r[0] - results[0][0]).abs().max() for r in results[1:]))
        spread_F = float(max((r[1] - results[0][1]).abs().max() for r in results[1:]))
    if args.save:
        np.savez(args.save, E=results[0][0].cpu().numpy(), F=results[0][1].cpu().numpy())
    print(json.dumps({'impl': 'reference_cuda', 'label': 'reference + 72-byte allocation fix', 'workload': args.workload,
                      'molecules': args.nmol, 'host_batch': args.batch, 'steps': args.steps, 'ms_per_pass': ms,
                      'value': args.nmol / (ms * 1e-3), 'unit': 'molecules/s',
                      'run_to_run_max_abs_dE': spread_E, 'run_to_run_max_abs_dF': spread_F}))


if __name__ == '__main__':
    main()
