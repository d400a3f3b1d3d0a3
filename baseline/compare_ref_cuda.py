"""Upstream's CUDA operators ("reference + 72-byte allocation fix", see baseline/build_ref.py) against this repository on
identical seeded inputs and model tensors: energy+force rate of both, their ratio, and the three distances that
settle parity (new vs reference, reference vs float64 oracle, new vs float64 oracle) plus the reference's run-to-run
spread (its float atomics make it non-deterministic).

    python baseline/compare_ref_cuda.py --workload c1 --nmol 2000 --batch 1000

The reference runs in a child process (``baseline/ref_cuda_bench.py``): both libraries register the same operator names.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--workload', default='c1', choices=['c0', 'c1'])
    ap.add_argument('--nmol', type=int, default=2000)
    ap.add_argument('--batch', type=int, default=1000)
    ap.add_argument('--steps', type=int, default=3)
    ap.add_argument('--oracle-molecules', type=int, default=8)
    args = ap.parse_args()
    import ref_cuda_bench as R
    with tempfile.TemporaryDirectory() as tmp:
        out = os.path.join(tmp, 'ref.npz')
        r = subprocess.run([sys.executable, os.path.join(HERE, 'ref_cuda_bench.py'), '--workload', args.workload, '--nmol', str(args.nmol),
                            '--batch', str(args.batch), '--steps', str(args.steps), '--save', out], capture_output=True, text=True,
                           timeout=900)
        lines = [ln for ln in r.stdout.splitlines() if ln.startswith('{')]
        if r.returncode != 0 or not lines:
            print(json.dumps({'reference_cuda': {'unavailable': (r.stderr or r.stdout)[-400:]}}))
            return
        ref = json.loads(lines[-1])
        if 'unavailable' in ref:
            print(json.dumps({'reference_cuda': ref}))
            return
        saved = np.load(out)
        E_ref, F_ref = torch.from_numpy(saved['E']).double(), torch.from_numpy(saved['F']).double()

    from oracle import FCHLParams, energy_and_forces
    from qml_lightning_b200 import cabi
    from qml_lightning_b200.utils import synthetic as syn
    dev = torch.device('cuda', 0)
    species, npcas, nstacks = R.CONFIGS[args.workload]
    charges = syn.C0_CHARGES if args.workload == 'c0' else syn.C1_CHARGES
    X, Z, counts = syn.conformers(1001, charges, args.nmol)
    red, Dmat, bias, alpha = R.model_tensors(syn, species, npcas, nstacks, dev)
    p = FCHLParams(species=species, **R.FCHL)
    kp = cabi.FchlKernelParams(torch.tensor(species, dtype=torch.float32, device=dev), p.Rs2.to(dev), p.Rs3.to(dev), p.eta2, p.eta3,
                               p.two_body_decay, p.w3, p.three_body_decay, p.rcut)
    packed = cabi.sorf_pack(Dmat, bias, alpha)
    pca_packed = cabi.pca_pair_pack(red)
    Xd, Zd, cd = (torch.from_numpy(a).to(dev) for a in (X, Z, counts))
    el = torch.tensor(species, dtype=torch.float32, device=dev)
    out = {}
    for fast in (True, False):
        def run():
            return cabi.sorf_predict(Xd, Zd, cd, kp, el, red, packed, nstacks, 1, 2.0, fast_math=fast, pca_packed=pca_packed)
        for _ in range(2):
            run()
        torch.cuda.synchronize()
        times = []
        for _ in range(max(args.steps, 5)):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            E, gX = run()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        ms = float(np.mean(times))
        E, Fo = E.cpu().double(), -gX.cpu().double()
        key = 'fast_math' if fast else 'accurate'
        rms = float(torch.sqrt(torch.mean(E_ref ** 2)))
        out[key] = {'value': args.nmol / (ms * 1e-3), 'ms': ms, 'ratio_to_reference': (args.nmol / (ms * 1e-3)) / ref['value'],
                    'new_vs_reference': {'max_rel_dE': float(((E - E_ref).abs() / torch.clamp(E_ref.abs(), min=rms)).max()),
                                         'max_abs_dF': float((Fo - F_ref).abs().max())}}
        if fast:
            E_new, F_new = E, Fo
    model = dict(kind='sorf', elements=species, reductors=red.cpu(), Dmat=Dmat.cpu(), bias=bias.cpu(), alpha=alpha.cpu(), sigma=2.0,
                 ntransforms=1)

    def against_oracle(idx):
        E_o, F_o = energy_and_forces(torch.from_numpy(X[idx]), torch.from_numpy(Z[idx]), torch.from_numpy(counts[idx]), p, model, batch=4)
        rms = float(torch.sqrt(torch.mean(E_o ** 2)))
        rel = lambda a: float(((a[idx] - E_o).abs() / torch.clamp(E_o.abs(), min=rms)).max())
        return {'molecules': len(idx),
                'reference_vs_oracle': {'max_rel_dE': rel(E_ref), 'max_abs_dF': float((F_ref[idx] - F_o).abs().max())},
                'new_vs_oracle': {'max_rel_dE': rel(E_new), 'max_abs_dF': float((F_new[idx] - F_o).abs().max())}}

    n = min(args.oracle_molecules, args.nmol)
    out['oracle_first_molecules'] = against_oracle(list(range(n)))
    # where the two implementations disagree most, the float64 oracle says which one is off
    per_mol = (F_new - F_ref).abs().amax(dim=(1, 2))
    worst = torch.argsort(per_mol, descending=True)[:min(2 * n, args.nmol)].tolist()
    out['oracle_worst_disagreements'] = against_oracle(worst)
    out['oracle_worst_disagreements']['median_per_molecule_max_abs_dF_new_vs_reference'] = float(per_mol.median())
    out['reference_cuda'] = ref
    out['same_inputs'] = f'{args.nmol} seeded conformers of {args.workload}, identical model tensors; reference in host batches of {args.batch}'
    print(json.dumps(out))


if __name__ == '__main__':
    main()
