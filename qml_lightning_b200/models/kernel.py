"""``BaseKernel``: host-side orchestration shared by the SORF and RFF models.

Mirrors the public surface of upstream qml_lightning/models/kernel.py (constructor attributes, ``format_data``,
``get_reductors``, ``build_Z_components``, ``train``, self-energy helpers).  ``format_data`` is vectorised (upstream
concatenates per molecule, which is quadratic in the batch size); the normal equations can be sharded over ranks
and combined with one all-reduce.
"""
import numpy as np
import torch


class BaseKernel():

    def __init__(self, rep, npcas, elements, sigma, llambda):
        super(BaseKernel, self).__init__()
        self.npcas = npcas
        self.self_energy = None
        self.elements = torch.tensor(np.asarray(elements))
        self.rep = rep
        dev = rep.device if rep is not None else torch.device('cpu')
        self.reductors = torch.zeros(len(elements), rep.get_repsize(), npcas, dtype=torch.float32, device=dev)
        self.element2index = torch.zeros(int(max(elements)) + 1, dtype=torch.long)
        for i, e in enumerate(self.elements):
            self.element2index[int(e)] = i
        self._convert_from_hartree_to_kcal = False
        self.hartree2kcalmol = 627.5
        self._subtract_self_energies = False
        self.sigma = sigma
        self.llambda = llambda

    # ---- abstract --------------------------------------------------------------------------------------------
    def calculate_features(self, rep, element, indexes, feature_matrix, grad=None, derivative_matrix=None):
        raise NotImplementedError("Abstract method only.")

    def nfeatures(self):
        raise NotImplementedError("Abstract method only.")

    def predict(self, X, Q, max_natoms, cells=None, inv_cells=None, forces=False, print_info=True):
        raise NotImplementedError("Abstract method only.")

    # ---- flags -----------------------------------------------------------------------------------------------
    def set_subtract_self_energies(self, subtract):
        self._subtract_self_energies = subtract

    def subtract_self_energies(self):
        return self._subtract_self_energies

    def set_convert_hartree2kcal(self, convert):
        self._convert_from_hartree_to_kcal = convert

    def convert_hartree2kcal(self):
        return self._convert_from_hartree_to_kcal

    # ---- input formatting ------------------------------------------------------------------------------------
    def format_data(self, X, Q, E=None, F=None, cells=None, inv_cells=None):
        """Lists of per-molecule arrays -> zero-padded device tensors plus ``atomIDs`` / ``molIDs`` / ``natom_counts``.

        Same keys and dtypes as upstream ``format_data`` (kernel.py:601-722); built with one host pass and one copy
        per tensor instead of a ``torch.cat`` per molecule.
        """
        if self.subtract_self_energies() and self.self_energy is None:
            raise RuntimeError("must call model.calculate_self_energy first - this computes atomic contributions to the potential energy.")
        dev = self.rep.device
        zbatch = len(X)
        counts = np.fromiter((x.shape[0] for x in X), dtype=np.int32, count=zbatch)
        max_atoms = int(counts.max()) if zbatch else 0
        total = int(counts.sum())
        mol_ids = np.repeat(np.arange(zbatch, dtype=np.int32), counts)
        starts = (np.cumsum(counts) - counts).astype(np.int64)
        atom_ids = (np.arange(total, dtype=np.int64) - np.repeat(starts, counts)).astype(np.int32)
        coords = np.zeros((zbatch, max_atoms, 3), dtype=np.float32)
        charges = np.zeros((zbatch, max_atoms), dtype=np.float32)
        if total:
            coords[mol_ids, atom_ids] = np.concatenate([np.asarray(x, dtype=np.float32).reshape(-1, 3) for x in X])
            charges[mol_ids, atom_ids] = np.concatenate([np.asarray(q, dtype=np.float32).reshape(-1) for q in Q])
        data = {
            'coordinates': torch.from_numpy(coords).to(dev),
            'charges': torch.from_numpy(charges).to(dev),
            'natom_counts': torch.from_numpy(counts).to(dev),
            'atomIDs': torch.from_numpy(atom_ids).to(dev),
            'molIDs': torch.from_numpy(mol_ids).to(dev),
            'energies': None,
            'forces': None,
            'cells': torch.empty((0, 3, 3), device=dev),
            'inv_cells': torch.empty((0, 3, 3), device=dev),
        }
        if E is not None:
            energies = np.asarray(E, dtype=np.float64).copy()
            if self.convert_hartree2kcal():
                energies *= self.hartree2kcalmol
            if self.subtract_self_energies():
                se = self.self_energy.numpy() if isinstance(self.self_energy, torch.Tensor) else np.asarray(self.self_energy)
                per_atom = se[charges.astype(np.int64)] * (charges > 0)
                energies -= per_atom.sum(axis=1)
            data['energies'] = torch.from_numpy(energies).to(dev)
        if F is not None:
            forces = np.zeros((zbatch, max_atoms, 3), dtype=np.float64)
            if total:
                forces[mol_ids, atom_ids] = np.concatenate([np.asarray(f, dtype=np.float64).reshape(-1, 3) for f in F])
            if self.convert_hartree2kcal():
                forces *= self.hartree2kcalmol
            data['forces'] = torch.from_numpy(forces).to(dev)
        if cells is not None:
            data['cells'] = torch.from_numpy(np.stack([np.asarray(c, dtype=np.float32) for c in cells])).to(dev)
            data['inv_cells'] = torch.from_numpy(np.stack([np.asarray(c, dtype=np.float32) for c in inv_cells])).to(dev)
        return data

    # ---- self energies ---------------------------------------------------------------------------------------
    def calculate_self_energy(self, Q, E):
        """Least-squares per-element contribution to ``E`` (upstream kernel.py:556-599)."""
        nmol = len(Q)
        comp = torch.zeros(nmol, len(self.elements), dtype=torch.float64)
        for i, q in enumerate(Q):
            q = np.asarray(q)
            for k, e in enumerate(self.elements.tolist()):
                comp[i, k] = float((q == e).sum())
        energies = torch.as_tensor(np.asarray(E, dtype=np.float64))
        if self.convert_hartree2kcal():
            energies = energies * self.hartree2kcalmol
        beta = torch.linalg.lstsq(comp.T @ comp, comp.T @ energies[:, None]).solution[:, 0]
        species = self.elements.long()
        self.self_energy = torch.zeros(int(torch.max(species)) + 1, dtype=torch.float64)
        self.self_energy[species] = beta

    # ---- projection matrices ---------------------------------------------------------------------------------
    def get_reductors(self, X, Q, cells=None, inv_cells=None, npcas=128, npca_choice=256, nsamples=4096, print_info=True):
        """Per element: SVD of sampled atom representations, first ``npcas`` left singular vectors
        (sampling rule of upstream kernel.py:447-540: up to 1024 molecules containing the element, at most
        ``npca_choice`` atoms per batch, stop after ``nsamples``)."""
        for e in self.elements:
            ei = int(self.element2index[int(e)])
            have = np.array([i for i in range(len(Q)) if int(e) in np.asarray(Q[i])], dtype=np.int64)
            if have.size == 0:
                continue
            pick = np.random.choice(have, size=min(len(have), 1024))
            inputs, nselected = [], 0
            for s in range(0, len(pick), self.nbatch_train):
                if nselected > nsamples:
                    break
                idx = pick[s:s + self.nbatch_train]
                data = self.format_data([X[i] for i in idx], [Q[i] for i in idx],
                                        cells=None if cells is None else [cells[i] for i in idx],
                                        inv_cells=None if inv_cells is None else [inv_cells[i] for i in idx])
                rep = self.rep.get_representation(data['coordinates'], data['charges'], data['atomIDs'], data['molIDs'],
                                                  data['natom_counts'], data['cells'], data['inv_cells'])
                rows = rep[data['charges'] == float(e)]
                if rows.shape[0] == 0:
                    continue
                rows = rows[torch.randperm(rows.size(0), device=rows.device)[:npca_choice]]
                nselected += rows.shape[0]
                inputs.append(rows)
            if not inputs:
                continue
            mat = torch.cat(inputs)
            u, s, _ = torch.linalg.svd(mat.T, full_matrices=False)
            if print_info:
                cev = 100 - (s.sum() - s[:npcas].sum()) / s.sum() * 100
                print(f"element {int(e)}: {u.shape[0]} -> {npcas}  Cumulative Explained Feature Variance = {float(cev):6.2f} %")
            if u.shape[1] < npcas:
                raise RuntimeError(f"not enough atomic environments in input dataset for element {int(e)}. "
                                   "Either increase npca_choice or provide more structures.")
            self.reductors[ei] = u[:, :npcas]
        self._parameters_changed()

    def _parameters_changed(self):
        """Hook for subclasses that cache derived parameter buffers."""
