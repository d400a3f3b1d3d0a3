"""``BaseKernel``: host-side orchestration shared by the SORF and RFF models.

Mirrors the public surface of upstream qml_lightning/models/kernel.py (constructor attributes, ``format_data``,
``get_reductors``, ``build_Z_components``, ``train``, self-energy helpers).  ``format_data`` is vectorised (upstream
concatenates per molecule, which is quadratic in the batch size); the normal equations can be sharded over ranks
and combined with one all-reduce.
"""
import numpy as np
import torch

from ..utils.staging import PinnedStage


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
        dev = torch.device(self.rep.device)
        zbatch = len(X)
        counts_np = np.fromiter((x.shape[0] for x in X), dtype=np.int32, count=zbatch)
        max_atoms = int(counts_np.max()) if zbatch else 0
        total = int(counts_np.sum())
        specs = [((zbatch, max_atoms, 3), np.float32), ((zbatch, max_atoms), np.float32), ((zbatch,), np.int32),
                 ((total,), np.int32), ((total,), np.int32)]
        staged = dev.type == 'cuda' and zbatch > 0
        if staged:       # page-locked staging, copies enqueued without blocking the host (utils/staging.py)
            if getattr(self, '_stage', None) is None:
                self._stage = PinnedStage()
            (coords, charges, counts, atom_ids, mol_ids), pinned = self._stage.arrays(specs)
        else:
            coords, charges, counts, atom_ids, mol_ids = (np.zeros(shape, dtype=dt) for shape, dt in specs)
        counts[:] = counts_np
        mol_ids[:] = np.repeat(np.arange(zbatch, dtype=np.int32), counts_np)
        starts = (np.cumsum(counts_np) - counts_np).astype(np.int64)
        atom_ids[:] = np.arange(total, dtype=np.int64) - np.repeat(starts, counts_np)
        if total:
            coords[mol_ids, atom_ids] = np.concatenate([np.asarray(x, dtype=np.float32).reshape(-1, 3) for x in X])
            charges[mol_ids, atom_ids] = np.concatenate([np.asarray(q, dtype=np.float32).reshape(-1) for q in Q])
        if staged:
            d_coords, d_charges, d_counts, d_atom, d_mol = self._stage.upload(pinned, dev)
        else:
            d_coords, d_charges, d_counts, d_atom, d_mol = (torch.from_numpy(a).to(dev)
                                                           for a in (coords, charges, counts, atom_ids, mol_ids))
        data = {
            'coordinates': d_coords,
            'charges': d_charges,
            'natom_counts': d_counts,
            'atomIDs': d_atom,
            'molIDs': d_mol,
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
    def sample_representations(self, X, Q, element, pick, cells=None, inv_cells=None, npca_choice=256, nsamples=4096):
        """Rows ``f32[n, repsize]`` of the SVD sample matrix of ``element`` for the molecules ``pick`` (see
        ``get_reductors`` for the rule); everything up to the final row gather runs on the device without a host wait."""
        from .. import cabi
        dev = self.rep.device
        data = self.format_data([X[i] for i in pick], [Q[i] for i in pick],
                                cells=None if cells is None else [cells[i] for i in pick],
                                inv_cells=None if inv_cells is None else [inv_cells[i] for i in pick])
        Zc, counts = data['charges'], data['natom_counts']
        A = Zc.shape[1]
        one = torch.tensor([float(element)], dtype=torch.float32, device=dev)
        g = cabi.group_by_element(Zc, counts, one, data['atomIDs'].shape[0])          # rows = the atoms of this element
        rows = torch.zeros(g.rows_cap, self.rep.get_repsize(), dtype=torch.float32, device=dev)
        cabi.fchl19_forward(data['coordinates'], Zc, counts, self.rep.kernel_params(dev), data['cells'], data['inv_cells'],
                            row_of_slot=g.row_of_slot, out=rows)
        slot = g.slot_of_row.long()
        real = slot >= 0
        nbatches = (len(pick) + self.nbatch_train - 1) // self.nbatch_train
        batch = torch.where(real, torch.div(slot, A, rounding_mode='floor') // self.nbatch_train,
                            torch.full_like(slot, nbatches))                           # padding rows sort last
        # random order inside every batch: sort by (batch, random key); rank = position within the batch
        key = batch.double() + torch.rand(slot.shape[0], device=dev, dtype=torch.float64) * 0.5
        order = torch.argsort(key)
        sorted_batch = batch[order]
        per_batch = torch.bincount(sorted_batch, minlength=nbatches + 1)[:nbatches]
        first = torch.cumsum(per_batch, 0) - per_batch
        rank = torch.arange(slot.shape[0], device=dev) - first[sorted_batch.clamp(max=nbatches - 1)]
        taken = torch.clamp(per_batch, max=npca_choice)
        before = torch.cumsum(taken, 0) - taken                                        # atoms collected before each batch
        batch_ok = before <= nsamples                                                  # upstream stops once nselected > nsamples
        keep = (sorted_batch < nbatches) & (rank < npca_choice) & batch_ok[sorted_batch.clamp(max=nbatches - 1)]
        return rows[order[keep]]                                                       # the one host wait: its row count

    def get_reductors(self, X, Q, cells=None, inv_cells=None, npcas=128, npca_choice=256, nsamples=4096, print_info=True):
        """Per element: SVD of sampled atom representations, first ``npcas`` left singular vectors.

        Sampling rule of upstream kernel.py:447-540: up to 1024 molecules containing the element (drawn with
        replacement by numpy, like upstream), cut into batches of ``nbatch_train`` molecules; from every batch at most
        ``npca_choice`` randomly chosen atoms of the element; batches are taken until more than ``nsamples`` atoms have
        been collected.  Upstream formats every batch, evaluates the representation per batch and gathers the rows with
        boolean masks (one host synchronisation per batch); here the picked molecules are formatted once, the
        representation is written straight into element-grouped rows by one kernel launch, and the per-batch selection
        is index arithmetic on the device, so the host waits once per element (for the size of the sample matrix)."""
        for e in self.elements:
            ei = int(self.element2index[int(e)])
            have = np.array([i for i in range(len(Q)) if int(e) in np.asarray(Q[i])], dtype=np.int64)
            if have.size == 0:
                continue
            pick = np.random.choice(have, size=min(len(have), 1024))
            mat = self.sample_representations(X, Q, int(e), pick, cells, inv_cells, npca_choice, nsamples)
            if mat.shape[0] == 0:
                continue
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

    def pca_packed(self):
        """Split and tiled images of ``self.reductors`` for the tensor-core projection, rebuilt only when the tensor
        was replaced or written to since the last call (``get_reductors``, direct assignment, in-place edits)."""
        from .. import cabi
        red = self.reductors
        key = (red.data_ptr(), red._version, tuple(red.shape), red.device)
        if getattr(self, '_pca_packed_key', None) != key:
            self._pca_packed = cabi.pca_pair_pack(self.kernel_reductors().contiguous().float())
            self._pca_packed_key = key
        return self._pca_packed

    def kernel_reductors(self):
        """The projection matrices as the kernels read them; models whose kernels need another width override this."""
        return self.reductors

    # ---- training --------------------------------------------------------------------------------------------
    def training_rows(self, data, with_forces):
        """``(Z f64[zbatch,F], G f64[zbatch,A,3,F] | None)`` for one formatted batch; implemented by the models."""
        raise NotImplementedError("Abstract method only.")

    def _element_features(self, x, dx, element_idx, grouping, counts, nb, A):
        """``(Z, G)`` of the rows of one element through the model's training kernels; implemented by the models."""
        raise NotImplementedError("Abstract method only.")

    def calculate_features(self, rep, element, indexes, feature_matrix, grad=None, derivative_matrix=None):
        """Upstream's per-element training step (hadamard_features.py:66-80, random_features.py:60-67), kept for callers
        that drive the element loop themselves: ``rep f32[n_e, npcas]`` are the projected rows of the atoms of
        ``element``, ``indexes[n_e]`` their molecule numbers; adds the per-molecule features into
        ``feature_matrix f64[nmol, F]`` and, given ``grad f32[n_e, A, 3, npcas]``, the force features (-dZ/dr) into
        ``derivative_matrix f64[nmol, A, 3, F]``.  ``training_rows`` does the same for all elements of a batch at once."""
        from .. import cabi
        dev = rep.device
        n, nb = rep.shape[0], feature_matrix.shape[0]
        if n == 0:
            return
        with_grad = grad is not None and derivative_matrix is not None
        g, A = cabi.grouping_from_ordering(indexes.to(dev), nb, int(grad.shape[1]) if with_grad else None)
        x = cabi.pad_rows(rep.float(), g.rows_cap)
        dx = cabi.pad_rows(grad.float(), g.rows_cap) if with_grad else None
        counts = torch.full((nb,), A, dtype=torch.int32, device=dev)
        Z, G = self._element_features(x, dx, int(self.element2index[int(element)]), g, counts, nb, A)
        feature_matrix += Z
        if with_grad:
            derivative_matrix += G

    @staticmethod
    def allreduce_normal_equations(ZTZ, ZtrainY):
        """Sum the per-rank partial normal equations in place (packed upper triangle, one all-reduce) and mirror the
        triangle; without an initialised process group only the mirroring happens."""
        from ..utils.distributed import allreduce_normal_equations
        return allreduce_normal_equations(ZTZ, ZtrainY)

    def build_Z_components(self, X, Q, E=None, F=None, cells=None, inv_cells=None, print_info=True, cpu_solve=False, ntiles=1,
                           use_specialized_matmul=False, distributed=False):
        """Accumulate ``Z^T Z`` (float64) and ``Z^T y`` over host batches of ``nbatch_train`` molecules.

        Rows per molecule: one energy row and, with forces, ``3 * max_atoms`` force rows (``G = -dZ/dr``), targets
        ``cat(E, F.flatten())`` -- the construction of upstream build_Z_components (kernel.py:46-217).  Only the upper
        triangle is accumulated and mirrored once at the end.  With ``distributed=True`` every rank of the
        initialised process group takes a contiguous, atom-balanced share of the molecules and the partial sums are
        combined with one all-reduce of the packed triangle.  ``use_specialized_matmul`` rounds the rows to float32 before the product, as
        upstream's matmul_and_reduce path does (the products are still accumulated in float64).  ``ntiles`` is accepted
        for signature compatibility: the full matrix is kept on the device.
        """
        from .. import cabi
        from ..utils.sharding import my_shard
        if E is None and F is None:
            raise RuntimeError("must have either E, F or both as input to train().")
        lo, hi = 0, len(X)
        if distributed:
            import torch.distributed as dist
            lo, hi = my_shard([np.asarray(q).shape[0] for q in Q], dist.get_rank(), dist.get_world_size())
        dev = self.rep.device
        nf = self.nfeatures()
        ZTZ = torch.zeros(nf, nf, device=dev, dtype=torch.float64)
        ZtrainY = torch.zeros(nf, 1, device=dev, dtype=torch.float64)
        for i in range(lo, hi, self.nbatch_train):
            sl = slice(i, min(i + self.nbatch_train, hi))
            data = self.format_data(X[sl], Q[sl], E=None if E is None else E[sl], F=None if F is None else F[sl],
                                    cells=None if cells is None else cells[sl],
                                    inv_cells=None if inv_cells is None else inv_cells[sl])
            zbatch = data['coordinates'].shape[0]
            Ztrain, Gtrain = self.training_rows(data, with_forces=F is not None)
            if E is None:
                Ztrain.zero_()       # energy rows must not contribute when only forces are fitted (kernel.py:164-165)
                targets = torch.cat((torch.zeros(zbatch, dtype=torch.float64, device=dev), data['forces'].flatten()))
            elif F is None:
                targets = data['energies']
            else:
                targets = torch.cat((data['energies'], data['forces'].flatten()))
            rows = Ztrain if Gtrain is None else torch.cat((Ztrain, Gtrain.reshape(-1, nf)), dim=0)
            if use_specialized_matmul:
                # upstream hands float32 copies of the rows to matmul_and_reduce (kernel.py:176-188); Z^T y keeps the
                # float64 rows (kernel.py:192)
                cabi.normal_equations_accumulate(rows.float().double(), None, ZTZ, None)
                cabi.gemv_t(rows, targets.contiguous(), ZtrainY)
            else:
                cabi.normal_equations_accumulate(rows, targets.contiguous(), ZTZ, ZtrainY)
        if distributed:
            self.allreduce_normal_equations(ZTZ, ZtrainY)       # packed triangle over the ranks, mirrored afterwards
        else:
            cabi.symmetrize_upper(ZTZ)
        if cpu_solve:
            ZTZ = ZTZ.cpu()
        return ZTZ, ZtrainY

    def train(self, X, Q, E=None, F=None, cells=None, inv_cells=None, print_info=True, cpu_solve=False, ntiles=1,
              use_specialized_matmul=False, distributed=False):
        """Solve ``(Z^T Z + llambda I) alpha = Z^T y`` (upstream kernel.py:219-247).  The system is symmetric positive
        definite, so a Cholesky factorisation replaces upstream's LU; LU is the fallback if the factorisation fails."""
        ZTZ, ZtrainY = self.build_Z_components(X, Q, E, F, cells, inv_cells, print_info, cpu_solve, ntiles,
                                               use_specialized_matmul, distributed)
        if distributed:
            # one factorisation on rank 0, the weights (8 bytes per feature) broadcast to the others
            from ..utils.distributed import solve_on_rank0_and_broadcast
            alpha = solve_on_rank0_and_broadcast(self.solve_normal_equations, ZTZ, ZtrainY, self.nfeatures(), self.rep.device)
        else:
            alpha = self.solve_normal_equations(ZTZ, ZtrainY)
        self.alpha = alpha.to(self.rep.device)
        self.is_trained = True
        self._parameters_changed()
        del ZTZ, ZtrainY

    def solve_normal_equations(self, ZTZ, ZtrainY):
        """alpha of ``(Z^T Z + llambda I) alpha = Z^T y``; adds llambda to the diagonal of ``ZTZ`` in place."""
        ZTZ.diagonal().add_(self.llambda)
        rhs = ZtrainY.to(ZTZ.device)
        L, info = torch.linalg.cholesky_ex(ZTZ)
        if int(info) == 0:
            return torch.cholesky_solve(rhs, L)[:, 0]
        return torch.linalg.solve(ZTZ, rhs)[:, 0]
