"""``HadamardFeaturesModel``: SORF kernel model with the upstream constructor, attributes and methods
(upstream qml_lightning/models/hadamard_features.py).

``forward`` keeps the TorchScript signature ``forward(X, Z, atomIDs, molIDs, atom_counts, cell, inv_cell)`` and returns
energies without self energies; it calls one fused operator (FCHL19 -> PCA -> SORF -> energy, with the coordinate
gradient produced in the same pass and handed to autograd), so ``torch.autograd.grad(-E.sum(), X)`` works as before.
``forward_unfused`` evaluates the same model through the fine-grained operators that saved upstream archives call.
"""
import numpy as np
import torch

from .. import cabi
from .kernel import BaseKernel


class HadamardFeaturesModel(BaseKernel, torch.nn.Module):

    def __init__(self, rep=None, elements=np.array([1, 6, 7, 8]), ntransforms=2, sigma=3.0, llambda=1e-11, npcas=128,
                 nbatch_train=64, nbatch_test=64, nstacks=32, fast_math=True):
        super(HadamardFeaturesModel, self).__init__(rep, npcas, elements, sigma, llambda)
        dev = rep.device
        self.device = dev
        self.ntransforms = torch.tensor(ntransforms)
        self.ntransforms_int = int(ntransforms)
        self.nstacks = nstacks
        self.nbatch_train = nbatch_train
        self.nbatch_test = nbatch_test
        self.species = torch.from_numpy(np.asarray(elements)).float().to(dev)
        self.npcas = npcas
        self.fast_math = bool(fast_math)
        self.Dmat = torch.zeros((len(elements), ntransforms, nstacks, npcas), dtype=torch.float32, device=dev)
        self.get_SORF_diagonals(elements, ntransforms, nstacks, npcas)
        self.bias = torch.zeros((len(elements), self.nfeatures()), dtype=torch.float32, device=dev)
        self.get_bias(elements, nstacks * npcas)
        self.is_trained = False
        self.alpha = torch.zeros(self.nfeatures(), device=dev, dtype=torch.float)
        self.packed = torch.zeros(1, dtype=torch.float32, device=dev)
        self._parameters_changed()

    # ---- random bases (numpy RNG, like upstream :45-63) -----------------------------------------------------------
    def get_SORF_diagonals(self, elements, ntransforms, nstacks, npcas):
        for e in elements:
            D = np.where(np.random.uniform(-1, 1, (ntransforms, nstacks, npcas)) > 0.0, 1.0, -1.0)
            self.Dmat[int(self.element2index[int(e)])] = torch.from_numpy(D).float().to(self.Dmat.device)

    def get_bias(self, elements, nfeatures):
        for e in elements:
            v = np.random.uniform(0.0, 1.0, [nfeatures]) * 2.0 * np.pi
            self.bias[int(self.element2index[int(e)])] = torch.from_numpy(v).float().to(self.bias.device)

    def nfeatures(self):
        return self.npcas * self.nstacks

    def _parameters_changed(self):
        """Re-pack Dmat / bias / alpha for the fused kernel; call after changing any of them."""
        if self.Dmat.is_cuda:
            self.packed = torch.ops.qml_lightning_b200.sorf_pack(self.Dmat, self.bias, self.alpha.float())

    def set_alpha(self, alpha):
        self.alpha = alpha.to(self.device)
        self.is_trained = True
        self._parameters_changed()

    # ---- training ------------------------------------------------------------------------------------------------
    def training_rows(self, data, with_forces):
        """Per-molecule features and force features of one formatted batch (upstream calculate_features :66-80 applied
        to all elements at once): representation (+ explicit Jacobian) -> PCA -> SORF training kernels."""
        X, Zc, counts = data['coordinates'], data['charges'], data['natom_counts']
        nb, A = Zc.shape
        kp = self.rep.kernel_params(X.device)
        g = cabi.group_by_element(Zc, counts, self.species, data['atomIDs'].shape[0])
        if with_forces:
            rep_rows, jac_rows = cabi.fchl19_forward_jacobian(X, Zc, counts, kp, data['cells'], data['inv_cells'], grouping=g)
            dx = cabi.pca_project_jacobian(jac_rows, self.reductors, g)
            del jac_rows
        else:
            rep_rows = torch.zeros(g.rows_cap, self.rep.get_repsize(), dtype=torch.float32, device=X.device)
            cabi.fchl19_forward(X, Zc, counts, kp, data['cells'], data['inv_cells'], row_of_slot=g.row_of_slot, out=rep_rows)
            dx = None
        x = cabi.pca_project(rep_rows, self.reductors, g)
        return cabi.sorf_train_features(x, dx, self.Dmat[:, :self.ntransforms_int].contiguous(), self.bias, g, counts, nb, A,
                                        self.sigma)

    def _element_features(self, x, dx, element_idx, grouping, counts, nb, A):
        e = element_idx
        return cabi.sorf_train_features(x, dx, self.Dmat[e:e + 1, :self.ntransforms_int].contiguous(), self.bias[e:e + 1].contiguous(),
                                        grouping, counts, nb, A, self.sigma)

    # ---- inference -----------------------------------------------------------------------------------------------
    def forward(self, X, Z, atomIDs, molIDs, atom_counts, cell=torch.empty(0, 3, 3), inv_cell=torch.empty(0, 3, 3)):
        assert X.is_cuda, "X tensor must reside on GPU"
        assert Z.device == X.device, "Z tensor must reside on the same GPU as X"
        assert atom_counts.device == X.device, "atom_counts tensor must reside on the same GPU as X"
        return torch.ops.qml_lightning_b200.sorf_energy(X, Z, atom_counts, cell, inv_cell, self.rep.species, self.rep.Rs2,
                                                        self.rep.Rs3, self.rep.kernel_scalars, self.species,
                                                        self.reductors, self.packed, self.nstacks, self.ntransforms_int,
                                                        self.sigma, atomIDs.shape[0], self.fast_math)

    def forward_unfused(self, X, Z, atomIDs, molIDs, atom_counts, cell=torch.empty(0, 3, 3), inv_cell=torch.empty(0, 3, 3)):
        """The upstream operator chain (hadamard_features.py:93-121): one representation operator, then per element a
        projection, ``get_SORF_coefficients`` and ``get_cos_features``.  Kept for saved models and for cross-checks."""
        coeff_normalisation = torch.sqrt(torch.tensor(float(self.npcas))) / self.sigma
        rep = self.rep.forward(X, Z, atomIDs, molIDs, atom_counts, cell, inv_cell)
        Ztest = torch.zeros(X.shape[0], self.nfeatures(), device=X.device, dtype=torch.float32)
        for e in self.elements:
            mask = Z.int() == int(e)
            ei = int(self.element2index[int(e)])
            batch_indexes = torch.where(mask)[0].type(torch.int)
            sub = rep[mask]
            if sub.shape[0] == 0:
                continue
            sub = torch.matmul(sub, self.reductors[ei])
            coeffs = torch.ops.qml_lightning_sorf.get_SORF_coefficients(sub, self.Dmat[ei], coeff_normalisation, self.ntransforms)
            coeffs = coeffs.view(coeffs.shape[0], coeffs.shape[1] * coeffs.shape[2])
            Ztest = Ztest + torch.ops.qml_lightning_sorf.get_cos_features(coeffs, self.bias[ei], torch.tensor(X.shape[0]),
                                                                            batch_indexes)
        return torch.matmul(Ztest, self.alpha.float())

    def predict_opt(self, coordinates, charges, atomIDs, molIDs, natom_counts, cells=None, inv_cells=None, forces=True,
                    print_info=False, profiler=False):
        """Prediction on pre-formatted device tensors; returns ``energies`` or ``(energies, forces)``."""
        if self.is_trained is False:
            raise RuntimeError("must train the model first by calling train()!")
        dev = coordinates.device
        cells = torch.empty(0, 3, 3, device=dev) if cells is None else cells
        inv_cells = torch.empty(0, 3, 3, device=dev) if inv_cells is None else inv_cells
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        if forces:
            # the fused operator already holds dE/dX; calling the C entry point directly skips the autograd graph
            energies, grad = cabi.sorf_predict(coordinates, charges, natom_counts, self.rep.kernel_params(dev), self.species,
                                               self.reductors, self.packed, self.nstacks, self.ntransforms_int, self.sigma,
                                               cells, inv_cells, n_atoms_upper=atomIDs.shape[0], fast_math=self.fast_math,
                                               pca_packed=self.pca_packed())
            result = (energies, -grad)
        else:
            with torch.no_grad():
                result = self.forward(coordinates, charges, atomIDs, molIDs, natom_counts, cells, inv_cells)
        end.record()
        if print_info:
            torch.cuda.synchronize()
            print("prediction for", coordinates.shape[0], "molecules time: ", start.elapsed_time(end), "ms")
        return result

    def predict(self, X, Z, max_natoms, cells=None, inv_cells=None, forces=True, print_info=False, profiler=False):
        """Lists of numpy arrays in, ``energies [n]`` (and ``forces [n, max_natoms, 3]``) out, in host batches of
        ``nbatch_test`` molecules (upstream :181-249)."""
        n = len(X)
        energies = torch.zeros(n, device=self.device, dtype=torch.float32)
        all_forces = torch.zeros(n, max_natoms, 3, device=self.device, dtype=torch.float32)
        for i in range(0, n, self.nbatch_test):
            sl = slice(i, i + self.nbatch_test)
            data = self.format_data(X[sl], Z[sl], cells=None if cells is None else cells[sl],
                                    inv_cells=None if inv_cells is None else inv_cells[sl])
            out = self.predict_opt(data['coordinates'], data['charges'], data['atomIDs'], data['molIDs'], data['natom_counts'],
                                   data['cells'], data['inv_cells'], forces=forces, print_info=print_info)
            if forces:
                energies[sl] = out[0]
                all_forces[sl, :out[1].shape[1]] = out[1]      # padded atoms carry exact zeros
            else:
                energies[sl] = out
        return (energies, all_forces) if forces else energies

    def save_jit_model(self, file_name='model_sorf.pt'):
        script = torch.jit.script(self)
        script.save(file_name)
