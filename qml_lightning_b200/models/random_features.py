"""``RandomFourrierFeaturesModel``: dense random Fourier feature model (upstream qml_lightning/models/random_features.py)."""
import numpy as np
import torch

from .. import cabi
from .kernel import BaseKernel


KERNEL_WIDTHS = (32, 64, 128, 256)   # projected widths the feature kernels are built for


class RandomFourrierFeaturesModel(BaseKernel, torch.nn.Module):
    """Any ``npcas`` up to 256 is accepted, as upstream accepts any: the feature kernels exist for 32, 64, 128 and 256
    projected components, and a model of another width runs on the next of these with zero columns appended to the
    projection matrices and zero rows to ``W`` (the argument ``x W + b`` is unchanged term by term).  ``reductors``,
    ``W``, ``b`` and ``alpha`` keep upstream's shapes."""

    def __init__(self, rep=None, elements=np.array([1, 6, 7, 8]), sigma=2.0, llambda=1e-10, nstacks=8192, npcas=128,
                 nbatch_train=64, nbatch_test=64, fast_math=True):
        super(RandomFourrierFeaturesModel, self).__init__(rep, npcas, elements, sigma, llambda)
        self.device = rep.device
        self.npcas = npcas
        widths = [k for k in KERNEL_WIDTHS if k >= npcas]
        if not widths:
            raise ValueError(f"npcas must be at most {KERNEL_WIDTHS[-1]}, got {npcas}")
        self._pad = int(widths[0] - npcas)
        self.nbatch_train = nbatch_train
        self.nbatch_test = nbatch_test
        self._nfeatures = nstacks * self.npcas
        self.species = torch.from_numpy(np.asarray(elements)).float().to(self.device)
        self.sample_elemental_basis()
        self.feature_normalisation = np.sqrt(2.0 / self._nfeatures)
        self.alpha = torch.zeros(self._nfeatures, device=self.device, dtype=torch.float)
        self.is_trained = False
        self.fast_math = bool(fast_math)
        self.packed = torch.zeros(1, dtype=torch.uint8, device=self.device)
        self._parameters_changed()

    def sample_elemental_basis(self):
        """W ~ N(0,1)/(2 sigma^2), b ~ U(0, 2 pi) per element (upstream :42-55)."""
        D, d = self.nfeatures(), self.npcas
        self.W = torch.zeros((len(self.elements), d, D), dtype=torch.float32, device=self.device)
        self.b = torch.zeros((len(self.elements), D), dtype=torch.float32, device=self.device)
        for e in self.elements:
            idx = int(self.element2index[int(e)])
            self.W[idx] = torch.from_numpy(np.random.normal(0.0, 1.0, [d, D]) / (2 * self.sigma ** 2)).float().to(self.device)
            self.b[idx] = torch.from_numpy(np.random.uniform(0.0, 1.0, [D]) * 2.0 * np.pi).float().to(self.device)

    def nfeatures(self):
        return self._nfeatures

    def set_alpha(self, alpha):
        self.alpha = alpha.to(self.device)
        self.is_trained = True
        self._parameters_changed()

    # ---- training ------------------------------------------------------------------------------------------------
    def training_rows(self, data, with_forces):
        """Per-molecule features and force features of one formatted batch (upstream calculate_features :60-67 applied
        to all elements at once)."""
        X, Zc, counts = data['coordinates'], data['charges'], data['natom_counts']
        nb, A = Zc.shape
        kp = self.rep.kernel_params(X.device)
        red = self.kernel_reductors()
        g = cabi.group_by_element(Zc, counts, self.species, data['atomIDs'].shape[0])
        if with_forces:
            rep_rows, jac_rows = cabi.fchl19_forward_jacobian(X, Zc, counts, kp, data['cells'], data['inv_cells'], grouping=g)
            dx = cabi.pca_project_jacobian(jac_rows, red, g)
            del jac_rows
        else:
            rep_rows = torch.zeros(g.rows_cap, self.rep.get_repsize(), dtype=torch.float32, device=X.device)
            cabi.fchl19_forward(X, Zc, counts, kp, data['cells'], data['inv_cells'], row_of_slot=g.row_of_slot, out=rep_rows)
            dx = None
        x = cabi.pca_project(rep_rows, red, g)
        return cabi.rff_train_features(x, dx, self._kernel_W(), self.b, g, counts, nb, A)

    def _element_features(self, x, dx, element_idx, grouping, counts, nb, A):
        e = element_idx
        if self._pad > 0:      # rows arrive at the model's own width
            x = torch.nn.functional.pad(x, [0, self._pad])
            dx = None if dx is None else torch.nn.functional.pad(dx, [0, self._pad])
        return cabi.rff_train_features(x, dx, self._kernel_W()[e:e + 1].contiguous(), self.b[e:e + 1].contiguous(), grouping,
                                       counts, nb, A)

    def kernel_reductors(self):
        """Projection matrices at the width of the kernels (zero columns appended), cached like :meth:`pca_packed`."""
        red = self.reductors
        if self._pad == 0:
            return red
        key = (red.data_ptr(), red._version, tuple(red.shape), red.device)
        if getattr(self, '_red_k_key', None) != key:
            self._red_k = torch.nn.functional.pad(red.float(), [0, self._pad]).contiguous()
            self._red_k_key = key
        return self._red_k

    def _kernel_W(self):
        if self._pad == 0:
            return self.W
        key = (self.W.data_ptr(), self.W._version, tuple(self.W.shape), self.W.device)
        if getattr(self, '_W_k_key', None) != key:
            self._W_k = torch.nn.functional.pad(self.W, [0, 0, 0, self._pad]).contiguous()
            self._W_k_key = key
        return self._W_k

    def _parameters_changed(self):
        """Rebuild the packed image of (W, b, alpha) that the tensor-core feature kernel reads; call after changing any
        of them by hand."""
        self.packed = torch.ops.qml_lightning_b200.rff_pack(self._kernel_W(), self.b, self.alpha.float())

    # ---- inference -----------------------------------------------------------------------------------------------
    def forward(self, X, Z, atomIDs, molIDs, atom_counts, cell=torch.empty(0, 3, 3), inv_cell=torch.empty(0, 3, 3)):
        """Energies ``[nbatch]`` (no self energies); differentiable with respect to ``X`` (upstream :69-102)."""
        assert X.is_cuda, "X tensor must reside on GPU"
        assert Z.device == X.device, "Z tensor must reside on the same GPU as X"
        assert atom_counts.device == X.device, "atom_counts tensor must reside on the same GPU as X"
        red = self.reductors
        if self._pad > 0:
            red = torch.nn.functional.pad(red, [0, self._pad])
        return torch.ops.qml_lightning_b200.rff_energy(X, Z, atom_counts, cell, inv_cell, self.rep.species, self.rep.Rs2,
                                                       self.rep.Rs3, self.rep.kernel_scalars, self.species, red,
                                                       self.packed, atomIDs.shape[0], self.fast_math)

    def predict_opt(self, coordinates, charges, atomIDs, molIDs, natom_counts, zcells=None, zinv_cells=None, forces=True,
                    print_info=False, profiler=False):
        if self.is_trained is False:
            raise RuntimeError("must train the model first by calling train()!")
        dev = coordinates.device
        energies, grad = cabi.rff_predict_packed(coordinates, charges, natom_counts, self.rep.kernel_params(dev), self.species,
                                                 self.kernel_reductors(), self.packed, zcells, zinv_cells,
                                                 n_atoms_upper=atomIDs.shape[0], fast_math=self.fast_math,
                                                 pca_packed=self.pca_packed())
        if print_info:
            torch.cuda.synchronize()
            print("prediction for", coordinates.shape[0], "molecules")
        return (energies, -grad) if forces else energies

    def predict(self, X, Z, max_natoms, cells=None, inv_cells=None, forces=True, print_info=False, profiler=False):
        n = len(X)
        energies = torch.zeros(n, device=self.device, dtype=torch.float32)
        all_forces = torch.zeros(n, max_natoms, 3, device=self.device, dtype=torch.float32)
        for i in range(0, n, self.nbatch_test):
            sl = slice(i, i + self.nbatch_test)
            data = self.format_data(X[sl], Z[sl], cells=None if cells is None else cells[sl],
                                    inv_cells=None if inv_cells is None else inv_cells[sl])
            out = self.predict_opt(data['coordinates'], data['charges'], data['atomIDs'], data['molIDs'], data['natom_counts'],
                                   data['cells'], data['inv_cells'], forces=forces)
            if forces:
                energies[sl] = out[0]
                all_forces[sl, :out[1].shape[1]] = out[1]
            else:
                energies[sl] = out
        return (energies, all_forces) if forces else energies

    def save_jit_model(self, file_name='model_rff.pt'):
        script = torch.jit.script(self)
        script.save(file_name)
