"""``FCHLCuda``: the FCHL19 representation module with the upstream constructor and methods
(upstream qml_lightning/representations/FCHL.py:16-132), backed by the qmlb200 kernels.
"""
import numpy as np
import torch

from .. import cabi


def _default_device():
    return torch.device('cuda', torch.cuda.current_device()) if torch.cuda.is_available() else torch.device('cpu')


class FCHLCuda(torch.nn.Module):

    def __init__(self, species=np.array([1, 6, 7, 8]), rcut=6.0, nRs2=24, nRs3=20,
                 eta2=0.32, eta3=2.7, two_body_decay=1.8, three_body_weight=13.4, three_body_decay=0.57, device=None):
        super().__init__()
        dev = torch.device(device) if device is not None else _default_device()
        species = np.asarray(species)
        self.species = torch.from_numpy(species).float().to(dev)
        self.nspecies = len(species)
        # hyper-parameters stay 0-dim CPU tensors: saved upstream models pass them to the operators that way
        self.rcut = torch.tensor(rcut)
        self.nRs2 = torch.tensor(nRs2)
        self.nRs3 = torch.tensor(nRs3)
        self.eta2 = torch.tensor(eta2)
        self.eta3 = torch.tensor(eta3)
        self.two_body_decay = torch.tensor(two_body_decay)
        # the kernels take the weight already multiplied by sqrt(eta3/pi) (upstream FCHL.py:35)
        self.three_body_weight = np.sqrt(eta3 / np.pi) * torch.tensor(three_body_weight)
        self.three_body_decay = torch.tensor(three_body_decay)
        # grids without the point at zero (upstream FCHL.py:39-40)
        self.Rs2 = torch.linspace(0.0, rcut, nRs2 + 1)[1:].to(dev)
        self.Rs3 = torch.linspace(0.0, rcut, nRs3 + 1)[1:].to(dev)
        self.fp_size = self.nspecies * nRs2 + (self.nspecies * (self.nspecies + 1)) * nRs3
        self.pi = (torch.acos(torch.zeros(1)) * 2).to(dev)
        self.device = dev
        # eta2, eta3, two_body_decay, three_body_weight, three_body_decay, rcut for the fused operator
        self.kernel_scalars = torch.tensor([float(self.eta2), float(self.eta3), float(self.two_body_decay),
                                            float(self.three_body_weight), float(self.three_body_decay), float(self.rcut)],
                                           dtype=torch.float64)

    def kernel_params(self, device=None):
        dev = device if device is not None else self.species.device
        s = self.kernel_scalars.tolist()
        return cabi.FchlKernelParams(self.species.to(dev), self.Rs2.to(dev), self.Rs3.to(dev), *s)

    def get_repsize(self):
        return self.fp_size

    def get_neighbourlist(self, X, Z, max_neighbours, atom_counts, cell=None, inv_cell=None):
        return cabi.neighbour_list(X, atom_counts, max_neighbours, self.rcut.item(), cell, inv_cell,
                                   A_out=int(atom_counts.max().item()))

    def get_neighbours(self, X, Z, atom_counts, cell=None, inv_cell=None):
        return cabi.num_neighbours(X, atom_counts, self.rcut.item(), cell, inv_cell, A_out=int(atom_counts.max().item()))

    def get_element_types(self, X, Z, atom_counts):
        return cabi.element_types(X, Z, atom_counts, self.species.to(Z.device))

    def get_representation(self, X, Z, atomIDs, molIDs, atom_counts, cell=None, inv_cell=None, nneighbours=None,
                           neighbourlist=None):
        """``[nbatch, natoms, repsize]``.  Neighbours are found inside the kernel; ``nneighbours`` / ``neighbourlist`` are
        accepted for signature compatibility and ignored."""
        return cabi.fchl19_forward(X, Z, atom_counts, self.kernel_params(X.device), cell, inv_cell)

    def get_representation_and_derivative(self, X, Z, atomIDs, molIDs, atom_counts, cell=None, inv_cell=None,
                                          nneighbours=None, neighbourlist=None):
        """Representation and its explicit Jacobian ``[nbatch, natoms, natoms, 3, repsize]``."""
        return cabi.fchl19_forward_jacobian(X, Z, atom_counts, self.kernel_params(X.device), cell, inv_cell)

    def rep_deriv_fd(self, X, Z, atomIDs, molIDs, natom_counts, cells=None, inv_cells=None, dx=0.005):
        """Central finite differences of the representation (float64 accumulation of float32 evaluations)."""
        out = torch.zeros(X.shape[0], X.shape[1], X.shape[1], 3, self.fp_size, dtype=torch.float64, device=X.device)
        for i in range(X.shape[1]):
            for x in range(3):
                Xp = X.clone()
                Xp[:, i, x] += dx
                plus = self.get_representation(Xp, Z, atomIDs, molIDs, natom_counts, cells, inv_cells)
                Xp[:, i, x] -= 2.0 * dx
                minus = self.get_representation(Xp, Z, atomIDs, molIDs, natom_counts, cells, inv_cells)
                out[:, :, i, x, :] = (plus.double() - minus.double()) / (2.0 * dx)
        return out

    def forward(self, X, Z, atomIDs, molIDs, atom_counts, cell=torch.empty(0, 3, 3), inv_cell=torch.empty(0, 3, 3)):
        return torch.ops.qml_lightning_fchl.fchl_forwards(X, Z, self.species, atomIDs, molIDs, atom_counts,
                                                          cell.to(X.device), inv_cell.to(X.device),
                                                          self.Rs2, self.Rs3, self.eta2, self.eta3, self.two_body_decay,
                                                          self.three_body_weight, self.three_body_decay, self.rcut)
