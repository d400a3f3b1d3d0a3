"""``fchl_gpu`` of the upstream project (cuda/fchl_cuda.cpp:28-212).  ``three_body_weight`` is the already scaled value
the upstream Python class passes (representations/FCHL.py:35)."""
import torch

from .. import cabi


def _params(species, Rs2, Rs3, eta2, eta3, two_body_decay, three_body_weight, three_body_decay, rcut):
    return cabi.FchlKernelParams(species, Rs2, Rs3, eta2, eta3, two_body_decay, three_body_weight, three_body_decay, rcut)


def _counts(charges, blockMolIDs):
    """Atoms per molecule from upstream's per-atom molecule ids (kernel.py:601-722 builds them in molecule order)."""
    nb = charges.shape[0]
    return torch.bincount(blockMolIDs.long(), minlength=nb).to(torch.int32)


def get_element_types_gpu(coordinates, charges, natom_counts, species):
    return cabi.element_types(coordinates, charges, natom_counts, species)


def get_fchl_representation(coordinates, charges, species, element_types, cell, inv_cell, blockAtomIDs, blockMolIDs,
                            neighbourlist, nneighbours, two_body_gridpoints, three_body_gridpoints, eta2, eta3,
                            two_body_decay, three_body_weight, three_body_decay, rcut):
    """``f32[nbatch, natoms, repsize]`` (fchl_cuda.cpp:56-90)."""
    p = _params(species, two_body_gridpoints, three_body_gridpoints, eta2, eta3, two_body_decay, three_body_weight,
                three_body_decay, rcut)
    return cabi.fchl19_forward(coordinates, charges, _counts(charges, blockMolIDs), p, cell, inv_cell)


def get_fchl_and_derivative(coordinates, charges, species, element_types, cell, inv_cell, blockAtomIDs, blockMolIDs,
                            neighbourlist, nneighbours, two_body_gridpoints, three_body_gridpoints, eta2, eta3,
                            two_body_decay, three_body_weight, three_body_decay, rcut, gradients):
    """``[rep]`` or ``[rep, jac f32[nbatch, natoms, natoms, 3, repsize]]`` (fchl_cuda.cpp:157-202)."""
    p = _params(species, two_body_gridpoints, three_body_gridpoints, eta2, eta3, two_body_decay, three_body_weight,
                three_body_decay, rcut)
    counts = _counts(charges, blockMolIDs)
    if not gradients:
        return [cabi.fchl19_forward(coordinates, charges, counts, p, cell, inv_cell)]
    rep, jac = cabi.fchl19_forward_jacobian(coordinates, charges, counts, p, cell, inv_cell)
    return [rep, jac]


def get_fchl_derivative(coordinates, charges, species, element_types, cell, inv_cell, blockAtomIDs, blockMolIDs,
                        neighbourlist, nneighbours, two_body_gridpoints, three_body_gridpoints, eta2, eta3,
                        two_body_decay, three_body_weight, three_body_decay, rcut):
    """The explicit Jacobian alone (fchl_cuda.cpp:92-126)."""
    return get_fchl_and_derivative(coordinates, charges, species, element_types, cell, inv_cell, blockAtomIDs, blockMolIDs,
                                   neighbourlist, nneighbours, two_body_gridpoints, three_body_gridpoints, eta2, eta3,
                                   two_body_decay, three_body_weight, three_body_decay, rcut, True)[1]


def fchl_backwards(coordinates, charges, species, element_types, cell, inv_cell, blockAtomIDs, blockMolIDs, neighbourlist,
                   nneighbours, two_body_gridpoints, three_body_gridpoints, eta2, eta3, two_body_decay, three_body_weight,
                   three_body_decay, rcut, grad_in):
    """Vector-Jacobian product ``f32[nbatch, natoms, 3]`` for ``grad_in f32[nbatch, natoms, repsize]`` (fchl_cuda.cpp:128-155)."""
    p = _params(species, two_body_gridpoints, three_body_gridpoints, eta2, eta3, two_body_decay, three_body_weight,
                three_body_decay, rcut)
    return cabi.fchl19_backward(coordinates, charges, _counts(charges, blockMolIDs), p, grad_in, cell, inv_cell)
