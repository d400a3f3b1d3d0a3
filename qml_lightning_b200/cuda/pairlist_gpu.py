"""``pairlist_gpu`` of the upstream project (cuda/pairlist_cuda.cpp:21-72)."""
from .. import cabi


def get_num_neighbours_gpu(coordinates, natoms, rcut, lattice_vecs, inv_lattice_vecs):
    """``i32[nbatch, max(natoms)]`` neighbour counts (pairlist_cuda.cpp:21-37)."""
    return cabi.num_neighbours(coordinates, natoms, rcut, lattice_vecs, inv_lattice_vecs, A_out=int(natoms.max().item()))


def get_neighbour_list_gpu(coordinates, natoms, max_neighbours, rcut, lattice_vecs, inv_lattice_vecs):
    """``i32[nbatch, max(natoms), max_neighbours]``, ascending neighbour index, padded with -1 (pairlist_cuda.cpp:47-65)."""
    return cabi.neighbour_list(coordinates, natoms, max_neighbours, rcut, lattice_vecs, inv_lattice_vecs,
                               A_out=int(natoms.max().item()))


def safe_fill_gpu(pairlist):
    """Upstream fills the list with -1 before building it (pairlist_cuda.cpp:39-45)."""
    pairlist.fill_(-1)
