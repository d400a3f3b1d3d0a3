"""Thin torch-tensor wrappers over the C ABI of ``libqmlb200.so``.

PyTorch is used only as the owner of device memory and of the current CUDA stream: every function checks its tensors
(CUDA, contiguous, dtype), allocates outputs with ``torch.empty`` and passes raw pointers plus the current stream to
the C entry point of the same name (``qmlb_<name>``).  No arithmetic happens in Python.
"""
import ctypes
import functools
import os

import torch

from . import _lib
from ._lib import FchlParamsC, check

ROW_TILE = 128  # QMLB_ROW_TILE


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _p(t, dtype=None, name='tensor'):
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")  # wording of the upstream TORCH_CHECKs (FCHL19.cpp:40-44)
    if dtype is not None and t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    return ctypes.c_void_p(t.data_ptr())


def _cells(cell, inv_cell):
    """Upstream passes empty [0,3,3] tensors for non-periodic input; the C ABI takes NULL."""
    if cell is None or cell.numel() == 0:
        return None, None
    return cell.contiguous().float(), inv_cell.contiguous().float()


class FchlKernelParams:
    """Device-resident FCHL19 grids plus the kernel-level scalars (``qmlb_fchl_params``)."""

    def __init__(self, species, Rs2, Rs3, eta2, eta3, two_body_decay, three_body_weight, three_body_decay, rcut):
        self.species = species.contiguous().float()
        self.Rs2 = Rs2.contiguous().float()
        self.Rs3 = Rs3.contiguous().float()
        self.scalars = tuple(float(v) for v in (eta2, eta3, two_body_decay, three_body_weight, three_body_decay, rcut))
        self.repsize = _lib.load().qmlb_fchl19_repsize(self.species.numel(), self.Rs2.numel(), self.Rs3.numel())

    def c(self):
        eta2, eta3, d2, w3, d3, rcut = self.scalars
        return FchlParamsC(_p(self.species, torch.float32, 'species'), self.species.numel(),
                           _p(self.Rs2, torch.float32, 'Rs2'), self.Rs2.numel(),
                           _p(self.Rs3, torch.float32, 'Rs3'), self.Rs3.numel(), eta2, eta3, d2, w3, d3, rcut)


def _batch(X, Z, atom_counts):
    if X.dim() == 2:
        X = X.unsqueeze(0)
    if Z.dim() == 1:
        Z = Z.unsqueeze(0)
    X = X.contiguous()
    Z = Z.contiguous()
    nb, A = Z.shape
    return X, Z, atom_counts.contiguous(), nb, A


def element_types(X, Z, atom_counts, species):
    X, Z, atom_counts, nb, A = _batch(X, Z, atom_counts)
    out = torch.zeros(nb, A, dtype=torch.int32, device=Z.device)
    check(_lib.load().qmlb_element_types(_p(Z, torch.float32, 'charges'), _p(atom_counts, torch.int32, 'natom_counts'),
                                         _p(species, torch.float32, 'species'), species.numel(), nb, A, _p(out),
                                         _stream(Z.device)), 'qmlb_element_types')
    return out


def num_neighbours(X, atom_counts, rcut, cell=None, inv_cell=None, A_out=None):
    if X.dim() == 2:
        X = X.unsqueeze(0)
    X = X.contiguous()
    nb, A = X.shape[0], X.shape[1]
    A_out = A if A_out is None else int(A_out)
    cell, inv_cell = _cells(cell, inv_cell)
    out = torch.zeros(nb, A_out, dtype=torch.int32, device=X.device)
    check(_lib.load().qmlb_num_neighbours(_p(X, torch.float32, 'coordinates'), _p(atom_counts.contiguous(), torch.int32, 'natoms'),
                                          nb, A, float(rcut), _p(cell), _p(inv_cell), _p(out), A_out, _stream(X.device)),
          'qmlb_num_neighbours')
    return out


def neighbour_list(X, atom_counts, max_neighbours, rcut, cell=None, inv_cell=None, A_out=None):
    if X.dim() == 2:
        X = X.unsqueeze(0)
    X = X.contiguous()
    nb, A = X.shape[0], X.shape[1]
    A_out = A if A_out is None else int(A_out)
    cell, inv_cell = _cells(cell, inv_cell)
    out = torch.full((nb, A_out, int(max_neighbours)), -1, dtype=torch.int32, device=X.device)
    check(_lib.load().qmlb_neighbour_list(_p(X, torch.float32, 'coordinates'), _p(atom_counts.contiguous(), torch.int32, 'natoms'),
                                          nb, A, float(rcut), _p(cell), _p(inv_cell), int(max_neighbours), _p(out), A_out,
                                          _stream(X.device)), 'qmlb_neighbour_list')
    return out


def fchl19_forward(X, Z, atom_counts, params, cell=None, inv_cell=None, row_of_slot=None, out=None):
    X, Z, atom_counts, nb, A = _batch(X, Z, atom_counts)
    cell, inv_cell = _cells(cell, inv_cell)
    if out is None:
        assert row_of_slot is None
        out = torch.empty(nb, A, params.repsize, dtype=torch.float32, device=X.device)
    pc = params.c()
    check(_lib.load().qmlb_fchl19_forward(_p(X, torch.float32, 'coordinates'), _p(Z, torch.float32, 'charges'),
                                          _p(atom_counts, torch.int32, 'atom_counts'), nb, A, ctypes.byref(pc), _p(cell),
                                          _p(inv_cell), _p(row_of_slot, torch.int32, 'row_of_slot'),
                                          _p(out, torch.float32, 'rep'), _stream(X.device)), 'qmlb_fchl19_forward')
    return out


def fchl19_backward(X, Z, atom_counts, params, grad_rep, cell=None, inv_cell=None, row_of_slot=None, atom_energy=None):
    X, Z, atom_counts, nb, A = _batch(X, Z, atom_counts)
    cell, inv_cell = _cells(cell, inv_cell)
    grad_X = torch.empty(nb, A, 3, dtype=torch.float32, device=X.device)
    mol_energy = torch.empty(nb, dtype=torch.float32, device=X.device) if atom_energy is not None else None
    pc = params.c()
    check(_lib.load().qmlb_fchl19_backward(_p(X, torch.float32, 'coordinates'), _p(Z, torch.float32, 'charges'),
                                           _p(atom_counts, torch.int32, 'atom_counts'), nb, A, ctypes.byref(pc), _p(cell),
                                           _p(inv_cell), _p(row_of_slot, torch.int32, 'row_of_slot'),
                                           _p(grad_rep.contiguous(), torch.float32, 'grad_rep'), _p(grad_X),
                                           _p(atom_energy, torch.float32, 'atom_energy'), _p(mol_energy),
                                           _stream(X.device)), 'qmlb_fchl19_backward')
    return (grad_X, mol_energy) if atom_energy is not None else grad_X


def fchl19_forward_jacobian(X, Z, atom_counts, params, cell=None, inv_cell=None, grouping=None):
    """Representation and explicit Jacobian; in element-grouped row order when ``grouping`` is given."""
    X, Z, atom_counts, nb, A = _batch(X, Z, atom_counts)
    cell, inv_cell = _cells(cell, inv_cell)
    if grouping is None:
        rep = torch.empty(nb, A, params.repsize, dtype=torch.float32, device=X.device)
        jac = torch.empty(nb, A, A, 3, params.repsize, dtype=torch.float32, device=X.device)
        ros = None
    else:
        rep = torch.zeros(grouping.rows_cap, params.repsize, dtype=torch.float32, device=X.device)
        jac = torch.zeros(grouping.rows_cap, A, 3, params.repsize, dtype=torch.float32, device=X.device)
        ros = grouping.row_of_slot
    pc = params.c()
    check(_lib.load().qmlb_fchl19_forward_jacobian(_p(X, torch.float32, 'coordinates'), _p(Z, torch.float32, 'charges'),
                                                   _p(atom_counts, torch.int32, 'atom_counts'), nb, A, ctypes.byref(pc),
                                                   _p(cell), _p(inv_cell), _p(ros), _p(rep), _p(jac), _stream(X.device)),
          'qmlb_fchl19_forward_jacobian')
    return rep, jac


class Grouping:
    """Element-grouped row order of one batch (see ``qmlb_group_by_element``)."""

    def __init__(self, row_of_slot, slot_of_row, group_start, rows_cap, nelements):
        self.row_of_slot, self.slot_of_row, self.group_start = row_of_slot, slot_of_row, group_start
        self.rows_cap, self.nelements = rows_cap, nelements


def grouping_from_ordering(ordering, nmol, A=None):
    """Single-element :class:`Grouping` for ``n`` rows whose molecules are given by ``ordering[n]`` (upstream's
    ``batch_indexes`` / ``indexes`` argument): row ``a`` becomes the ``k``-th row of molecule ``ordering[a]`` and gets the
    private slot ``ordering[a] * A + k``.  Returns ``(grouping, A)`` with ``A`` = rows per molecule (at least the largest
    count found).  Uses a few torch index operations and one host read of the largest count."""
    dev = ordering.device
    n = ordering.shape[0]
    idx = ordering.long()
    order = torch.argsort(idx, stable=True)
    cnt = torch.bincount(idx, minlength=int(nmol))
    first = torch.cumsum(cnt, 0) - cnt
    rank = torch.empty_like(idx)
    rank[order] = torch.arange(n, device=dev) - first[idx[order]]
    most = int(cnt.max()) if n else 0
    if A is None:
        A = max(most, 1)
    elif most > A:
        raise RuntimeError("more rows of one molecule than atoms in the derivative tensor")
    rows_cap = max((n + ROW_TILE - 1) // ROW_TILE * ROW_TILE, ROW_TILE)
    slot = (idx * A + rank).to(torch.int32)
    slot_of_row = torch.full((rows_cap,), -1, dtype=torch.int32, device=dev)
    slot_of_row[:n] = slot
    row_of_slot = torch.full((int(nmol) * A,), -1, dtype=torch.int32, device=dev)
    row_of_slot[slot.long()] = torch.arange(n, dtype=torch.int32, device=dev)
    group_start = torch.tensor([0, n], dtype=torch.int32, device=dev)
    return Grouping(row_of_slot, slot_of_row, group_start, rows_cap, 1), A


def pad_rows(t, rows_cap):
    """``t`` with its first dimension zero-padded to ``rows_cap`` (the row capacity of a :class:`Grouping`)."""
    if t.shape[0] == rows_cap:
        return t.contiguous()
    out = torch.zeros((rows_cap,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    out[:t.shape[0]] = t
    return out


def group_by_element(Z, atom_counts, elements, n_atoms_upper=None):
    Z = Z.contiguous()
    nb, A = Z.shape
    lib = _lib.load()
    nel = elements.numel()
    upper = nb * A if n_atoms_upper is None else min(int(n_atoms_upper), nb * A)
    rows_cap = lib.qmlb_rows_capacity(upper, nel)
    dev = Z.device
    row_of_slot = torch.empty(nb * A, dtype=torch.int32, device=dev)
    slot_of_row = torch.empty(rows_cap, dtype=torch.int32, device=dev)
    group_start = torch.empty(nel + 1, dtype=torch.int32, device=dev)
    scratch = torch.empty(lib.qmlb_group_scratch_bytes(nb, nel), dtype=torch.uint8, device=dev)
    check(lib.qmlb_group_by_element(_p(Z, torch.float32, 'charges'), _p(atom_counts.contiguous(), torch.int32, 'atom_counts'),
                                    _p(elements.contiguous(), torch.float32, 'elements'), nel, nb, A, _p(row_of_slot),
                                    _p(slot_of_row), _p(group_start), rows_cap, _p(scratch), _stream(dev)),
          'qmlb_group_by_element')
    return Grouping(row_of_slot, slot_of_row, group_start, rows_cap, nel)


def pca_project(inp, reductors, grouping, transpose=False, out=None, tensor_cores=False):
    nel, repsize, npcas = reductors.shape
    rows = grouping.rows_cap
    width = repsize if transpose else npcas
    if out is None:
        out = torch.empty(rows, width, dtype=torch.float32, device=inp.device)
    if tensor_cores:
        check(_lib.load().qmlb_pca_project_tc(_p(inp, torch.float32, 'in'), _p(reductors.contiguous(), torch.float32, 'reductors'),
                                              _p(grouping.group_start), nel, rows, 1, repsize, npcas, int(bool(transpose)),
                                              _p(out), _stream(inp.device)), 'qmlb_pca_project_tc')
        return out
    check(_lib.load().qmlb_pca_project(_p(inp, torch.float32, 'in'), _p(reductors.contiguous(), torch.float32, 'reductors'),
                                       _p(grouping.group_start), nel, rows, repsize, npcas, int(bool(transpose)), _p(out),
                                       _stream(inp.device)), 'qmlb_pca_project')
    return out


def tc_timeouts():
    """Number of tensor-core blocks that ever gave up on a bounded wait (synchronises the device)."""
    return _lib.load().qmlb_tc_timeouts()


def sorf_coefficients(u, D, normalisation, ntransforms):
    u = u.contiguous()
    D = D.contiguous()
    n, N = u.shape
    T, S, N2 = D.shape
    if N2 != N or T < int(ntransforms):
        raise RuntimeError("dmatrix shape does not match the input")
    out = torch.empty(n, S, N, dtype=torch.float32, device=u.device)
    check(_lib.load().qmlb_sorf_coefficients(_p(u, torch.float32, 'input'), _p(D, torch.float32, 'dmatrix'), n, N, S,
                                             int(ntransforms), float(normalisation), _p(out), _stream(u.device)),
          'qmlb_sorf_coefficients')
    return out


def sorf_coefficients_backward(grad, D, normalisation, ntransforms):
    grad = grad.contiguous()
    D = D.contiguous()
    n, S, N = grad.shape
    out = torch.empty(n, N, dtype=torch.float32, device=grad.device)
    check(_lib.load().qmlb_sorf_coefficients_backward(_p(grad, torch.float32, 'grad'), _p(D, torch.float32, 'dmatrix'), n, N,
                                                      S, int(ntransforms), float(normalisation), _p(out),
                                                      _stream(grad.device)), 'qmlb_sorf_coefficients_backward')
    return out


def cos_features(coeffs, bias, nmol, batch_indexes):
    coeffs = coeffs.contiguous()
    n, F = coeffs.shape
    out = torch.empty(int(nmol), F, dtype=torch.float32, device=coeffs.device)
    check(_lib.load().qmlb_cos_features(_p(coeffs, torch.float32, 'coeffs'), _p(bias.contiguous(), torch.float32, 'b'),
                                        _p(batch_indexes.contiguous(), torch.int32, 'batch_indexes'), n, F, int(nmol),
                                        _p(out), _stream(coeffs.device)), 'qmlb_cos_features')
    return out


def cos_features_backward(grads, coeffs, bias, batch_indexes):
    coeffs = coeffs.contiguous()
    n, F = coeffs.shape
    out = torch.empty(n, F, dtype=torch.float32, device=coeffs.device)
    check(_lib.load().qmlb_cos_features_backward(_p(grads.contiguous(), torch.float32, 'grads'), _p(coeffs, torch.float32, 'coeffs'),
                                                 _p(bias.contiguous(), torch.float32, 'b'),
                                                 _p(batch_indexes.contiguous(), torch.int32, 'batch_indexes'), n, F, _p(out),
                                                 _stream(coeffs.device)), 'qmlb_cos_features_backward')
    return out


def sorf_pack(Dmat, bias, alpha):
    """Dmat f32[nel,T,S,N], bias f32[nel,S*N], alpha f32[S*N] -> opaque packed parameter buffer."""
    Dmat = Dmat.contiguous().float()
    nel, T, S, N = Dmat.shape
    lib = _lib.load()
    packed = torch.empty(lib.qmlb_sorf_pack_bytes(nel, N, S, T) // 4, dtype=torch.float32, device=Dmat.device)
    check(lib.qmlb_sorf_pack(_p(Dmat, torch.float32, 'Dmat'), _p(bias.contiguous().float(), torch.float32, 'bias'),
                             _p(alpha.contiguous().float(), torch.float32, 'alpha'), nel, N, S, T, _p(packed),
                             _stream(Dmat.device)), 'qmlb_sorf_pack')
    return packed


def sorf_energy_grad(x, grouping, packed, N, S, T, sigma, fast_math=True):
    rows = grouping.rows_cap
    dev = x.device
    atom_energy = torch.empty(rows, dtype=torch.float32, device=dev)
    grad_x = torch.empty(rows, N, dtype=torch.float32, device=dev)
    check(_lib.load().qmlb_sorf_energy_grad(_p(x, torch.float32, 'x'), _p(grouping.group_start), _p(grouping.slot_of_row),
                                            grouping.nelements, rows, N, S, T, float(sigma), _p(packed), int(bool(fast_math)),
                                            _p(atom_energy), _p(grad_x), _stream(dev)), 'qmlb_sorf_energy_grad')
    return atom_energy, grad_x


def sorf_predict_staged(X, Z, atom_counts, fchl, elements, reductors, packed, S, T, sigma, cell=None, inv_cell=None,
                        n_atoms_upper=None, fast_math=True):
    """Same result as ``sorf_predict`` through the individual stage entry points (used by tests and profiling)."""
    X, Z, atom_counts, nb, A = _batch(X, Z, atom_counts)
    nel, repsize, N = reductors.shape
    g = group_by_element(Z, atom_counts, elements, n_atoms_upper)
    rep = torch.empty(g.rows_cap, repsize, dtype=torch.float32, device=X.device)
    fchl19_forward(X, Z, atom_counts, fchl, cell, inv_cell, row_of_slot=g.row_of_slot, out=rep)
    x = pca_project(rep, reductors, g, transpose=False)
    atom_energy, grad_x = sorf_energy_grad(x, g, packed, N, S, T, sigma, fast_math)
    pca_project(grad_x, reductors, g, transpose=True, out=rep)  # rep buffer reused for d/d(rep)
    grad_X, energy = fchl19_backward(X, Z, atom_counts, fchl, rep, cell, inv_cell, row_of_slot=g.row_of_slot,
                                     atom_energy=atom_energy)
    return energy, grad_X


_workspaces = {}


def _workspace(device, nbytes):
    """Grow-only scratch buffer per (device, stream), so steady-state prediction allocates nothing and predictions
    issued on different streams never share scratch.  A buffer that is outgrown goes back to the caching allocator,
    which keeps it away from other streams until the work queued on its own stream has finished."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(int(nbytes * 1.1) + 256, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def pca_pair_pack(reductors):
    """Split and tiled images of the projection matrices for both directions (``qmlb_pca_pair_pack``); pass the result
    as ``pca_packed`` to the predict functions so that nothing is re-packed per call."""
    nel, repsize, N = reductors.shape
    lib = _lib.load()
    nbytes = lib.qmlb_pca_pair_pack_bytes(nel, repsize, N)
    packed = torch.empty(nbytes, dtype=torch.uint8, device=reductors.device)
    check(lib.qmlb_pca_pair_pack(_p(reductors.contiguous(), torch.float32, 'reductors'), nel, repsize, N, _p(packed), nbytes,
                                 _stream(reductors.device)), 'qmlb_pca_pair_pack')
    return packed


def sorf_predict(X, Z, atom_counts, fchl, elements, reductors, packed, S, T, sigma, cell=None, inv_cell=None,
                 n_atoms_upper=None, fast_math=True, energy=None, grad_X=None, pca_packed=None):
    """Energies ``[nb]`` and ``dE/dX [nb,A,3]`` through ``qmlb_sorf_predict`` (one C call, no host sync)."""
    X, Z, atom_counts, nb, A = _batch(X, Z, atom_counts)
    cell, inv_cell = _cells(cell, inv_cell)
    nel, repsize, N = reductors.shape
    lib = _lib.load()
    upper = nb * A if n_atoms_upper is None else int(n_atoms_upper)
    if energy is None:
        energy = torch.empty(nb, dtype=torch.float32, device=X.device)
    if grad_X is None:
        grad_X = torch.empty(nb, A, 3, dtype=torch.float32, device=X.device)
    if nb == 0:
        return energy, grad_X
    need = lib.qmlb_predict_workspace_bytes(nb, A, upper, nel, repsize, N)
    ws = _workspace(X.device, need)
    pc = fchl.c()
    check(lib.qmlb_sorf_predict(_p(X, torch.float32, 'coordinates'), _p(Z, torch.float32, 'charges'),
                                _p(atom_counts, torch.int32, 'atom_counts'), nb, A, ctypes.byref(pc), _p(cell), _p(inv_cell),
                                _p(elements.contiguous(), torch.float32, 'elements'), nel,
                                _p(reductors.contiguous(), torch.float32, 'reductors'), _p(pca_packed), N, _p(packed), int(S), int(T),
                                float(sigma), int(bool(fast_math)), upper, _p(ws), ws.numel(), _p(energy), _p(grad_X),
                                _stream(X.device)), 'qmlb_sorf_predict')
    return energy, grad_X


def rff_energy_grad(x, grouping, W, b, alpha, fast_math=True):
    """Per-row energies and gradients of the RFF feature stage (``qmlb_rff_energy_grad``)."""
    nel, K, D = W.shape
    rows = grouping.rows_cap
    atom_energy = torch.empty(rows, dtype=torch.float32, device=x.device)
    grad_x = torch.empty(rows, K, dtype=torch.float32, device=x.device)
    check(_lib.load().qmlb_rff_energy_grad(_p(x, torch.float32, 'x'), _p(grouping.group_start), _p(grouping.slot_of_row), nel,
                                           rows, K, D, _p(W.contiguous(), torch.float32, 'W'),
                                           _p(b.contiguous(), torch.float32, 'b'), _p(alpha.contiguous(), torch.float32, 'alpha'),
                                           int(bool(fast_math)), _p(atom_energy), _p(grad_x), _stream(x.device)),
          'qmlb_rff_energy_grad')
    return atom_energy, grad_x


def rff_pack(W, b, alpha):
    """Packed fp16 hi/lo image of the RFF parameters for the tensor-core kernel (``qmlb_rff_pack``); uint8 tensor."""
    nel, K, D = W.shape
    lib = _lib.load()
    nbytes = lib.qmlb_rff_pack_bytes(nel, K, D)
    if nbytes == 0:
        raise RuntimeError(f'qmlb_rff_pack: unsupported sizes (nelements={nel}, npcas={K}, nfeatures={D})')
    packed = torch.empty(nbytes, dtype=torch.uint8, device=W.device)
    check(lib.qmlb_rff_pack(_p(W.contiguous(), torch.float32, 'W'), _p(b.contiguous(), torch.float32, 'b'),
                            _p(alpha.contiguous(), torch.float32, 'alpha'), nel, K, D, _p(packed), nbytes, _stream(W.device)),
          'qmlb_rff_pack')
    return packed


def rff_energy_grad_tc(x, grouping, packed, nelements, fast_math=True):
    """Tensor-core version of :func:`rff_energy_grad` on parameters packed by :func:`rff_pack`."""
    rows = grouping.rows_cap
    K = x.shape[1]
    atom_energy = torch.empty(rows, dtype=torch.float32, device=x.device)
    grad_x = torch.empty(rows, K, dtype=torch.float32, device=x.device)
    check(_lib.load().qmlb_rff_energy_grad_tc(_p(x, torch.float32, 'x'), _p(grouping.group_start), _p(grouping.slot_of_row),
                                              int(nelements), rows, K, _p(packed), int(bool(fast_math)), _p(atom_energy),
                                              _p(grad_x), _stream(x.device)), 'qmlb_rff_energy_grad_tc')
    return atom_energy, grad_x


def rff_predict(X, Z, atom_counts, fchl, elements, reductors, W, b, alpha, cell=None, inv_cell=None, n_atoms_upper=None,
                fast_math=True, energy=None, grad_X=None, pca_packed=None):
    """Energies ``[nb]`` and ``dE/dX [nb,A,3]`` of the RFF model through ``qmlb_rff_predict``."""
    X, Z, atom_counts, nb, A = _batch(X, Z, atom_counts)
    cell, inv_cell = _cells(cell, inv_cell)
    nel, repsize, N = reductors.shape
    D = W.shape[-1]
    lib = _lib.load()
    upper = nb * A if n_atoms_upper is None else int(n_atoms_upper)
    if energy is None:
        energy = torch.empty(nb, dtype=torch.float32, device=X.device)
    if grad_X is None:
        grad_X = torch.empty(nb, A, 3, dtype=torch.float32, device=X.device)
    if nb == 0:
        return energy, grad_X
    ws = _workspace(X.device, lib.qmlb_predict_workspace_bytes(nb, A, upper, nel, repsize, N))
    pc = fchl.c()
    check(lib.qmlb_rff_predict(_p(X, torch.float32, 'coordinates'), _p(Z, torch.float32, 'charges'),
                               _p(atom_counts, torch.int32, 'atom_counts'), nb, A, ctypes.byref(pc), _p(cell), _p(inv_cell),
                               _p(elements.contiguous(), torch.float32, 'elements'), nel,
                               _p(reductors.contiguous(), torch.float32, 'reductors'), _p(pca_packed), N,
                               _p(W.contiguous(), torch.float32, 'W'), _p(b.contiguous(), torch.float32, 'b'),
                               _p(alpha.contiguous(), torch.float32, 'alpha'), D, int(bool(fast_math)), upper, _p(ws),
                               ws.numel(), _p(energy), _p(grad_X), _stream(X.device)), 'qmlb_rff_predict')
    return energy, grad_X


def rff_predict_packed(X, Z, atom_counts, fchl, elements, reductors, packed, cell=None, inv_cell=None, n_atoms_upper=None,
                       fast_math=True, energy=None, grad_X=None, pca_packed=None):
    """:func:`rff_predict` on parameters packed by :func:`rff_pack` (tensor-core feature stage, ``qmlb_rff_predict_packed``)."""
    X, Z, atom_counts, nb, A = _batch(X, Z, atom_counts)
    cell, inv_cell = _cells(cell, inv_cell)
    nel, repsize, N = reductors.shape
    lib = _lib.load()
    upper = nb * A if n_atoms_upper is None else int(n_atoms_upper)
    if energy is None:
        energy = torch.empty(nb, dtype=torch.float32, device=X.device)
    if grad_X is None:
        grad_X = torch.empty(nb, A, 3, dtype=torch.float32, device=X.device)
    if nb == 0:
        return energy, grad_X
    ws = _workspace(X.device, lib.qmlb_predict_workspace_bytes(nb, A, upper, nel, repsize, N))
    pc = fchl.c()
    check(lib.qmlb_rff_predict_packed(_p(X, torch.float32, 'coordinates'), _p(Z, torch.float32, 'charges'),
                                      _p(atom_counts, torch.int32, 'atom_counts'), nb, A, ctypes.byref(pc), _p(cell),
                                      _p(inv_cell), _p(elements.contiguous(), torch.float32, 'elements'), nel,
                                      _p(reductors.contiguous(), torch.float32, 'reductors'), _p(pca_packed), N, _p(packed),
                                      int(bool(fast_math)), upper, _p(ws), ws.numel(), _p(energy), _p(grad_X),
                                      _stream(X.device)), 'qmlb_rff_predict_packed')
    return energy, grad_X


def pca_project_packed(inp, reductors, grouping, transpose=False, out=None):
    """:func:`pca_project` through ``qmlb_pca_pack`` + ``qmlb_pca_project_packed`` (pre-split B operand, bulk copies)."""
    nel, repsize, npcas = reductors.shape
    lib = _lib.load()
    nbytes = lib.qmlb_pca_pack_bytes(nel, repsize, npcas, int(bool(transpose)))
    packed = torch.empty(nbytes, dtype=torch.uint8, device=inp.device)
    check(lib.qmlb_pca_pack(_p(reductors.contiguous(), torch.float32, 'reductors'), nel, repsize, npcas, int(bool(transpose)),
                            _p(packed), nbytes, _stream(inp.device)), 'qmlb_pca_pack')
    rows = grouping.rows_cap
    if out is None:
        out = torch.empty(rows, repsize if transpose else npcas, dtype=torch.float32, device=inp.device)
    check(lib.qmlb_pca_project_packed(_p(inp, torch.float32, 'in'), _p(packed), _p(grouping.group_start), nel, rows, repsize, npcas,
                                      int(bool(transpose)), _p(out), _stream(inp.device)), 'qmlb_pca_project_packed')
    return out


def pca_project_jacobian(jac_rows, reductors, grouping):
    """``[rows, A, 3, repsize] -> [rows, A, 3, npcas]`` on element-grouped rows."""
    nel, repsize, npcas = reductors.shape
    rows, A = jac_rows.shape[0], jac_rows.shape[1]
    out = torch.empty(rows, A, 3, npcas, dtype=torch.float32, device=jac_rows.device)
    check(_lib.load().qmlb_pca_project_jacobian(_p(jac_rows, torch.float32, 'jac_rows'), _p(reductors.contiguous(), torch.float32, 'reductors'),
                                                _p(grouping.group_start), nel, rows, 3 * A, repsize, npcas, _p(out),
                                                _stream(jac_rows.device)), 'qmlb_pca_project_jacobian')
    return out


def sorf_train_features(x, dx, Dmat, bias, grouping, atom_counts, nb, A, sigma):
    """Per-molecule features ``Z f64[nb,F]`` and force features ``G f64[nb,A,3,F]`` (``None`` without ``dx``)."""
    nel, T, S, N = Dmat.shape
    F = S * N
    dev = x.device
    Z = torch.empty(nb, F, dtype=torch.float64, device=dev)
    G = torch.empty(nb, A, 3, F, dtype=torch.float64, device=dev) if dx is not None else None
    sinc = torch.empty(grouping.rows_cap, F, dtype=torch.float32, device=dev)
    check(_lib.load().qmlb_sorf_train_features(_p(x, torch.float32, 'x'), _p(dx, torch.float32, 'dx'),
                                               _p(Dmat.contiguous(), torch.float32, 'Dmat'), _p(bias.contiguous(), torch.float32, 'bias'),
                                               _p(grouping.group_start), _p(grouping.slot_of_row), _p(grouping.row_of_slot),
                                               _p(atom_counts.contiguous(), torch.int32, 'atom_counts'), nel, nb, A,
                                               grouping.rows_cap, N, S, T, float(sigma), _p(Z), _p(G), _p(sinc), _stream(dev)),
          'qmlb_sorf_train_features')
    return Z, G


def normal_equations_accumulate(M, y, ZTZ, ZTy, library=False):
    """``ZTZ += M^T M`` (upper triangle) and ``ZTy += M^T y`` in float64; ``library=True`` takes the cuBLAS route that is
    kept for timing comparisons."""
    rows, F = M.shape
    lib = _lib.load()
    fn = lib.qmlb_normal_equations_accumulate_cublas if library else lib.qmlb_normal_equations_accumulate
    check(fn(_p(M.contiguous(), torch.float64, 'M'), rows, F,
                                                       _p(None if y is None else y.contiguous(), torch.float64, 'y'),
                                                       _p(ZTZ, torch.float64, 'ZTZ'), _p(ZTy, torch.float64, 'ZTy'),
                                                       _stream(M.device)), 'qmlb_normal_equations_accumulate')


def gemv_t(M, y, ZTy):
    """``ZTy += M^T y`` in float64 (``qmlb_gemv_t_f64``)."""
    rows, F = M.shape
    check(_lib.load().qmlb_gemv_t_f64(_p(M.contiguous(), torch.float64, 'M'), rows, F, _p(y.contiguous(), torch.float64, 'y'),
                                      _p(ZTy, torch.float64, 'ZTy'), _stream(M.device)), 'qmlb_gemv_t_f64')


def symmetrize_upper(ZTZ):
    check(_lib.load().qmlb_symmetrize_upper(_p(ZTZ, torch.float64, 'ZTZ'), ZTZ.shape[0], _stream(ZTZ.device)), 'qmlb_symmetrize_upper')


def hadamard_features_accumulate(coeffs, bias, ordering, features):
    """``features f64[nmol,F] += sqrt(2/F) cos(coeffs + bias)`` per row, row ``a`` going to molecule ``ordering[a]``."""
    n, F = coeffs.shape
    check(_lib.load().qmlb_hadamard_features_accumulate(_p(coeffs.contiguous(), torch.float32, 'sorf_matrix'),
                                                        _p(bias.contiguous(), torch.float32, 'bias'),
                                                        _p(ordering.contiguous(), torch.int32, 'ordering'), n, F,
                                                        _p(features, torch.float64, 'features'), _stream(coeffs.device)),
          'qmlb_hadamard_features_accumulate')


def partial_feature_derivatives(coeffs, bias, out):
    """``out f64[n,F] = sqrt(2/F) sin(coeffs + bias)``."""
    n, F = coeffs.shape
    check(_lib.load().qmlb_partial_feature_derivatives(_p(coeffs.contiguous(), torch.float32, 'sorf_matrix'),
                                                       _p(bias.contiguous(), torch.float32, 'bias'), n, F,
                                                       _p(out, torch.float64, 'sin_coeffs'), _stream(coeffs.device)),
          'qmlb_partial_feature_derivatives')


def featurization_derivative_accumulate(partial, normalisation, D, input_derivatives, ordering, feature_derivatives):
    """``feature_derivatives f64[nmol,A,3,F] += normalisation * partial * (HD)^T input_derivatives`` (see the header)."""
    T, S, N = D.shape
    n, A = input_derivatives.shape[0], input_derivatives.shape[1]
    check(_lib.load().qmlb_featurization_derivative_accumulate(
        _p(partial.contiguous(), torch.float64, 'partial_feature_derivatives'), float(normalisation),
        _p(D.contiguous(), torch.float32, 'scaling'), _p(input_derivatives.contiguous(), torch.float32, 'input_derivatives'),
        _p(ordering.contiguous(), torch.int32, 'ordering'), n, A, N, S, T,
        _p(feature_derivatives, torch.float64, 'feature_derivatives'), _stream(partial.device)),
        'qmlb_featurization_derivative_accumulate')


def matmul_and_reduce(A, B, C):
    """``C f64[M,N] += A[M,K] @ B[K,N]`` in place (upstream ``utils_gpu.matmul_and_reduce``): the operands are taken at
    float32 precision, as upstream passes them, promoted, and multiplied by ``qmlb_gemm_tn_f64``."""
    if not (A.is_cuda and B.is_cuda and C.is_cuda):
        raise RuntimeError("matmul_and_reduce: tensors must be CUDA tensors")
    if C.dtype != torch.float64 or not C.is_contiguous():
        raise RuntimeError("matmul_and_reduce: C must be a contiguous float64 tensor")
    M, K = A.shape
    K2, N = B.shape
    if K2 != K or tuple(C.shape) != (M, N):
        raise RuntimeError("matmul_and_reduce: shape mismatch")
    P = A.float().T.contiguous().double()          # [K, M]; no copy of the float32 data when A is a transposed view
    Q = P if (B.data_ptr() == A.data_ptr() and B.shape == P.shape and B.is_contiguous() and A.stride() == (1, M)) \
        else B.float().contiguous().double()
    check(_lib.load().qmlb_gemm_tn_f64(_p(P, torch.float64, 'A'), _p(Q, torch.float64, 'B'), K, M, N, _p(C), _stream(C.device)),
          'qmlb_gemm_tn_f64')


def pack_upper(ZTZ):
    """Accumulated upper triangle of ``ZTZ f64[F,F]`` as a contiguous ``f64[F(F+1)/2]`` tensor."""
    F = ZTZ.shape[0]
    lib = _lib.load()
    packed = torch.empty(lib.qmlb_packed_upper_elements(F), dtype=torch.float64, device=ZTZ.device)
    check(lib.qmlb_pack_upper(_p(ZTZ, torch.float64, 'ZTZ'), F, _p(packed), _stream(ZTZ.device)), 'qmlb_pack_upper')
    return packed


def unpack_upper(packed, ZTZ):
    """Inverse of :func:`pack_upper`; also mirrors the triangle, so ``ZTZ`` is symmetric afterwards."""
    F = ZTZ.shape[0]
    check(_lib.load().qmlb_unpack_upper(_p(packed, torch.float64, 'packed'), F, _p(ZTZ, torch.float64, 'ZTZ'),
                                        _stream(ZTZ.device)), 'qmlb_unpack_upper')
    return ZTZ


def rff_train_features(x, dx, W, b, grouping, atom_counts, nb, A):
    """RFF per-molecule features ``Z f64[nb,D]`` and force features ``G f64[nb,A,3,D]`` (``None`` without ``dx``)."""
    nel, K, D = W.shape
    dev = x.device
    Z = torch.empty(nb, D, dtype=torch.float64, device=dev)
    G = torch.empty(nb, A, 3, D, dtype=torch.float64, device=dev) if dx is not None else None
    check(_lib.load().qmlb_rff_train_features(_p(x, torch.float32, 'x'), _p(dx, torch.float32, 'dx'), _p(W.contiguous(), torch.float32, 'W'),
                                              _p(b.contiguous(), torch.float32, 'b'), _p(grouping.group_start),
                                              _p(grouping.slot_of_row), _p(grouping.row_of_slot),
                                              _p(atom_counts.contiguous(), torch.int32, 'atom_counts'), nel, nb, A,
                                              grouping.rows_cap, K, D, _p(Z), _p(G), _stream(dev)),
          'qmlb_rff_train_features')
    return Z, G


def _on_tensor_device(fn):
    """Run ``fn`` with the device of its first CUDA tensor argument current: kernel launches, per-device caches
    inside the library (cuBLAS handle, built-in scratch address) and ``cudaFuncSetAttribute`` all act on the current
    device, which need not be the one the caller's tensors live on."""
    def on_device(*args, **kwargs):
        for a in list(args) + list(kwargs.values()):
            t = a.row_of_slot if isinstance(a, Grouping) else (a.species if isinstance(a, FchlKernelParams) else a)
            if isinstance(t, torch.Tensor) and t.is_cuda:
                if t.device.index == torch.cuda.current_device():
                    break
                with torch.cuda.device(t.device):
                    return fn(*args, **kwargs)
        return fn(*args, **kwargs)

    @functools.wraps(fn)
    def wrapped(*args, **kwargs):
        if not NVTX_RANGES:
            return on_device(*args, **kwargs)
        torch.cuda.nvtx.range_push('qmlb200.' + fn.__name__)   # one named range per stage on a profiler's timeline
        try:
            return on_device(*args, **kwargs)
        finally:
            torch.cuda.nvtx.range_pop()
    return wrapped


# Set QMLB200_NVTX=1 (before import) or this flag to wrap every stage of this module in an NVTX range named after it.
NVTX_RANGES = os.environ.get('QMLB200_NVTX', '0') not in ('', '0')


for _name, _fn in list(globals().items()):
    if callable(_fn) and getattr(_fn, '__module__', None) == __name__ and not _name.startswith('_') \
            and not isinstance(_fn, type) and _name not in ('tc_timeouts',):
        globals()[_name] = _on_tensor_device(_fn)
del _name, _fn
