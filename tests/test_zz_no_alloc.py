"""The allocation-free grouping entry point against the regular one.

``qmlb_group_by_element_noalloc`` exists for callers that get every buffer from their host application and are not
allowed to allocate device memory themselves (for instance a force plug-in inside a simulation engine that owns
the memory budget).  It keeps its scratch counters in a fixed array inside the library, which every call shares and
which still holds the previous call's values; the test therefore calls it twice in a row, on different batches,
and requires bit-identical permutations to the entry point that uses caller-owned scratch.  The file name sorts
last so that a run stopping at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

from tests import helpers as H

pytestmark = pytest.mark.gpu
DEV = 'cuda:0'


def _noalloc(Z, counts, elements):
    from qml_lightning_b200 import _lib, cabi
    lib = _lib.load()
    nb, A = Z.shape
    nel = elements.numel()
    rows_cap = lib.qmlb_rows_capacity(nb * A, nel)
    # outputs are caller-owned, as for a caller that cannot allocate: created before the call, only passed in
    row_of_slot = torch.empty(nb * A, dtype=torch.int32, device=DEV)
    slot_of_row = torch.empty(rows_cap, dtype=torch.int32, device=DEV)
    group_start = torch.empty(nel + 1, dtype=torch.int32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = lib.qmlb_group_by_element_noalloc(Z.data_ptr(), counts.data_ptr(), elements.data_ptr(), nel, nb, A,
                                           row_of_slot.data_ptr(), slot_of_row.data_ptr(), group_start.data_ptr(),
                                           rows_cap, stream)
    return rc, row_of_slot, slot_of_row, group_start


def test_noalloc_grouping_matches_regular_entry_point_twice_in_a_row():
    from qml_lightning_b200 import cabi
    # more than 1,024 molecules each: smaller batches are grouped by a single-block kernel that needs no scratch at all
    batches = [H.batch_mixed(1500, seed=21), H.batch_c0(2100, seed=22)]   # second call sees the first call's leftovers
    for X, Z, c, species in batches:
        Zd, cd = Z.to(DEV).contiguous(), c.to(DEV).contiguous()
        el = torch.tensor(species, dtype=torch.float32, device=DEV)
        ref = cabi.group_by_element(Zd, cd, el)
        rc, ros, sor, gs = _noalloc(Zd, cd, el)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.equal(ros, ref.row_of_slot)      # integer index work: bit-exact
        assert torch.equal(sor, ref.slot_of_row)
        assert torch.equal(gs, ref.group_start)


def test_noalloc_grouping_rejects_batches_beyond_the_built_in_scratch():
    from qml_lightning_b200 import _lib
    lib = _lib.load()
    nel = 4
    nb = 32 * (1 << 20) // (4 * nel) + 64          # one block of 32 molecules more than 1 MiB of counters holds
    assert lib.qmlb_group_scratch_bytes(nb, nel) > (1 << 20)
    # sizes are validated before any pointer is touched, so dummy (non-null) device pointers are enough
    dummy = torch.zeros(8, dtype=torch.int32, device=DEV)
    rc = lib.qmlb_group_by_element_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), nel, nb, 1,
                                           dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 64, None)
    assert rc == 1                                   # QMLB_ERR_INVALID
    assert b'scratch' in lib.qmlb_last_error()
