"""CPU oracle for the FCHL19 -> PCA -> SORF/RFF -> energy/force path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; it is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` as the checker and
the timed CPU baseline, never as a compute path of the product.

The upstream project has no CPU implementation of this path (its kernels are
CUDA only), so the oracle is a restatement of the kernel arithmetic in torch
(CPU tensors, float64 by default).  Each function cites the upstream file and
line range whose arithmetic it restates.

Parity pin: ``tests/test_oracle_kat.py`` feeds the oracle with the tensors of
the upstream TorchScript fixture ``unit_tests/models/saved_models/model_sorf.pt``
and the geometry / expected energy / expected forces parsed from
``unit_tests/models/unit_test_sorf.py`` (both committed under
``tests/golden/upstream/``) and applies that script's own ``np.isclose``
criteria.  The RFF and training (Z^T Z) restatements have no
upstream fixture: their parity is unpinned by upstream tests and rests on the
shared FCHL19/PCA front end plus self-consistency checks.
"""

from .qml_oracle import (  # noqa: F401
    FCHLParams,
    fchl19_representation,
    minimum_image,
    neighbour_lists,
    kahan_gram,
    fwht,
    sorf_coefficients,
    sorf_energy,
    rff_energy,
    energy_and_forces,
    training_rows,
)
