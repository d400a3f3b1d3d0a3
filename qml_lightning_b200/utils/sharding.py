"""Molecule sharding for multi-GPU prediction and training (one process per GPU, no data-path collective)."""
import numpy as np


def shard_bounds(atom_counts, world_size):
    """Contiguous molecule ranges ``[(start, stop), ...]``, one per rank, balanced by atom count.

    The cost of the path is proportional to the number of atoms (one SORF transform chain per atom), so the cut
    points sit where the prefix sum of ``atom_counts`` crosses multiples of total/world_size.  Every molecule belongs
    to exactly one rank; ranks may be empty only if there are fewer molecules than ranks.
    """
    counts = np.asarray(atom_counts, dtype=np.int64)
    n = len(counts)
    prefix = np.concatenate(([0], np.cumsum(counts)))
    total = prefix[-1]
    cuts = [0]
    for r in range(1, world_size):
        target = total * r / world_size
        idx = int(np.searchsorted(prefix, target, side='left'))
        cuts.append(min(max(idx, cuts[-1]), n))
    cuts.append(n)
    return [(cuts[r], cuts[r + 1]) for r in range(world_size)]


def my_shard(atom_counts, rank, world_size):
    return shard_bounds(atom_counts, world_size)[rank]
