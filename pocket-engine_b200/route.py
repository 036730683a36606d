"""Adapter-affine data partitioning over GPUs (no counterpart in pocket-engine, which is single-GPU): every GPU
has its own registry holding only its adapters, a router sends each sequence to its adapter's GPU, and base-only
sequences fill whichever GPU has the least work. No collective on the data path: a token's adapter work depends
only on its own adapter's slabs."""
import numpy as np


def assign_adapters(n_adapters, world, load=None):
    """GPU of every adapter (index 0 .. n_adapters - 1). Without ``load``: adapter i on GPU i mod world. With
    ``load`` (expected tokens per adapter, e.g. a popularity estimate): heaviest first onto the least loaded
    GPU, ties to the lowest rank, so that a skewed popularity does not pile onto one GPU."""
    if load is None:
        return np.arange(n_adapters, dtype=np.int32) % world
    load = np.asarray(load, dtype=np.float64)
    owner = np.zeros(n_adapters, np.int32)
    total = np.zeros(world)
    for i in np.argsort(-load, kind="stable"):
        g = int(np.argmin(total))
        owner[i] = g
        total[g] += load[i]
    return owner


def split_batch(row_n, row_adapter, owner, world):
    """Routes a step's sequences. ``row_adapter[i]`` is the adapter index of sequence i, or -1 for base only.
    Returns per rank the indices of its sequences, in step order: adapter-bearing sequences on their adapter's
    GPU, base-only sequences (longest first) on the GPU with the fewest tokens so far."""
    row_n = np.asarray(row_n, dtype=np.int64)
    row_adapter = np.asarray(row_adapter, dtype=np.int64)
    parts = [[] for _ in range(world)]
    tokens = np.zeros(world, np.int64)
    for i in np.nonzero(row_adapter >= 0)[0]:
        g = int(owner[row_adapter[i]])
        parts[g].append(int(i))
        tokens[g] += row_n[i]
    base = np.nonzero(row_adapter < 0)[0]
    for i in base[np.argsort(-row_n[base], kind="stable")]:
        g = int(np.argmin(tokens))
        parts[g].append(int(i))
        tokens[g] += row_n[i]
    return [np.array(sorted(p), dtype=np.int64) for p in parts]


def local_slots(row_adapter, owner, rank):
    """The rank's GPU slot (1-based, 0 = none) of every adapter it owns, in adapter order, and a function from
    a sequence's adapter index to that slot."""
    mine = [int(a) for a in np.nonzero(np.asarray(owner) == rank)[0]]
    slot_of = {a: k + 1 for k, a in enumerate(mine)}
    return mine, lambda a: 0 if a < 0 else slot_of[int(a)]
