"""Token-balanced partition of a jagged batch over ranks (no collective on the data path).

Sequences are independent units of the attention and of every per-token stage, so a batch is
split at sequence granularity: each rank gets a subset of the sequences with its own re-based
``seq_offsets`` and ``num_targets``.  The reference spawns one process per GPU the same way
(main.py:69-74) and has no sequence- or context-parallel path.
"""

from typing import List, Sequence

import torch


def partition_by_tokens(lengths: Sequence[int], world_size: int, cost_quadratic: float = 0.0) -> List[List[int]]:
    """Greedy longest-first assignment of sequence indices to ``world_size`` bins.

    ``cost = L + cost_quadratic * L^2``: 0 balances tokens (the partition named for the multi-GPU
    configuration), a positive value balances attention FLOPs as well.  Deterministic; indices
    inside a bin keep ascending order.
    """
    lengths = [int(x) for x in lengths]
    order = sorted(range(len(lengths)), key=lambda i: (-lengths[i], i))
    load = [0.0] * world_size
    bins: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (load[j], j))
        bins[r].append(i)
        load[r] += lengths[i] + cost_quadratic * lengths[i] * lengths[i]
    return [sorted(b) for b in bins]


def shard_jagged(values: torch.Tensor, seq_offsets: torch.Tensor, indices: Sequence[int]):
    """Rows of ``values`` that belong to the sequences ``indices`` + their re-based offsets."""
    offs = seq_offsets.to(torch.int64).cpu()
    idx = torch.as_tensor(list(indices), dtype=torch.int64)
    lens = (offs[1:] - offs[:-1])[idx]
    new_offs = torch.cat([torch.zeros(1, dtype=torch.int64), torch.cumsum(lens, 0)])
    rows = torch.cat([torch.arange(int(offs[i]), int(offs[i + 1])) for i in idx.tolist()]) if len(idx) else \
        torch.zeros(0, dtype=torch.int64)
    return values[rows.to(values.device)], new_offs


def unshard_jagged(parts: Sequence[torch.Tensor], seq_offsets: torch.Tensor, bins: Sequence[Sequence[int]]):
    """Inverse of :func:`shard_jagged` over all ranks: rebuilds the full jagged tensor."""
    offs = seq_offsets.to(torch.int64).cpu()
    total = int(offs[-1])
    out = parts[0].new_zeros((total,) + tuple(parts[0].shape[1:]))
    for part, idxs in zip(parts, bins):
        pos = 0
        for i in idxs:
            n = int(offs[i + 1] - offs[i])
            out[int(offs[i]):int(offs[i + 1])] = part[pos:pos + n]
            pos += n
    return out
